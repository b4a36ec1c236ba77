"""The Norevik decoder without a GPU: configuration, plan, tensor names, cache requests, and the
plain implementation's mechanisms against values worked out by hand."""
import copy
import math

import pytest
import torch

import helpers
import plain_norevik as P
from llama_rs_metal_b200.config.norevik import NorevikConfig
from llama_rs_metal_b200.engine.model import DecoderModel
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError
from llama_rs_metal_b200.parts.base import CompositeRequest, KeyValueRequest, StateRequest
from llama_rs_metal_b200.registry import find_architecture
from llama_rs_metal_b200.runtime import Runtime

F64 = torch.float64


def build(name):
    root = helpers.NOREVIK[name]["config"]
    arch = find_architecture(root)
    config = arch.config_class.from_dict(root)
    return config, arch.plan(config)


def cpu_model(plan):
    return DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32))


@pytest.mark.parametrize("name", sorted(helpers.NOREVIK))
def test_configuration_reads_every_size_and_writes_it_back(name):
    config, _ = build(name)
    again = NorevikConfig.from_dict(config.to_dict())
    assert again == config
    assert len(config.layers) == len(helpers.NOREVIK[name]["config"]["layers"])


def test_absent_options_are_off():
    config, plan = build("N3")
    assert config.embedding_scale == 1.0 and plan.embedding_scale is None
    mlp = config.layers[2].mlp
    assert (mlp.identity, mlp.groups, mlp.shared_ff) == (0, None, 24)
    assert config.layers[0].mlp is None and plan.layers[0].block == "post_norm_mixer"
    config1, plan1 = build("N1")
    assert config1.layers[2].mlp.shared_ff is None and plan1.layers[2].parts["feed_forward"].params["shared"] is None
    assert plan1.layers[1].parts["feed_forward"].params["groups"] == (3, 2)


def test_configuration_names_what_is_missing_or_not_built():
    root = helpers.NOREVIK["N1"]["config"]

    def changed(path, value):
        out = copy.deepcopy(root)
        at = out
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        return out
    with pytest.raises(InvalidError, match="width"):
        NorevikConfig.from_dict(changed(["width"], None))
    with pytest.raises(InvalidError, match="state"):
        NorevikConfig.from_dict(changed(["layers", 0, "mixer", "state"], None))
    with pytest.raises(UnsupportedError, match="type"):
        NorevikConfig.from_dict(changed(["layers", 1, "type"], "convolution"))
    with pytest.raises(UnsupportedError, match="kind"):
        NorevikConfig.from_dict(changed(["layers", 0, "mlp", "kind"], "gated"))
    with pytest.raises(InvalidError, match="groups"):
        NorevikConfig.from_dict(changed(["layers", 0, "mixer", "groups"], 3))           # 4 heads in 3 groups
    with pytest.raises(InvalidError, match="norm_groups"):
        NorevikConfig.from_dict(changed(["layers", 0, "mixer", "norm_groups"], 5))      # 48 channels in 5 parts
    with pytest.raises(InvalidError, match="rot"):
        NorevikConfig.from_dict(changed(["layers", 1, "mixer", "rot", "dims"], 4))      # not the rotated part's size
    with pytest.raises(InvalidError, match="gate_cap"):
        NorevikConfig.from_dict(changed(["layers", 2, "mixer", "gate_cap"], 0.0))
    with pytest.raises(InvalidError, match="groups"):
        NorevikConfig.from_dict(changed(["layers", 1, "mlp", "router", "groups", "count"], 4))   # 6 outputs in 4 groups
    with pytest.raises(InvalidError, match="top"):
        NorevikConfig.from_dict(changed(["layers", 1, "mlp", "router", "top"], 5))      # 2 kept groups hold 4


def test_cache_requests_follow_the_mixers():
    _, plan = build("N1")
    requests = cpu_model(plan).cache_requests()
    f32 = torch.float32
    # state-space: S [heads, state, vdim] and the last taps - 1 inputs of x | B | C
    assert requests[0] == CompositeRequest((StateRequest((4, 20, 12), f32), StateRequest((2, 4 * 12 + 2 * 2 * 20), f32)))
    # latent attention: one key head of kv_rank + rot_dim whose first kv_rank columns are the values
    assert requests[1] == KeyValueRequest(1, 26, None, 20, values_in_keys=True)
    # matrix memory: S with the normalizer as one more column (filled up to a multiple of four), and the maximum
    assert requests[2] == CompositeRequest((StateRequest((3, 8, 24), f32), StateRequest((3,), f32)))
    assert requests[3] == CompositeRequest((StateRequest((2, 8, 24), f32), StateRequest((0, 2 * 24 + 2 * 8), f32)))


def test_tensor_names_and_shapes_follow_the_configuration():
    _, plan = build("N1")
    shapes = {n: tuple(s.shape) for n, s in cpu_model(plan).tensor_specs().items()}
    assert shapes["embed"] == (211, 72) and shapes["head"] == (211, 72)
    assert shapes["final.norm"] == (72,) and shapes["final.norm.b"] == (72,)
    inner, channels = 4 * 12, 4 * 12 + 2 * 2 * 20
    assert shapes["l0.mix.in"] == (inner + channels + 4, 72) and shapes["l0.mix.conv"] == (channels, 3)
    assert shapes["l0.mix.conv.b"] == (channels,) and shapes["l0.mix.norm"] == (inner,) and shapes["l0.mix.o"] == (72, inner)
    assert shapes["l0.mix.dt_bias"] == shapes["l0.mix.A_log"] == shapes["l0.mix.D"] == (4,)
    assert shapes["l0.mlp.up"] == (56, 72) and shapes["l0.mlp.down"] == (72, 56) and "l0.mlp.gate" not in shapes
    assert shapes["l1.mix.q"] == (3 * 18, 72) and shapes["l1.mix.dkv"] == (26, 72) and shapes["l1.mix.dkv.norm"] == (20,)
    assert shapes["l1.mix.uk"] == (36, 20) and shapes["l1.mix.uv"] == (30, 20) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l1.mix.g"] == (30, 72) and shapes["l1.mix.o"] == (72, 30)
    assert shapes["l1.mlp.router"] == (6, 72) and shapes["l1.mlp.correction"] == (6,)       # 5 experts + 1 identity
    assert shapes["l1.mlp.e4.gate"] == (24, 72) and "l1.mlp.e5.gate" not in shapes
    assert shapes["l1.mlp.shared.down"] == (72, 40)
    assert shapes["l2.mix.q"] == shapes["l2.mix.k"] == (24, 72) and shapes["l2.mix.v"] == shapes["l2.mix.g"] == (60, 72)
    assert shapes["l2.mix.i"] == (3, 72) and shapes["l2.mix.f.b"] == (3,) and shapes["l2.mix.norm"] == (60,)
    assert "l2.mlp.shared.gate" not in shapes and "l3.mlp.up" not in shapes and "l3.norm2" not in shapes
    for i in range(5):
        assert shapes[f"l{i}.norm1"] == (72,) and shapes[f"l{i}.norm1.b"] == (72,)


def test_random_folder_is_read_back_by_the_plain_implementation(tmp_path):
    folder = helpers.make_norevik_dir(str(tmp_path / "n1"), "N1")
    config, tensors = P.read_model(folder)
    assert config["layers"][1]["mlp"]["router"]["groups"] == {"count": 3, "keep": 2}
    streams = []
    logits = P.forward(config, tensors, [1, 2, 3, 4, 5], streams)
    assert logits.shape == (5, 211) and torch.isfinite(logits).all() and len(streams) == 5


# --------------------------------------------------------------------------- the plain mechanisms by hand
def test_plain_layer_norm_takes_the_variance_of_the_deviations():
    x = torch.tensor([[1.0, 3.0, 5.0, 7.0]], dtype=F64)
    out = P.layer_norm(x, torch.tensor([1.0, 2.0, 1.0, 1.0], dtype=F64), torch.tensor([0.0, 0.0, 0.5, 0.0], dtype=F64), 1.0)
    under = math.sqrt(5.0 + 1.0)                         # mean 4, deviations -3 -1 1 3, variance 5
    assert torch.allclose(out, torch.tensor([[-3 / under, -2 / under, 1 / under + 0.5, 3 / under]], dtype=F64))


def test_plain_state_space_mixer_by_hand():
    """One head, state 1, value 1, one tap: S_t = exp(-e^A dt_t) S_(t-1) + dt_t B_t x_t, y = S C + D x."""
    m = dict(heads=1, vdim=1, state=1, groups=1, conv=1, norm_groups=1)
    # the projection's rows: z | x | B | C | dt, from a two-column input [u, 1]
    w = {"in": torch.tensor([[0.0, 2.0], [1.0, 0.0], [0.0, 1.5], [0.0, 0.5], [0.0, 0.3]], dtype=F64),
         "conv": torch.tensor([[1.0], [1.0], [1.0]], dtype=F64), "conv.b": torch.zeros(3, dtype=F64),
         "dt_bias": torch.tensor([0.2], dtype=F64), "A_log": torch.tensor([-0.5], dtype=F64),
         "D": torch.tensor([0.7], dtype=F64), "norm": torch.tensor([1.0], dtype=F64), "o": torch.tensor([[1.0]], dtype=F64)}
    u = [0.8, -1.2, 2.0]
    h = torch.tensor([[v, 1.0] for v in u], dtype=F64)
    out = P.mamba2(h, m, w, "", 1e-12)
    silu = lambda z: z / (1 + math.exp(-z))
    dt = math.log1p(math.exp(0.5))
    decay, B, C = math.exp(-math.exp(-0.5) * dt), silu(1.5), silu(0.5)
    S = 0.0
    for t, v in enumerate(u):
        x = silu(v)
        S = decay * S + dt * B * x
        y = (S * C + 0.7 * x) * silu(2.0)
        assert abs(float(out[t, 0]) - y / math.sqrt(y * y + 1e-12)) < 1e-9     # a part of one channel is its sign


def test_plain_convolution_starts_from_zeros_and_ends_on_the_current_token():
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=F64)
    out = P.causal_conv(x, torch.tensor([[0.5, 2.0, 3.0]], dtype=F64), torch.tensor([0.25], dtype=F64))
    assert out[:, 0].tolist() == [3.25, 32.25, 320.75]


def test_plain_rotation_pairs_neighbours():
    x = torch.tensor([[1.0, 0.0, 0.0, 2.0, 9.0]], dtype=F64)
    out = P.rotate_pairs(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 9.0]
    assert torch.allclose(out[0], torch.tensor(want, dtype=F64))


def test_plain_sink_counts_once_and_is_not_scaled():
    """A zero query makes every score 0: the weights are 1 / (t + 1 + e^sink) each, whatever the scale."""
    m = dict(heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1, scale=7.0, rot=dict(dims=2, base=10.0))
    w = {"q": torch.zeros(3, 2, dtype=F64), "dkv": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 1.0]], dtype=F64),
         "dkv.norm": torch.ones(1, dtype=F64), "uk": torch.ones(1, 1, dtype=F64), "uv": torch.tensor([[2.0]], dtype=F64),
         "sink": torch.tensor([math.log(3.0)], dtype=F64), "g": torch.zeros(1, 2, dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    h = torch.tensor([[1.0, 0.0], [-1.0, 0.0], [1.0, 0.0]], dtype=F64)
    out = P.latent_attention(h, m, w, "", 1e-12)
    # the latent of one number is its sign; values 2 c; the gate is sigmoid(0) = 1/2
    assert torch.allclose(out[:, 0], torch.tensor([2.0 / 4, 0.0 / 5, 2.0 / 6], dtype=F64) * 0.5, atol=1e-9)


def test_plain_matrix_memory_by_hand():
    """One head of one dimension: the maximum starts at 0, so a first input gate of -2 leaves it there."""
    m = dict(heads=1, dim=1, vdim=1, gate_cap=4.0)
    one = torch.ones(1, 1, dtype=F64)
    w = {"q": one, "k": one * 0.5, "v": one * 2.0, "g": one * 0.0, "i": one * 0.0, "f": one * 0.0,
         "i.b": torch.tensor([-2.0], dtype=F64), "f.b": torch.tensor([1.0], dtype=F64), "norm": torch.ones(1, dtype=F64), "o": one}
    h = torch.tensor([[1.0], [3.0]], dtype=F64)
    i = 4.0 * math.tanh(-2.0 / 4.0)
    f = -math.log1p(math.exp(-4.0 * math.tanh(1.0 / 4.0)))
    top0 = max(f + 0.0, i)
    assert top0 == f and f < 0                                      # the forget gate rules: m_0 = f, not i
    S0 = math.exp(i - top0) * 0.5 * 2.0
    n0 = math.exp(i - top0) * 0.5
    o0 = S0 * 1.0 / (max(abs(n0 * 1.0), math.exp(-top0)) + 1e-6)
    top1 = max(f + top0, i)
    S1 = math.exp(f + top0 - top1) * S0 + math.exp(i - top1) * 1.5 * 6.0
    n1 = math.exp(f + top0 - top1) * n0 + math.exp(i - top1) * 1.5
    o1 = S1 * 3.0 / (max(abs(n1 * 3.0), math.exp(-top1)) + 1e-6)
    out = P.mlstm(h, m, w, "", 0.5)
    for t, o in enumerate((o0, o1)):
        assert abs(float(out[t, 0]) - o / math.sqrt(o * o + 0.5) * 0.5) < 1e-9


def test_plain_routing_by_hand():
    """Six outputs in three groups of neighbours, two kept, three chosen: the corrections decide the
    choice, the plain scores are the weights, an expert outside the kept groups is never chosen
    although its (negative) choice score is the largest but one."""
    f = dict(router=dict(experts=5, identity=1, top=3, groups=dict(count=3, keep=2)))
    z = torch.log(torch.tensor([[0.05, 0.10, 0.30, 0.05, 0.20, 0.30]], dtype=F64))
    w = {"router": torch.eye(6, dtype=F64), "correction": torch.tensor([-1.0, -1.0, -2.0, -1.2, -1.05, -1.3], dtype=F64)}
    chosen, weights, scores = P.route(z, f, w, "")
    assert torch.allclose(scores[0], torch.tensor([0.05, 0.10, 0.30, 0.05, 0.20, 0.30], dtype=F64))
    # choice scores -0.95 -0.90 | -1.70 -1.15 | -0.85 -1.00: the groups score -0.90, -1.15, -0.85
    assert sorted(chosen[0].tolist()) == [0, 1, 4]
    assert torch.allclose(weights[0].sort().values, torch.tensor([0.05, 0.10, 0.20], dtype=F64))
    # choice scores -0.95 -0.60 | 0.80 -2.00 | -0.70 -0.75: groups 1 and 0 are kept; the third best of all,
    # -0.70, lies in group 2 and is not chosen, the kept groups' -0.95 is
    w["correction"] = torch.tensor([-1.0, -0.70, 0.5, -2.05, -0.90, -1.05], dtype=F64)
    chosen, weights, _ = P.route(z, f, w, "")
    assert sorted(chosen[0].tolist()) == [0, 1, 2]
    assert torch.allclose(weights[0].sort().values, torch.tensor([0.05, 0.10, 0.30], dtype=F64))
    assert abs(float(weights.sum()) - 0.45) < 1e-12               # the weights are not renormalized


def test_plain_identity_expert_passes_its_input_on():
    f = dict(kind="moe", router=dict(experts=1, identity=1, top=1))
    w = {"router": torch.tensor([[0.0, 0.0], [0.0, 5.0]], dtype=F64), "correction": torch.zeros(2, dtype=F64),
         "e0.gate": torch.ones(1, 2, dtype=F64), "e0.up": torch.ones(1, 2, dtype=F64), "e0.down": torch.ones(2, 1, dtype=F64)}
    h = torch.tensor([[1.0, 2.0]], dtype=F64)
    out = P.experts(h, f, w, "")
    share = 1 / (1 + math.exp(-10.0))
    assert torch.allclose(out, share * h)


def test_plain_dense_feed_forward_squares_the_positive_part():
    w = {"up": torch.tensor([[1.0], [-1.0]], dtype=F64), "down": torch.tensor([[1.0, 10.0]], dtype=F64)}
    out = P.dense(torch.tensor([[3.0], [-2.0]], dtype=F64), None, w, "")
    assert out[:, 0].tolist() == [9.0, 40.0]

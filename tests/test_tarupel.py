"""The Tarupel decoder without a GPU: configuration, plan, tensor names, cache requests, and the
plain implementation's mechanisms against values worked out by hand."""
import copy
import math

import pytest
import torch

import helpers
import plain_tarupel as P
from llama_rs_metal_b200.config.tarupel import TarupelConfig
from llama_rs_metal_b200.engine.model import DecoderModel
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError
from llama_rs_metal_b200.parts.base import CompositeRequest, KeyValueRequest, StateRequest
from llama_rs_metal_b200.registry import find_architecture
from llama_rs_metal_b200.runtime import Runtime

F64 = torch.float64


def build(name):
    root = helpers.TARUPEL[name]["config"]
    arch = find_architecture(root)
    config = arch.config_class.from_dict(root)
    return config, arch.plan(config)


def cpu_model(plan):
    return DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32))


# --------------------------------------------------------------------------- configuration and plan
@pytest.mark.parametrize("name", sorted(helpers.TARUPEL))
def test_configuration_reads_every_size_and_writes_it_back(name):
    config, _ = build(name)
    assert TarupelConfig.from_dict(config.to_dict()) == config
    assert len(config.layers) == len(helpers.TARUPEL[name]["config"]["layers"])


def test_absent_options_are_off():
    config, plan = build("T3")
    assert (config.embedding_scale, config.residual_mult, config.loops) == (1.0, 1.0, False)
    assert plan.embedding_scale is None and plan.stream_offsets is None
    assert all(e.add_offset is None and not e.add_embedding for e in plan.schedule)
    mlp = config.layers[2].mlp
    assert (mlp.scale, mlp.groups, mlp.shared_ff) == (1.0, None, 24)
    assert config.layers[0].mlp is None and plan.layers[0].block == "scaled_pre_norm_mixer"
    root = copy.deepcopy(helpers.TARUPEL["T3"]["config"])
    del root["layers"][1]["mixer"]["mask"], root["layers"][1]["mixer"]["rot"]
    bare = find_architecture(root).plan(TarupelConfig.from_dict(root)).layers[1].parts["mixer"].params
    assert bare["window"] is None and bare["position"] is None


def test_configuration_names_what_is_missing_or_not_built():
    root = helpers.TARUPEL["T1"]["config"]

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
    for path, value, word in [(("width",), None, "width"), (("layers", 0, "mixer", "kv_heads"), None, "kv_heads"),
                              (("layers", 2, "mixer", "conv"), None, "conv"), (("layers", 1, "mixer", "dim"), 0, "dim"),
                              (("layers", 2, "mixer", "heads"), 3, "multiple"), (("layers", 1, "mlp", "router", "top"), 5, "top"),
                              (("layers", 0, "mixer", "rot", "dims"), 14, "rot"), (("loop", "stop"), 9, "loop"),
                              (("norm", "eps"), None, "eps")]:
        with pytest.raises(InvalidError, match=word):
            TarupelConfig.from_dict(changed(path, value))
    with pytest.raises(UnsupportedError, match="type"):
        TarupelConfig.from_dict(changed(("layers", 0, "type"), "attention_3"))
    with pytest.raises(UnsupportedError, match="kind"):
        TarupelConfig.from_dict(changed(("layers", 0, "mlp", "kind"), "sparse"))


def test_the_looped_run_repeats_with_cache_entries_of_its_own():
    config, plan = build("T1")       # five layers, layers 1 and 2 three times
    runs = [(e.layer, e.cache, e.add_offset, e.add_embedding) for e in plan.schedule]
    assert runs == [(0, 0, None, False), (1, 1, 0, False), (2, 2, None, False), (1, 3, 1, True), (2, 4, None, False),
                    (1, 5, 2, True), (2, 6, None, False), (3, 7, None, False), (4, 8, None, False)]
    assert plan.stream_offsets == ("loop.step", 3)
    assert P.layer_runs(helpers.TARUPEL["T1"]["config"]) == [(e.layer, e.add_offset) for e in plan.schedule]
    _, plan2 = build("T2")           # the loop starts at the first layer: the first pass adds no embedding
    assert [(e.layer, e.add_offset, e.add_embedding) for e in plan2.schedule][:3] == [(0, 0, False), (1, None, False), (0, 1, True)]


def test_tensor_names_and_shapes():
    config, plan = build("T1")
    specs = cpu_model(plan).tensor_specs()
    shapes = {name: spec.shape for name, spec in specs.items()}
    assert shapes["embed"] == (211, 72) and shapes["head"] == (211, 72) and shapes["loop.step"] == (3, 72)
    assert shapes["final.norm"] == () and shapes["l0.norm1"] == () and shapes["l0.norm2"] == ()
    assert shapes["l0.ls1"] == shapes["l0.ls2"] == shapes["l0.shift"] == (72,)
    assert "l2.ls2" not in shapes and "l2.norm2" not in shapes and shapes["l2.ls1"] == (72,)
    # attention_2: 3 heads of 12, 1 key head, values of 20, row norms
    assert shapes["l0.mix.q"] == (36, 72) and shapes["l0.mix.k"] == (12, 72) and shapes["l0.mix.v"] == (20, 72)
    assert shapes["l0.mix.q.b"] == (36,) and shapes["l0.mix.v.b"] == (20,) and shapes["l0.mix.o"] == (72, 60)
    assert shapes["l0.mix.q.norm"] == (36,) and shapes["l0.mix.k.norm"] == (12,) and "l0.mix.q.conv" not in shapes
    # attention: taps, no row norms
    assert shapes["l2.mix.q.conv"] == (96, 3) and shapes["l2.mix.k.conv"] == (48, 3) and shapes["l2.mix.v.conv"] == (20, 3)
    assert "l2.mix.q.norm" not in shapes
    # general delta
    for own, shape in dict(r=(60, 72), k=(60, 72), v=(60, 72), g=(60, 72), a=(60, 72), o=(72, 60), w1=(5, 72), w2=(60, 5)).items():
        assert shapes["l1.mix." + own] == shape, own
    assert shapes["l1.mix.a.b"] == shapes["l1.mix.w0"] == shapes["l1.mix.norm"] == (60,)
    # experts
    assert shapes["l1.mlp.router"] == (6, 72) and shapes["l1.mlp.e5.gate"] == (24, 72) and shapes["l1.mlp.e0.down"] == (72, 24)
    assert shapes["l1.mlp.shared.up"] == (40, 72) and shapes["l1.mlp.shared.sg"] == (1, 72)
    assert "l3.mlp.shared.sg" not in shapes and shapes["l0.mlp.gate"] == (56, 72)
    # without decay_rank in the configuration the rank is the checkpoint's
    root = copy.deepcopy(helpers.TARUPEL["T1"]["config"])
    del root["layers"][1]["mixer"]["decay_rank"]
    open_specs = cpu_model(find_architecture(root).plan(TarupelConfig.from_dict(root))).tensor_specs()
    assert open_specs["l1.mix.w1"].shape == (None, 72) and open_specs["l1.mix.w1"].fits((16, 72))


def test_cache_requests_keep_what_each_layer_needs():
    _, plan = build("T1")
    requests = cpu_model(plan).cache_requests()
    assert len(requests) == 9
    shift = StateRequest((1, 72), torch.float32)
    assert requests[0] == CompositeRequest((KeyValueRequest(1, 12, 7, 20), shift))            # a window of 7
    assert requests[1] == CompositeRequest((StateRequest((3, 20, 20), torch.float32), shift))
    taps = StateRequest((2, 4 * 24 + 2 * (24 + 10)), torch.float32)
    assert requests[2] == CompositeRequest((CompositeRequest((KeyValueRequest(2, 24, 70, 10), taps)), shift))  # a chunk of 70
    assert requests[3] == requests[1] and requests[4] == requests[2]                          # a pass's own entries
    assert requests[7] == CompositeRequest((KeyValueRequest(2, 10, 1, None), shift))          # one tap: no tail


# --------------------------------------------------------------------------- the plain mechanisms by hand
def test_norm_shift_and_convolution_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(P.scalar_norm(x, torch.tensor(2.0, dtype=F64), 0.0), torch.tensor([[6.0, 8.0]], dtype=F64) / math.sqrt(12.5))
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]], dtype=F64)
    mu = torch.tensor([0.5, 1.0], dtype=F64)
    assert torch.equal(P.token_shift(h, mu), torch.tensor([[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]], dtype=F64))
    u = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=F64)
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)     # the last tap is the current token's
    assert torch.equal(P.causal_conv(u, taps), torch.tensor([[1.0], [12.0], [123.0], [234.0]], dtype=F64))
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=F64))) - 0.8411919906082768) < 1e-12


def test_rotations_pair_the_right_dimensions():
    x = torch.zeros(2, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0          # the first dimension of the first pair in both layouts
    x[:, 0, 5] = 7.0          # outside the rotated part
    halves = P.rotate_halves(x, torch.tensor([0, 3]), 4, 100.0)
    pairs = P.rotate_pairs(x, torch.tensor([0, 3]), 4, 100.0)
    assert torch.equal(halves[0], x[0]) and torch.equal(pairs[0], x[0])              # position 0 turns nothing
    c, s = math.cos(3.0), math.sin(3.0)                                              # pair 0 turns by position * 1
    assert torch.allclose(halves[1, 0], torch.tensor([c, 0.0, s, 0.0, 0.0, 7.0], dtype=F64))
    assert torch.allclose(pairs[1, 0], torch.tensor([c, s, 0.0, 0.0, 0.0, 7.0], dtype=F64))
    y = torch.zeros(1, 1, 4, dtype=F64)
    y[0, 0, 1] = 1.0          # pair 1 of the split layout is (1, 3), frequency 100^(-1/2)
    a = 5.0 * 0.1
    assert torch.allclose(P.rotate_halves(y, torch.tensor([5]), 4, 100.0)[0, 0],
                          torch.tensor([0.0, math.cos(a), 0.0, math.sin(a)], dtype=F64))


def test_chunks_and_windows_see_the_right_keys():
    T = 7
    q, k = torch.zeros(T, 1, 2, dtype=F64), torch.zeros(T, 1, 2, dtype=F64)      # all scores equal: plain averages
    v = torch.eye(T, dtype=F64).reshape(T, 1, T)
    chunked = P.softmax_attention(q, k, v, 1.0, lambda i, j: i // 3 == j // 3)
    window = P.softmax_attention(q, k, v, 1.0, lambda i, j: i - j < 3)
    assert torch.allclose(chunked[4], torch.tensor([0, 0, 0, 0.5, 0.5, 0, 0], dtype=F64))      # chunk 3..5, up to itself
    assert torch.allclose(chunked[3], torch.tensor([0, 0, 0, 1.0, 0, 0, 0], dtype=F64))        # a chunk's first token is alone
    assert torch.allclose(chunked[2], torch.tensor([1, 1, 1, 0, 0, 0, 0], dtype=F64) / 3)
    assert torch.allclose(window[4], torch.tensor([0, 0, 1, 1, 1, 0, 0], dtype=F64) / 3)       # itself and two before
    assert torch.allclose(window[1], torch.tensor([0.5, 0.5, 0, 0, 0, 0, 0], dtype=F64))


def test_generalized_delta_rule_with_one_channel_is_a_scalar_recurrence():
    """One head of one channel: the unit key is +-1 (up to the epsilon), so S_t = (g - a) S + k v with
    g = exp(-e^-1/2 sigmoid(.)) and a = sigmoid(.), both terms from the old S, and o = S r."""
    width, T = 3, 6
    gen = torch.Generator().manual_seed(4)
    w = {n: torch.randn(1, width, generator=gen, dtype=F64) for n in ("m.r", "m.k", "m.v", "m.g", "m.a", "m.w1", "m.o")}
    w["m.o"] = torch.randn(width, 1, generator=gen, dtype=F64)
    w.update({"m.w2": torch.tensor([[0.7]], dtype=F64), "m.w0": torch.tensor([0.3], dtype=F64),
              "m.a.b": torch.tensor([-0.2], dtype=F64), "m.norm": torch.tensor([1.5], dtype=F64)})
    h = torch.randn(T, width, generator=gen, dtype=F64)
    got = P.general_delta(h, dict(heads=1, dim=1), w, "m.", 1e-5)
    S, want = 0.0, []
    for t in range(T):
        r, k, v, gate, a_in, low = (float(h[t] @ w["m." + n][0]) for n in ("r", "k", "v", "g", "a", "w1"))
        g = math.exp(-math.exp(-0.5) / (1.0 + math.exp(-(0.7 * math.tanh(low) + 0.3))))
        a = 1.0 / (1.0 + math.exp(-(a_in - 0.2)))
        u2 = k * k / (k * k + 1e-6)
        S = g * S - a * u2 * S + k * v
        o = S * r
        o = o / math.sqrt(o * o + 1e-5) * 1.5 / (1.0 + math.exp(-gate))
        want.append(o * w["m.o"][:, 0])
    assert torch.allclose(got, torch.stack(want), rtol=1e-10, atol=1e-12)


def test_routing_inside_the_best_groups_with_scaled_weights():
    # six experts in three groups of neighbours, two groups kept; one token whose logits are given
    z = torch.tensor([[2.0, 0.0, 1.9, 1.8, 0.1, 1.95]], dtype=F64)
    s = torch.softmax(z, -1)[0]
    f = dict(router=dict(experts=6, top=3, scale=2.0, groups=dict(count=3, keep=2)))
    ids, weights = P.route(torch.ones(1, 1, dtype=F64), f, {"router": z.T}, "")    # input 1, router column = the logits
    # groups' best scores: {0,1}: s0, {2,3}: s2, {4,5}: s5 -> kept are the first and the last; expert 2 and 3 are out
    assert sorted(ids[0].tolist()) == [0, 4, 5]
    chosen = s[[0, 4, 5]]
    order = ids[0].sort().indices
    assert torch.allclose(weights[0][order], chosen / chosen.sum() * 2.0)
    # without groups the three best of all
    ids, weights = P.route(torch.ones(1, 1, dtype=F64), dict(router=dict(experts=6, top=3)), {"router": z.T}, "")
    assert sorted(ids[0].tolist()) == [0, 2, 5] and abs(float(weights.sum()) - 1.0) < 1e-12


def test_shared_expert_is_gated_per_token_and_experts_are_weighted():
    width, ff = 4, 3
    gen = torch.Generator().manual_seed(6)
    w = {}
    for e in ("e0.", "e1.", "shared."):
        w["p." + e + "gate"], w["p." + e + "up"] = torch.randn(ff, width, generator=gen, dtype=F64), torch.randn(ff, width, generator=gen, dtype=F64)
        w["p." + e + "down"] = torch.randn(width, ff, generator=gen, dtype=F64)
    w["p.router"] = torch.randn(2, width, generator=gen, dtype=F64)
    w["p.shared.sg"] = torch.randn(1, width, generator=gen, dtype=F64)
    h = torch.randn(5, width, generator=gen, dtype=F64)
    f = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=2, top=1, scale=3.0), shared=dict(ff=ff))
    got = P.feed_forward(h, f, w, "p.")
    for t in range(5):
        e = int((h[t] @ w["p.router"].T).argmax())
        one = P.gated(h[t:t + 1], w, f"p.e{e}.", P.silu)[0] * 3.0          # a single chosen score renormalizes to 1
        gate = 1.0 / (1.0 + math.exp(-float(h[t] @ w["p.shared.sg"][0])))
        assert torch.allclose(got[t], one + gate * P.gated(h[t:t + 1], w, "p.shared.", P.silu)[0])


def test_the_loop_adds_the_embedding_again_and_a_step_vector_each_pass():
    """A model whose sublayers add nothing (their factors are zero): the stream after each layer run is
    then the embedding, counted once more per pass, plus the step vectors so far."""
    spec = copy.deepcopy(helpers.TARUPEL["T2"])
    import tempfile

    def silence(tensors):
        for name, t in tensors.items():
            if name.endswith((".ls1", ".ls2")):
                t.zero_()
    folder = helpers.make_tarupel_dir(tempfile.mkdtemp(), spec, edit=silence)
    config, w = P.read_model(folder)
    tokens = [5, 9, 200]
    streams = []
    P.forward(config, w, tokens, streams)
    e = w["embed"][tokens] * 8.0
    assert torch.allclose(streams[0], e + w["loop.step"][0]) and torch.allclose(streams[1], streams[0])
    assert torch.allclose(streams[2], 2 * e + w["loop.step"][0] + w["loop.step"][1])
    assert torch.allclose(streams[-1], streams[2])

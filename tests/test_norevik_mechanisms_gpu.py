"""The Norevik decoder's mechanisms one at a time: models of a single layer whose weights are made so
that a fault shows, compared with the plain implementation (plain_norevik.py) as whole prompts, in
portions and in decoding; and the norm kernels against their definition."""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_norevik as P
from test_norevik_gpu import close, entry, open_runner, reference

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64
PAGE = 64  # rows of a cache page


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


def one_layer(kind, mixer, mlp=None, width=64, vocab=97, eps=1e-5, scale=2.0, seed=70, std=0.15):
    return dict(config=dict(architecture="Norevik", vocab=vocab, width=width, norm=dict(eps=eps),
                            embedding=dict(scale=scale), layers=[dict(type=kind, mixer=mixer, mlp=mlp)]),
                seed=seed, std=std)


SMALL_SSM = helpers._ssm(2, 8, 4, 1, 2, 1)   # a small mixer in front of a feed-forward that is the test's subject

ALONE = {
    "mamba2": one_layer("mamba2", helpers._ssm(6, 8, 12, 3, 4, 2)),
    "mamba2_one_tap": one_layer("mamba2", helpers._ssm(2, 40, 24, 2, 1, 5), width=88),
    "mamba2_wide_state": one_layer("mamba2", helpers._ssm(3, 12, 136, 1, 5, 3)),
    "latent": one_layer("latent_attention", helpers._sink_latent(5, 12, 6, 20, 24, 0.2, 1000.0), width=72),
    "latent_rot_only_two": one_layer("latent_attention", helpers._sink_latent(2, 64, 2, 8, 40, 0.1, 10.0)),
    "mlstm": one_layer("mlstm", helpers._memory(3, 12, 20, 5.0)),
    "mlstm_wide": one_layer("mlstm", helpers._memory(2, 72, 127, 20.0), width=136),
    "dense": one_layer("mamba2", SMALL_SSM, helpers._plain_ff(100)),
    "experts_plain": one_layer("mamba2", SMALL_SSM, helpers._experts(20, 7, 3)),
    "experts_one_of_two": one_layer("mamba2", SMALL_SSM, helpers._experts(36, 2, 1, identity=1, shared=20)),
    "experts_groups": one_layer("mamba2", SMALL_SSM, helpers._experts(24, 9, 4, identity=3, groups=(4, 2), shared=48)),
    "experts_many": one_layer("mamba2", SMALL_SSM, helpers._experts(16, 20, 5, identity=4, groups=(6, 3))),
    "experts_all_chosen": one_layer("mamba2", SMALL_SSM, helpers._experts(16, 3, 4, identity=1)),
}


@pytest.mark.parametrize("what", sorted(ALONE))
def test_each_mechanism_alone(engine, tmp_path, what):
    """A prompt of 300 tokens (more than the router's single-launch rows), then 12 tokens one by one;
    the residual stream behind the layer in float32, the logits in both types."""
    for dtype in ("float32", "bfloat16"):
        folder = helpers.make_norevik_dir(str(tmp_path / (what + dtype)), ALONE[what], steady_routing=dtype == "bfloat16")
        config, tensors = P.read_model(folder)
        tokens = helpers.random_tokens(3, 312, config["vocab"])
        streams = []
        ref = P.forward(config, tensors, tokens, streams).numpy()
        runner, cache, model = open_runner(engine, folder, dtype, use_graphs=False)
        seen = []
        block = model.blocks[0]
        inner = block.forward

        def wrapped(hidden, ctx, view):
            out = inner(hidden, ctx, view)
            seen.append(out.detach().clone().cpu().to(F64))
            return out
        block.forward = wrapped
        slot = cache.open_slot()
        rows = [runner.step([entry(slot, tokens[:300])]).cpu().numpy()]
        if dtype == "float32":
            err = float((seen[0][:300] - streams[0][:300]).abs().max() / streams[0].abs().max())
            assert err < 2e-5, f"{what}: the stream behind the layer is off by {err:.2e}"
        for t in tokens[300:]:
            rows.append(runner.step([entry(slot, [t])]).cpu().numpy())
        close(np.concatenate(rows), ref, dtype, what)
        runner.check_device_status()


# --------------------------------------------------------------------------- latent attention
def attention_weights(config, w, tokens, head):
    """The softmax weights [T, T + 1] of one head of layer 0 (the last column is the sink's share),
    from the design's equations, for the tests' own expectations."""
    m, p, eps = config["layers"][0]["mixer"], "l0.mix.", config["norm"]["eps"]
    d, r, rank, H = m["dim"], m["rot_dim"], m["kv_rank"], m["heads"]
    h = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    T = len(tokens)
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)[:, head]
    down = h @ w[p + "dkv"].T
    c = P.unit_rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).reshape(T, H, d)[:, head]
    shared = P.rotate_pairs(down[:, rank:], pos, r, m["rot"]["base"])
    q_rot = P.rotate_pairs(q[:, d:], pos, r, m["rot"]["base"])
    s = (q[:, :d] @ k.T + q_rot @ shared.T) * m["scale"]
    s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
    s = torch.cat([s, w[p + "sink"][head].expand(T, 1)], dim=1)
    return torch.softmax(s, dim=1)


@pytest.mark.parametrize("far_at", [2, PAGE - 1, PAGE])
def test_a_far_key_wins_and_a_sink_takes_its_share(engine, tmp_path, far_at):
    """Token A stands once, far back (among the first tokens, or on either side of a page's border);
    its unnormed rotated key part is made large, so that late queries give it most of head 0's
    weight: a kernel that loses it, rotates it by another angle or reads another page shows. Head
    1's sink is made large and takes most of that head's weight; head 0's is small."""
    spec = one_layer("latent_attention", helpers._sink_latent(2, 8, 8, 16, 12, 0.3, 100.0), seed=71)
    V, A = spec["config"]["vocab"], 5

    def edit(t):
        t["embed"][A] *= 60.0
        t["l0.mix.sink"][0], t["l0.mix.sink"][1] = -6.0, 7.0
    folder = helpers.make_norevik_dir(str(tmp_path / "far"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    tokens = [t if t != A else A + 1 for t in helpers.random_tokens(4, 330, V)]
    tokens[far_at] = A
    weights = attention_weights(config, tensors, tokens, 0)
    late = [t for t in range(250, 330) if float(weights[t, far_at]) > 0.5]
    assert len(late) >= 8, "the test's far key does not stand out"
    sunk = [t for t in range(250, 330) if float(attention_weights(config, tensors, tokens, 1)[t, -1]) > 0.5]
    assert len(sunk) >= 8, "the test's sink does not stand out"
    ref = P.forward(config, tensors, tokens).numpy()
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folder, dtype)
        slot = cache.open_slot()
        close(runner.step([entry(slot, tokens)]).cpu().numpy()[late], ref[late], dtype, "whole prompt", strict=True)
        cache.close_slot(slot)
        slot = cache.open_slot()                                  # portions: the far key lies in an earlier one
        rows = [runner.step([entry(slot, tokens[a:b])]).cpu().numpy() for a, b in [(0, 3), (3, 130), (130, 250), (250, 252)]]
        rows += [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens[252:]]      # then token by token
        close(np.concatenate(rows)[late], ref[late], dtype, "portions and decoding", strict=True)
        close(np.concatenate(rows), ref, dtype, "every position")
        runner.check_device_status()


@pytest.mark.parametrize("splits", [1, 3, 7])
def test_the_sink_counts_once_however_a_decode_steps_keys_are_cut(engine, tmp_path, splits):
    """Decoding over 300 cached tokens with the key tiles of a sequence cut into splits that are merged
    afterwards: the sink joins the denominator once, in the merge, not once per split."""
    from llama_rs_metal_b200.kernels import attention_dispatch
    spec = one_layer("latent_attention", helpers._sink_latent(3, 16, 16, 32, 48, 0.2, 100.0), seed=76)

    def edit(t):
        t["l0.mix.sink"].copy_(torch.tensor([3.0, -1.0, 6.0]))
    folder = helpers.make_norevik_dir(str(tmp_path / "cut"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    a, b = helpers.random_tokens(10, 330, 97), helpers.random_tokens(11, 90, 97)
    ref_a, ref_b = P.forward(config, tensors, a).numpy(), P.forward(config, tensors, b).numpy()
    runner, cache, _ = open_runner(engine, folder, "bfloat16", use_graphs=False)
    sa, sb = cache.open_slot(), cache.open_slot()
    runner.step([entry(sa, a[:300], []), entry(sb, b[:60], [])])
    attention_dispatch.force_shared_key_splits = splits
    try:
        outs = [runner.step([entry(sa, [a[300 + t]]), entry(sb, [b[60 + t]])]).cpu().numpy() for t in range(30)]
    finally:
        attention_dispatch.force_shared_key_splits = None
    close(np.stack([o[0] for o in outs]), ref_a[300:], "bfloat16", "the long sequence", strict=True)
    close(np.stack([o[1] for o in outs]), ref_b[60:], "bfloat16", "the short sequence", strict=True)


def test_rotation_pairs_neighbours_and_counts_from_each_sequences_start(engine, tmp_path):
    """Only the rotated parts carry the scores (the unrotated query is zero), with a base so small
    that every frequency turns many times over the prompt: pairing other dimensions, another angle
    or a position that does not start at zero for the second sequence of a batch shows."""
    spec = one_layer("latent_attention", helpers._sink_latent(2, 4, 12, 8, 8, 1.5, 3.0), seed=72)

    def edit(t):
        t["l0.mix.q"].view(2, 16, -1)[:, :4] = 0
    folder = helpers.make_norevik_dir(str(tmp_path / "rot"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    a, b = helpers.random_tokens(5, 100, 97), helpers.random_tokens(6, 70, 97)
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folder, dtype)
        sa, sb = cache.open_slot(), cache.open_slot()
        out = runner.step([entry(sa, a[:90]), entry(sb, b[:2])]).cpu().numpy()
        close(out[:90], P.forward(config, tensors, a).numpy()[:90], dtype, "first sequence")
        close(out[90:], P.forward(config, tensors, b).numpy()[:2], dtype, "second sequence")
        outs = [runner.step([entry(sa, [a[90 + t]]), entry(sb, [b[2 + t]])]).cpu().numpy() for t in range(10)]
        close(np.stack([o[0] for o in outs]), P.forward(config, tensors, a).numpy()[90:], dtype, "first sequence, decoded")
        close(np.stack([o[1] for o in outs]), P.forward(config, tensors, b).numpy()[2:12], dtype, "second sequence, decoded")


# --------------------------------------------------------------------------- state-space mixer
def test_a_state_space_head_remembers_its_first_token(engine, tmp_path):
    """Head 0 hardly decays (A_log = -14) and the first token's embedding is large: what the state
    took at position 0 is still most of the read-out 400 tokens later, through prompt, portions of
    one and two tokens (the convolution's tail has 3 inputs) and decoding."""
    spec = one_layer("mamba2", helpers._ssm(2, 16, 8, 1, 4, 1), seed=73, vocab=120)
    A = 11

    def edit(t):
        t["l0.mix.A_log"][0] = -14.0
        t["embed"][A] *= 15.0
    folder = helpers.make_norevik_dir(str(tmp_path / "ssm"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    tokens = [A] + [t if t != A else A + 1 for t in helpers.random_tokens(7, 420, 120)]
    ref = P.forward(config, tensors, tokens).numpy()
    other = P.forward(config, tensors, [A + 2] + tokens[1:]).numpy()
    assert np.abs(ref[400:] - other[400:]).max() > 0.1 * np.abs(ref).max(), "the first token does not show at the end"
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folder, dtype)
        slot = cache.open_slot()
        close(runner.step([entry(slot, tokens)]).cpu().numpy(), ref, dtype, "whole prompt")
        cache.close_slot(slot)
        slot, rows, at = cache.open_slot(), [], 0
        for n in [1, 2, 1, 1, 2, 300, 2, 1, 64, 3]:
            rows.append(runner.step([entry(slot, tokens[at:at + n])]).cpu().numpy())
            at += n
        rows += [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens[at:]]
        close(np.concatenate(rows), ref, dtype, "portions and decoding")
        runner.check_device_status()


# --------------------------------------------------------------------------- matrix memory
def test_the_matrix_memory_starts_its_maximum_at_zero_and_caps_its_gates(engine, tmp_path):
    """Input gates far below zero at every token (bias -8): the running maximum stays at its start, 0,
    so exp(-m) = 1 rules the denominator from the first token on; a maximum that started at minus
    infinity would give other numbers. Head 1's gate matrices are made large, so that tanh saturates
    and the cap is what the gates are."""
    spec = one_layer("mlstm", helpers._memory(2, 8, 12, 4.0), seed=74)

    def edit(t):
        t["l0.mix.i.b"][0] = -8.0
        t["l0.mix.i"][0] *= 0.1
        t["l0.mix.i"][1] *= 60.0
        t["l0.mix.f"][1] *= 60.0
    folder = helpers.make_norevik_dir(str(tmp_path / "mem"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    tokens = helpers.random_tokens(8, 140, 97)
    ref = P.forward(config, tensors, tokens).numpy()
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folder, dtype)
        slot = cache.open_slot()
        close(runner.step([entry(slot, tokens)]).cpu().numpy(), ref, dtype, "whole prompt")
        cache.close_slot(slot)
        slot = cache.open_slot()
        rows = [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens[:70]]          # from the very first token
        rows += [runner.step([entry(slot, tokens[70:72])]).cpu().numpy(), runner.step([entry(slot, tokens[72:])]).cpu().numpy()]
        close(np.concatenate(rows), ref, dtype, "decoding, then portions")
        runner.check_device_status()


# --------------------------------------------------------------------------- routing
def test_negative_choice_scores_stay_inside_the_kept_groups(engine, tmp_path):
    """Every correction is far below zero, so every choice score is negative: an expert outside the
    kept groups whose score counted as 0 would beat all of them. Identity experts are among the
    chosen; weights are the scores without the correction, not renormalized."""
    mlp = helpers._experts(24, 6, 3, identity=2, groups=(4, 2), shared=32)
    spec = one_layer("mamba2", SMALL_SSM, mlp, seed=75)

    def edit(t):
        t["l0.mlp.correction"].mul_(0.1).sub_(3.0)
    folder = helpers.make_norevik_dir(str(tmp_path / "route"), spec, edit=edit)
    config, tensors = P.read_model(folder)
    tokens = helpers.random_tokens(9, 300, 97)
    streams = []
    ref = P.forward(config, tensors, tokens, streams).numpy()
    # the test's own expectations about the plain routing of this input
    x = tensors["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    h = x + P.layer_norm(P.mamba2(x, config["layers"][0]["mixer"], tensors, "l0.mix.", 1e-5), tensors["l0.norm1"],
                         tensors["l0.norm1.b"], 1e-5)
    chosen, weights, scores = P.route(h, mlp, tensors, "l0.mlp.")
    choice = scores + tensors["l0.mlp.correction"]
    assert float(choice.max()) < 0
    naive = torch.topk(choice, 3, dim=-1).indices
    differ = sum(sorted(a) != sorted(b) for a, b in zip(chosen.tolist(), naive.tolist()))
    assert differ > 30, "the groups do not change the choice often enough"
    assert int((chosen >= 6).sum()) > 30 and float(weights.sum(dim=1).max()) < 0.999
    assert len({c // 2 for row in chosen.tolist() for c in row}) == 4, "every group is kept for some token"
    for dtype in ("float32",):   # under bfloat16 activations a close call now and then falls the other way
        runner, cache, _ = open_runner(engine, folder, dtype)
        slot = cache.open_slot()
        close(runner.step([entry(slot, tokens[:280])]).cpu().numpy(), ref[:280], dtype, "prompt")
        rows = [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens[280:]]
        close(np.concatenate(rows), ref[280:], dtype, "decoding")
        runner.check_device_status()


# --------------------------------------------------------------------------- norms
@pytest.mark.parametrize("width", [24, 72, 320, 1000, 4100, 9000])
def test_layer_norm_and_the_norm_behind_a_sublayer(width):
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(width)
    T, eps = 37, 1e-5
    x = torch.randn(T, width, generator=gen) * 3 + 5          # a mean far from zero: the variance is of the deviations
    x[3] = 2.5                                                # a constant row: only eps keeps it finite
    w, b = torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    want = P.layer_norm(x.to(F64), w.to(F64), b.to(F64), eps)
    dev = lambda t: t.to(DEV).contiguous()
    got = ops.layer_norm(dev(x), dev(w), dev(b), eps, torch.float32).cpu()
    assert (got.to(F64) - want).abs().max() < 2e-5 * want.abs().max()
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=DEV)
    got = ops.layer_norm(dev(x), dev(w), dev(b), eps, torch.bfloat16, rows=rows).float().cpu()
    assert (got.to(F64) - want[[5, 0, 36]]).abs().max() < 1e-2 * want.abs().max()
    stream = torch.randn(T, width, generator=gen)
    for cast_dtype in (None, torch.bfloat16):
        s = dev(stream.clone())
        out = ops.layer_norm_add_(s, dev(x), dev(w), dev(b), eps, 0.5, cast_dtype=cast_dtype)
        expect = stream.to(F64) + 0.5 * want
        assert (s.cpu().to(F64) - expect).abs().max() < 2e-5 * expect.abs().max()
        if cast_dtype is not None:
            assert torch.equal(out, s.to(cast_dtype)), "the rounded copy is the rounding of the updated stream"


# --------------------------------------------------------------------------- awkward sizes
def test_sizes_that_are_multiples_of_nothing(engine, tmp_path):
    """Width 67, vocabulary 101, head, state, value, latent and expert sizes that are odd or prime: no
    size is a multiple of 4, 8 or 16, so every kernel's path for unaligned rows runs (and the
    vectorized or tensor-core path of none)."""
    spec = dict(config=dict(architecture="Norevik", vocab=101, width=67, norm=dict(eps=3e-6), embedding=dict(scale=2.5), layers=[
        dict(type="mamba2", mixer=helpers._ssm(3, 5, 7, 3, 3, 5), mlp=helpers._experts(9, 3, 2, identity=1, groups=(2, 2), shared=11)),
        dict(type="latent_attention", mixer=helpers._sink_latent(3, 5, 6, 7, 9, 0.3, 77.0), mlp=helpers._plain_ff(13)),
        dict(type="mlstm", mixer=helpers._memory(5, 3, 9, 3.5), mlp=None),
    ]), seed=77, std=0.2)
    for dtype in ("float32", "bfloat16"):
        folder = helpers.make_norevik_dir(str(tmp_path / dtype), spec, steady_routing=dtype == "bfloat16")
        plain = {("odd", dtype): P.read_model(folder)}
        a, b = helpers.random_tokens(12, 120, 101), helpers.random_tokens(13, 45, 101)
        ref_a, ref_b = reference(plain, ("odd", dtype), a), reference(plain, ("odd", dtype), b)   # with each row's allowance
        runner, cache, _ = open_runner(engine, folder, dtype)
        sa, sb = cache.open_slot(), cache.open_slot()
        out = runner.step([entry(sa, a[:100]), entry(sb, b[:25])]).cpu().numpy()
        close(out[:100], ref_a[:100], dtype, "the first prompt")
        close(out[100:], ref_b[:25], dtype, "the second prompt")
        outs = [runner.step([entry(sa, [a[100 + t]]), entry(sb, [b[25 + t]])]).cpu().numpy() for t in range(20)]
        close(np.stack([o[0] for o in outs]), ref_a[100:], dtype, "the first sequence, decoded")
        close(np.stack([o[1] for o in outs]), ref_b[25:], dtype, "the second sequence, decoded")
        runner.check_device_status()

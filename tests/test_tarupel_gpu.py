"""The Tarupel decoder on the GPU against the plain float64 implementation (tests/plain_tarupel.py):
whole models through the step function, the cache and the generation loop, then every new
mechanism alone with inputs made so that a fault shows."""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_tarupel as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64
NAMES = ["T1", "T2", "T3"]


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> folder; the bfloat16 folders route steadily (see helpers.make_tarupel_dir)."""
    root = tmp_path_factory.mktemp("tarupel")
    out = {}
    for name in NAMES:
        out[name, "float32"] = helpers.make_tarupel_dir(str(root / f"{name}_f"), name)
        out[name, "bfloat16"] = helpers.make_tarupel_dir(str(root / f"{name}_b"), name, steady_routing=True)
    return out


@pytest.fixture(scope="module")
def plain(folders):
    return {key: P.read_model(path) for key, path in folders.items()}


_REFS = {}


def reference(plain, which, tokens):
    key = (which, tuple(tokens))
    if key not in _REFS:
        config, tensors = plain[which]
        _REFS[key] = P.forward(config, tensors, tokens).numpy()
    return _REFS[key]


# Allowed error of a row of logits as a fraction of the largest reference logit. float32: sums in
# another order than the plain implementation's float64, and a recurrence that feeds back what it
# adds up. bfloat16: activations are rounded between kernels; a fault of any mechanism is far above.
# In bfloat16 one row in twenty may be up to four times over while the median stays below a third.
TOLERANCE = {"float32": 5e-5, "bfloat16": 5e-2}


def close(got, ref, dtype, what, factor=1.0):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got.reshape(1, -1), ref.reshape(1, -1)
    assert got.shape == ref.shape and np.all(np.isfinite(got)), what
    err = np.abs(got - ref).max(axis=-1) / max(float(np.abs(ref).max()), 1e-30)
    allowed = factor * TOLERANCE[dtype]
    worst = int(err.argmax())
    report = (f"{what}: row {worst} off by {err[worst]:.3e} of the largest logit (allowed {allowed:.0e}); first such row "
              f"{int(np.argmax(err > allowed))}; {int((err > allowed).sum())} of {len(err)} rows over; median {np.median(err):.3e}")
    if dtype == "bfloat16" and len(err) >= 8:
        assert (err > allowed).sum() <= max(1, len(err) // 20) and err[worst] <= 4 * allowed \
            and np.median(err) <= allowed / 3, report
    else:
        assert err[worst] <= allowed, report


def vocab_of(name):
    return helpers.TARUPEL[name]["config"]["vocab"]


def open_runner(engine, folder, dtype, max_tokens=2048, max_slots=8, use_graphs=True):
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.engine.session import build_model
    from llama_rs_metal_b200.engine.step import StepRunner
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype
    rt = Runtime(engine.device, parse_dtype(dtype))
    _, _, model, _ = build_model(folder, rt)
    cache = Cache(model.cache_requests(), rt.dtype, rt.device, max_tokens, max_slots, max_tokens)
    return StepRunner(model, cache, rt, use_graphs=use_graphs), cache, model


def entry(slot, tokens, want=None):
    from llama_rs_metal_b200.engine.batch import StepEntry
    return StepEntry(slot, tokens, range(len(tokens)) if want is None else want)


# --------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_match_the_plain_implementation(engine, folders, plain, name, dtype):
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    for i, n in enumerate([150, 37, 1, 2]):       # the first tokens of a sequence are rows 0, 1, ...
        tokens = helpers.random_tokens(300 + i, n, vocab_of(name))
        slot = cache.open_slot()
        got = runner.step([entry(slot, tokens)]).cpu().numpy()
        cache.close_slot(slot)                     # the next prompt takes the same slot and state
        close(got, reference(plain, (name, dtype), tokens), dtype, f"{name} prompt of {n}")
    runner.check_device_status()


@pytest.mark.parametrize("name", NAMES)
def test_every_layer_run_matches_the_plain_residual_stream(engine, folders, plain, name):
    dtype = "float32"
    runner, cache, model = open_runner(engine, folders[name, dtype], dtype, use_graphs=False)
    seen = []
    for block in model.blocks:
        def wrapped(hidden, ctx, view, inner=block.forward):
            out = inner(hidden, ctx, view)
            seen.append(out.detach().clone().cpu().to(F64))
            return out
        block.forward = wrapped
    tokens = helpers.random_tokens(8, 90, vocab_of(name))
    slot = cache.open_slot()
    runner.step([entry(slot, tokens, [])])
    config, tensors = plain[name, dtype]
    streams = []
    P.forward(config, tensors, tokens, streams)
    assert len(seen) == len(streams) == len(P.layer_runs(config))
    for i, (got, want) in enumerate(zip(seen, streams)):
        err = float((got[:len(tokens)] - want).abs().max() / want.abs().max())
        assert err < 2e-5, f"{name}: the stream after layer run {i} is off by {err:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_decoding_in_an_unequal_batch(engine, folders, plain, name, dtype):
    """Prompts of unequal lengths in one step, then one token each per step, past a page's border
    and past every window and chunk; the shorter requests end earlier and the batch shrinks."""
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    V = vocab_of(name)
    totals, prompts = [140, 75, 9, 58], [100, 60, 1, 2]
    seqs = [helpers.random_tokens(40 + i, n, V) for i, n in enumerate(totals)]
    refs = [reference(plain, (name, dtype), s) for s in seqs]
    slots = [cache.open_slot() for _ in seqs]
    out = runner.step([entry(sl, s[:n]) for sl, s, n in zip(slots, seqs, prompts)]).cpu().numpy()
    row = 0
    for b, n in enumerate(prompts):
        close(out[row:row + n], refs[b][:n], dtype, f"{name} prompt {b} in the batch")
        row += n
    at, decoded = list(prompts), [[] for _ in seqs]
    while any(a < t for a, t in zip(at, totals)):
        live = [b for b in range(len(seqs)) if at[b] < totals[b]]
        out = runner.step([entry(slots[b], [seqs[b][at[b]]]) for b in live]).cpu().numpy()
        for i, b in enumerate(live):
            decoded[b].append(out[i])
            at[b] += 1
            if at[b] == totals[b]:
                cache.close_slot(slots[b])
    for b, n in enumerate(prompts):
        close(np.stack(decoded[b]), refs[b][n:], dtype, f"{name} sequence {b}, decoded from position {n}")
    runner.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["T1", "T2"])
def test_a_prompt_geometry_that_comes_again_is_captured_and_replayed(engine, folders, plain, name, dtype):
    """The same shape of batch four times with other tokens, in slots that were used before: states,
    tails and shifted rows must start from zero each time, also under a captured graph's replay."""
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    V = vocab_of(name)
    following, expected = [], []
    for turn in range(4):
        seqs = [helpers.random_tokens(500 + 10 * turn + i, n, V) for i, n in enumerate([70, 3, 41])]
        slots = [cache.open_slot() for _ in seqs]
        out = runner.step([entry(sl, s) for sl, s in zip(slots, seqs)]).cpu().numpy()
        row = 0
        for s in seqs:
            close(out[row:row + len(s)], reference(plain, (name, dtype), s), dtype, f"{name} turn {turn}")
            row += len(s)
        nxt = [int(t) for t in helpers.random_tokens(900 + turn, len(seqs), V)]
        out = runner.step([entry(sl, [t]) for sl, t in zip(slots, nxt)]).cpu().numpy()
        for i, (s, t) in enumerate(zip(seqs, nxt)):
            following.append(out[i])
            expected.append(reference(plain, (name, dtype), s + [t])[-1])
        for sl in slots:
            cache.close_slot(sl)
    close(np.stack(following), np.stack(expected), dtype, f"{name}: the token after each prompt")
    runner.check_device_status()


@pytest.mark.parametrize("sizes", [[2], [3, 64, 5], [1, 70, 2], [64], [17]])
@pytest.mark.parametrize("name", ["T1", "T2"])
def test_portions_of_any_size_give_the_whole_prompt(engine, folders, plain, name, sizes):
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
        tokens = helpers.random_tokens(77, 150 if sizes != [2] else 40, vocab_of(name))
        ref = reference(plain, (name, dtype), tokens)
        slot, at, i, rows = cache.open_slot(), 0, 0, []
        while at < len(tokens):
            n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
            rows.append(runner.step([entry(slot, tokens[at:at + n])]).cpu().numpy())
            at, i = at + n, i + 1
        close(np.concatenate(rows), ref, dtype, f"{name} in portions of {sizes}")
        cache.close_slot(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_company_in_the_batch_changes_nothing_beyond_rounding(engine, folders, plain, dtype):
    name = "T2"
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    V = vocab_of(name)
    mine = helpers.random_tokens(5, 130, V)
    others = [helpers.random_tokens(6 + i, n, V) for i, n in enumerate([200, 3, 64])]
    slot = cache.open_slot()
    alone = runner.step([entry(slot, mine)]).cpu().numpy()
    cache.close_slot(slot)
    slots = [cache.open_slot() for _ in range(4)]
    together = runner.step([entry(slots[0], others[0], []), entry(slots[1], mine), entry(slots[2], others[1], []),
                            entry(slots[3], others[2], [])]).cpu().numpy()
    limit = 1e-5 if dtype == "float32" else 3e-2
    assert np.abs(alone - together).max() <= limit * np.abs(alone).max()
    close(together, reference(plain, (name, dtype), mine), dtype, "in company")


def test_a_freed_slot_and_its_pages_start_from_nothing(engine, folders, plain):
    """The state, the convolution's tail and the shifted row of a slot are cleared when it is taken
    again, and the pages a sequence gave back hold another sequence's keys when they are used again."""
    name = "T1"
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folders[name, dtype], dtype, max_tokens=512, max_slots=2)
        V = vocab_of(name)
        first = helpers.random_tokens(1, 200, V)
        slot = cache.open_slot()
        runner.step([entry(slot, first, [])])
        for t in helpers.random_tokens(2, 5, V):
            runner.step([entry(slot, [t], [])])
        cache.close_slot(slot)
        second = helpers.random_tokens(3, 90, V)
        again = cache.open_slot()
        assert again == slot
        got = [runner.step([entry(again, second[:50])]).cpu().numpy()]
        for t in second[50:]:
            got.append(runner.step([entry(again, [t])]).cpu().numpy())
        close(np.concatenate(got), reference(plain, (name, dtype), second), dtype, "the slot's second sequence")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(engine, folders, plain, dtype):
    """300 tokens one by one from the very first: several pages, windows and chunks pass by, the
    states are carried through hundreds of captured steps."""
    name = "T1"
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    tokens = helpers.random_tokens(9, 300, vocab_of(name))
    ref = reference(plain, (name, dtype), tokens)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens]
    close(np.concatenate(rows), ref, dtype, "token by token from the start", factor=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_session(engine, folders, plain, dtype):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    name = "T2"
    model = engine.load(folders[name, dtype], dtype=dtype)
    session = model.session(context=256, max_batch=4)
    V = vocab_of(name)
    prompts = [helpers.random_tokens(60 + i, n, V) for i, n in enumerate([70, 5, 33])]
    results = session.generate(prompts, GenerationOptions(max_tokens=12, sampling=Sampling(temperature=0.0)))
    config, tensors = plain[name, dtype]
    for prompt, result in zip(prompts, results):
        tokens = list(prompt)
        assert len(result.tokens) == 12
        for chosen in result.tokens:
            logits = P.forward(config, tensors, tokens)[-1].numpy()
            best = int(logits.argmax())
            if chosen != best:   # a near tie may fall the other way under rounding
                gap = (logits[best] - logits[chosen]) / np.abs(logits).max()
                assert gap < (1e-4 if dtype == "float32" else 5e-2), f"chose {chosen}, the plain model {best} by {gap:.2e}"
            tokens.append(chosen)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(folders, plain, dtype, tmp_path):
    name = "T1"
    V = vocab_of(name)
    requests = {f"r{i}": helpers.random_tokens(90 + i, n, V) for i, n in enumerate([120, 40, 77])}
    trace = helpers.Trace()
    trace.whole("whole:r0", requests["r0"])
    trace.tail_one_by_one("tail:r1", requests["r1"], tail=20)
    trace.batch({f"batch:{n}": t for n, t in requests.items()}, {"batch:r0": 90, "batch:r1": 10, "batch:r2": 70})
    outputs = helpers.run_trace(folders[name, dtype], dtype, trace, 1024, str(tmp_path / "out"))
    refs = {n: reference(plain, (name, dtype), t) for n, t in requests.items()}
    for step in sorted(trace.rows):
        rows = trace.rows[step]
        ref = np.stack([refs[rid.split(":")[-1]][pos] for rid, pos in rows])
        close(outputs[step], ref, dtype, f"step {step}")


# --------------------------------------------------------------------------- configurations drawn at random
def drawn_configuration(seed):
    rng = np.random.default_rng(seed)

    def pick(*values):
        return values[int(rng.integers(len(values)))]

    def feed_forward():
        kind = pick(None, "dense", "moe", "moe")
        if kind is None:
            return None
        if kind == "dense":
            return dict(kind="dense", ff=int(pick(24, 64, 100)))
        count, size = int(pick(1, 2, 3)), int(pick(1, 2, 4))      # groups, experts per group
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, keep * size + 1))
        return helpers._scored_experts(int(pick(8, 24, 40)), count * size, top, pick(None, 0.5, 2.0),
                                       (count, keep) if rng.integers(3) else None, pick(None, 16, 48))
    width = int(pick(40, 64, 88, 136))
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = pick("general_delta", "attention", "attention_2")
        if kind == "general_delta":
            mixer = helpers._delta(int(pick(1, 2, 3)), int(pick(4, 10, 16, 40)), int(pick(1, 4, 9)))
        else:
            kv = int(pick(1, 2, 3))
            dim = int(pick(4, 16, 24, 64))
            rot = int(pick(*[r for r in (2, 4, 8, 16, 64) if r <= dim]))
            mixer = helpers._masked(kv * int(pick(1, 2)), kv, dim, int(pick(dim, dim, 8, 12)), float(pick(0.1, 0.4)), rot,
                                    float(pick(30.0, 10000.0)), int(pick(1, 3, 40, 64, 65, 200)),
                                    conv=int(pick(1, 2, 4, 5)) if kind == "attention" else None)
        layers.append(dict(type=kind, mixer=mixer, mlp=feed_forward()))
    config = dict(architecture="Tarupel", vocab=int(pick(97, 256, 333)), width=width, norm=dict(eps=float(pick(1e-6, 1e-4))),
                  embedding=dict(scale=float(pick(0.5, 1.0, 6.0))), residual_mult=float(pick(1.0, 0.5, 1.3)), layers=layers)
    if rng.integers(3):
        start = int(rng.integers(0, len(layers)))
        config["loop"] = dict(start=start, stop=int(rng.integers(start + 1, len(layers) + 1)), times=int(pick(1, 2, 3)))
    return dict(config=config, seed=3000 + seed, std=float(pick(0.08, 0.15)))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(engine, tmp_path, seed):
    """Other sizes, orders of layers, loops and constants than the fixed configurations: a prompt
    whole, then tokens one by one, a second sequence beside it in portions."""
    spec = drawn_configuration(seed)
    for dtype in ("float32", "bfloat16"):
        folder = helpers.make_tarupel_dir(str(tmp_path / dtype), spec, steady_routing=dtype == "bfloat16")
        config, tensors = P.read_model(folder)
        V = spec["config"]["vocab"]
        a, b = helpers.random_tokens(seed, 150, V), helpers.random_tokens(seed + 50, 100, V)
        ref_a, ref_b = P.forward(config, tensors, a).numpy(), P.forward(config, tensors, b).numpy()
        runner, cache, _ = open_runner(engine, folder, dtype)
        sa, sb = cache.open_slot(), cache.open_slot()
        out = runner.step([entry(sa, a[:120]), entry(sb, b[:3])]).cpu().numpy()
        close(out[:120], ref_a[:120], dtype, f"seed {seed}: prompt a", factor=2.0)
        close(out[120:], ref_b[:3], dtype, f"seed {seed}: prompt b", factor=2.0)
        out = runner.step([entry(sa, a[120:121]), entry(sb, b[3:70])]).cpu().numpy()     # one token and a portion
        close(out[:1], ref_a[120:121], dtype, f"seed {seed}: a's next token", factor=2.0)
        close(out[1:], ref_b[3:70], dtype, f"seed {seed}: b's portion", factor=2.0)
        rows_a, rows_b = [], []
        for t in range(121, 150):
            entries = [entry(sa, [a[t]])] + ([entry(sb, [b[t - 51]])] if t - 51 < 100 else [])
            out = runner.step(entries).cpu().numpy()
            rows_a.append(out[0])
            if len(entries) > 1:
                rows_b.append(out[1])
        close(np.stack(rows_a), ref_a[121:], dtype, f"seed {seed}: a decoded", factor=2.0)
        close(np.stack(rows_b), ref_b[70:70 + len(rows_b)], dtype, f"seed {seed}: b decoded", factor=2.0)
        runner.check_device_status()


@pytest.mark.parametrize("experts,top,groups,shared", [(24, 3, (6, 2), 40), (20, 5, None, None), (32, 2, (4, 4), 16)])
def test_many_experts_take_the_logits_first_router(engine, tmp_path, experts, top, groups, shared):
    """More router outputs than a token's CTA scores itself and a prompt of 300 tokens: the logits come
    from the float32 product and the scored choice is made from them; then decoding (the one-launch
    router) from the same state."""
    layer = dict(type="attention_2", mixer=helpers._masked(2, 1, 16, 16, 0.25, 8, 100.0, 50),
                 mlp=helpers._scored_experts(24, experts, top, 1.7, groups, shared))
    spec = dict(config=dict(architecture="Tarupel", vocab=128, width=48, norm=dict(eps=1e-5), residual_mult=0.9,
                            layers=[layer, dict(layer, type="general_delta", mixer=helpers._delta(2, 8, 3))]),
                seed=77 + experts, std=0.15)
    folder = helpers.make_tarupel_dir(str(tmp_path / "m"), spec)
    config, tensors = P.read_model(folder)
    tokens = helpers.random_tokens(experts, 330, 128)
    ref = P.forward(config, tensors, tokens).numpy()
    runner, cache, _ = open_runner(engine, folder, "float32")
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, tokens[:300])]).cpu().numpy()]
    rows += [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens[300:]]
    close(np.concatenate(rows), ref, "float32", f"{experts} experts")


# --------------------------------------------------------------------------- the generalized delta rule
def plain_general_scan(r, k, v, g, look, put, state):
    """One sequence, float64: everything [T, H, d] but v [T, H, dv]; state [H, d, dv], updated in place."""
    T, H, _ = r.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for h in range(H):
            old = state[h]
            state[h] = g[t, h][:, None] * old + torch.outer(put[t, h], look[t, h] @ old) + torch.outer(k[t, h], v[t, h])
            out[t, h] = state[h].T @ r[t, h]
    return out


@pytest.mark.parametrize("H,d,dv", [(3, 24, 40), (2, 80, 8), (4, 64, 64), (1, 5, 3), (2, 130, 16)])
def test_generalized_scan_matches_the_recurrence_and_carries_its_state(H, d, dv):
    """Two sequences and a sequence of padding between them, in slots out of order; the state is
    carried over steps of 37, 1, 2 and 17 tokens. Some channels hardly decay, the removal is strong:
    a term that reads the decayed state instead of the old one, or a sign, shows at once."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(H * 1000 + d)
    lengths = [57, 57]
    rand = lambda *s: torch.randn(*s, generator=gen, dtype=F64)  # noqa: E731
    seqs = []
    for n in lengths:
        k = rand(n, H, d) * 0.5
        unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        g = torch.exp(-0.6 * torch.sigmoid(rand(n, H, d) * 3.0))
        g[:, :, 0] = 0.9999
        seqs.append(dict(r=rand(n, H, d), k=k, v=rand(n, H, dv), g=g, look=unit, put=-torch.sigmoid(rand(n, H, d) * 2.0) * unit))
    states = [torch.zeros(H, d, dv, dtype=F64) for _ in seqs]
    refs = [plain_general_scan(s["r"], s["k"], s["v"], s["g"], s["look"], s["put"], st) for s, st in zip(seqs, states)]
    device_state = torch.full((5, H, d, dv), 7.0, dtype=torch.float32, device=DEV)   # slots 3 and 1 are used
    slot_of = [3, 1]
    device_state[slot_of] = 0.0
    slots = torch.tensor([3, -1, 1], dtype=torch.int32, device=DEV)
    at, outs = 0, [[], []]
    for n in (37, 1, 2, 17):
        pad = 4
        parts = {name: torch.cat([seqs[0][name][at:at + n], torch.ones(pad, H, seqs[0][name].shape[2], dtype=F64),
                                  seqs[1][name][at:at + n]]).to(torch.float32).to(DEV).contiguous()
                 for name in ("r", "k", "v", "g", "look", "put")}
        cu = torch.tensor([0, n, n + pad, 2 * n + pad], dtype=torch.int32, device=DEV)
        o = ops.general_delta_scan(parts["r"], parts["k"], parts["v"], parts["g"], parts["look"], parts["put"], device_state,
                                   cu, slots).cpu().double()
        outs[0].append(o[:n])
        outs[1].append(o[n + pad:])
        at += n
    for b in range(2):
        got = torch.cat(outs[b])
        assert float((got - refs[b]).abs().max()) <= 3e-5 * float(refs[b].abs().max()), f"sequence {b}"
        assert float((device_state[slot_of[b]].cpu().double() - states[b]).abs().max()) <= 3e-5 * float(states[b].abs().max())
    assert float((device_state[[0, 2, 4]] - 7.0).abs().max()) == 0.0, "another slot's state was touched"


def test_generalized_delta_inputs():
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(3)
    T, H, d, dv, extra = 9, 3, 20, 12, 5
    W = 3 * H * d + H * dv + extra
    for dtype in (torch.float32, torch.bfloat16):
        proj = (torch.randn(T, W, generator=gen) * 1.5).to(dtype)
        z = torch.randn(T, H * d, generator=gen)
        zb, ab = torch.randn(H * d, generator=gen), torch.randn(H * d, generator=gen)
        offs = dict(r=extra, k=extra + H * d, v=extra + 2 * H * d, a=extra + 2 * H * d + H * dv)
        r, k, v, g, look, put = ops.general_delta_prepare(proj.to(DEV), offs["r"], offs["k"], offs["v"], offs["a"], z.to(DEV),
                                                          zb.to(DEV), ab.to(DEV), 0.55, 1e-6, H, d, dv)
        p = proj.double()
        kk = p[:, offs["k"]:offs["k"] + H * d].reshape(T, H, d)
        unit = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
        rate = torch.sigmoid(p[:, offs["a"]:offs["a"] + H * d] + ab.double()).reshape(T, H, d)
        want = dict(r=p[:, offs["r"]:offs["r"] + H * d].reshape(T, H, d), k=kk, v=p[:, offs["v"]:offs["v"] + H * dv].reshape(T, H, dv),
                    g=torch.exp(-0.55 * torch.sigmoid(z.double() + zb.double())).reshape(T, H, d), look=unit, put=-rate * unit)
        for name, got in dict(r=r, k=k, v=v, g=g, look=look, put=put).items():
            assert float((got.cpu().double() - want[name]).abs().max()) < 2e-6 * max(1.0, float(want[name].abs().max())), name


# --------------------------------------------------------------------------- shaped queries and keys
def shaped_reference(proj, bias, taps, q_norm, k_norm, row_eps, rot, adjacent, base, head_eps, Hq, Hk, d, dv):
    """One sequence from its first token, float64, with the plain implementation's own pieces."""
    T = proj.shape[0]
    x = proj + (bias if bias is not None else 0.0)
    if taps is not None:
        x = P.causal_conv(x, taps)
    q, k, v = x[:, :Hq * d], x[:, Hq * d:(Hq + Hk) * d], x[:, (Hq + Hk) * d:]
    if q_norm is not None:
        q, k = P.unit_rms(q, row_eps) * q_norm, P.unit_rms(k, row_eps) * k_norm
    q, k = q.reshape(T, Hq, d), k.reshape(T, Hk, d)
    if rot:
        turn = P.rotate_pairs if adjacent else P.rotate_halves
        q, k = turn(q, torch.arange(T), rot, base), turn(k, torch.arange(T), rot, base)
    if head_eps is not None:
        q, k = P.unit_rms(q, head_eps), P.unit_rms(k, head_eps)
    return q, k, v.reshape(T, Hk, dv)


@pytest.mark.parametrize("taps_n,row_norm,rot,adjacent,head_norm", [
    (4, False, 6, False, True), (1, False, 12, False, True), (0, True, 4, True, False), (5, True, 12, True, True),
    (3, False, 0, False, False), (2, False, 2, True, False)])
def test_shaped_split_in_portions_matches_the_definition(taps_n, row_norm, rot, adjacent, head_norm):
    """The whole sequence at once, and in portions of 1, 2, 7 and the rest (shorter and longer than
    the convolution's tail) from a slot whose tail held another sequence's numbers: positions far
    from zero, both pairings, both norms, the tail's zeros in front of the first tokens."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(taps_n * 10 + rot)
    T, Hq, Hk, d, dv, base = 40, 4, 2, 12, 5, 50.0
    W = Hq * d + Hk * (d + dv)
    proj = torch.randn(T, W, generator=gen, dtype=torch.float32)
    bias = torch.randn(W, generator=gen, dtype=torch.float32)
    taps = torch.randn(W, taps_n, generator=gen, dtype=torch.float32) if taps_n else None
    qw = (1.0 + 0.3 * torch.randn(Hq * d, generator=gen)) if row_norm else None
    kw = (1.0 + 0.3 * torch.randn(Hk * d, generator=gen)) if row_norm else None
    inv = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64, device=DEV) if rot else None
    dd = lambda t: None if t is None else t.double()  # noqa: E731
    want = shaped_reference(proj.double(), bias.double(), dd(taps), dd(qw), dd(kw), 1e-5, rot, adjacent, base,
                            1e-6 if head_norm else None, Hq, Hk, d, dv)
    dev = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    for cuts in ([T], [1, 2, 7, T - 10]):
        tails = torch.full((3, max(taps_n - 1, 1), W), 5.0, dtype=torch.float32, device=DEV)
        tails[1] = 0.0                                            # the slot as the cache hands it out
        got, at = [], 0
        for n in cuts:
            part = proj[at:at + n].to(DEV).contiguous()
            args = dict(bias=dev(bias), taps=None if taps is None else taps.t().contiguous().to(DEV),
                        tails=tails if taps_n > 1 else None,
                        cu_seqlens=torch.tensor([0, n], dtype=torch.int32, device=DEV),
                        seq_of_token=torch.zeros(n, dtype=torch.int32, device=DEV),
                        slots=torch.tensor([1], dtype=torch.int32, device=DEV),
                        row_norm=(dev(qw), dev(kw)) if row_norm else None, row_eps=1e-5, inv_freq=inv, rotary=rot,
                        adjacent_pairs=adjacent, head_norm_eps=1e-6 if head_norm else None)
            got.append(ops.shaped_qkv_store(part, Hq, Hk, d, dv, torch.arange(at, at + n, dtype=torch.int32, device=DEV),
                                            torch.float32, **args))
            at += n
        for i, name in enumerate("qkv"):
            have = torch.cat([g[i] for g in got]).cpu().double()
            assert float((have - want[i]).abs().max()) < 3e-6 * max(1.0, float(want[i].abs().max())), (name, cuts)
        assert float((tails[[0, 2]] - 5.0).abs().max()) == 0.0


# --------------------------------------------------------------------------- chunks and windows
def plain_masked_attention(q, k, v, scale, first_visible):
    """float64; q [L, H, d], k, v [L, G, d|dv]; query i sees keys first_visible(i) .. i."""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, v.shape[2], dtype=F64)
    for i in range(L):
        lo = first_visible(i)
        for h in range(H):
            kh = h // (H // G)
            out[i, h] = torch.softmax((k[lo:i + 1, kh] @ q[i, h]) * scale, 0) @ v[lo:i + 1, kh]
    return out


@pytest.mark.parametrize("dtype,d,dv,span,chunked", [
    (torch.float32, 24, 40, 7, True), (torch.float32, 96, 96, 64, True), (torch.float32, 16, 16, 70, True),
    (torch.bfloat16, 64, 64, 70, True), (torch.bfloat16, 32, 32, 64, True), (torch.bfloat16, 128, 128, 100, True),
    (torch.bfloat16, 48, 16, 65, True), (torch.bfloat16, 64, 64, 1, True), (torch.float32, 8, 8, 1, False),
    (torch.bfloat16, 64, 64, 40, False), (torch.float32, 96, 96, 200, True)])
def test_a_key_that_stands_out_just_inside_and_just_outside_a_chunk_or_window(dtype, d, dv, span, chunked):
    """One key's score is far above all others for every query that sees it, so a query's output is
    that key's value exactly while the key is visible. For chunks the key is the first of its chunk
    (seen up to span - 1 positions later, among up to hundreds of others) and then the last (the next
    query starts a new chunk and does not see it); for windows it is seen at distance span - 1 and not
    at span. Prompts, decoding and portions of three, with the edges on and next to page borders."""
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.kernels import ops
    from llama_rs_metal_b200.parts.base import KeyValueRequest
    H, G, L = 4, 2, 330
    gen = torch.Generator().manual_seed(d + span)
    first_visible = (lambda i: i - i % span) if chunked else (lambda i: max(0, i - span + 1))
    window = -span if chunked else span
    if chunked:
        start = (128 // span) * span if span > 1 else 128
        spikes = [start, start + span - 1]
    else:
        spikes = [64 - span + 64, 127]
    for spike in spikes:
        edge = (spike - spike % span + span) if chunked else spike + span     # the first query that does not see it
        if edge + 5 >= L:
            continue
        q = torch.randn(L, H, d, generator=gen, dtype=F64) * 0.1
        k = torch.randn(L, G, d, generator=gen, dtype=F64) * 0.1
        v = torch.randn(L, G, dv, generator=gen, dtype=F64)
        q[:, :, 0] = 6.0
        k[spike, :, 0] = 6.0                      # score 36 above the rest
        v[spike] = 9.0
        r = lambda t: t.to(dtype).to(DEV).contiguous()  # noqa: E731
        rq, rk, rv = r(q), r(k), r(v)
        ref = plain_masked_attention(rq.cpu().double(), rk.cpu().double(), rv.cpu().double(), 1.0, first_visible)
        assert float((ref[edge - 1] - 9.0).abs().max()) < 0.5 and float((ref[edge] - 9.0).abs().min()) > 3.0
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        cu = torch.tensor([0, L], dtype=torch.int32, device=DEV)
        seq_of = torch.zeros(L, dtype=torch.int32, device=DEV)
        got = ops.attention_prefill(rq, rk, rv, cu, seq_of, L, 1.0, window)
        assert float((got.cpu().double().reshape(L, H, dv) - ref).abs().max()) <= tol * 9.0, f"prompt, key {spike}"
        cache = Cache([KeyValueRequest(G, d, span, None if dv == d else dv)], dtype, torch.device(DEV), 512, 2, 512)
        cache.open_slot()
        slot = cache.open_slot()
        for portion in (1, 3):
            cache.reset_slot(slot)
            rows = []
            first = edge - 4
            cache.grow([(slot, first)])
            cache.sync()
            dest = torch.tensor(cache.destination_rows([slot], [0], [first])[0], device=DEV)
            packed = torch.cat([rq[:first].reshape(first, -1), rk[:first].reshape(first, -1),
                                rv[:first].reshape(first, -1)], dim=1).contiguous()
            ops.qkv_bias_store(packed, None, H, G, d, dv, kv=cache.view(0), dest_rows=dest, keep_packed=False)
            cache.commit([(slot, first)])
            for at in range(first, first + 9, portion):
                n = portion
                cache.grow([(slot, at + n, at)])
                cache.sync()
                dest = torch.tensor(cache.destination_rows([slot], [at], [n])[0], device=DEV)
                packed = torch.cat([rq[at:at + n].reshape(n, -1), rk[at:at + n].reshape(n, -1),
                                    rv[at:at + n].reshape(n, -1)], dim=1).contiguous()
                qn, _, _ = ops.qkv_bias_store(packed, None, H, G, d, dv, kv=cache.view(0), dest_rows=dest, keep_packed=False)
                cache.commit([(slot, at + n)])
                slots_t = torch.tensor([slot], dtype=torch.int32, device=DEV)
                lens = torch.tensor([at + n], dtype=torch.int32, device=DEV)
                if portion == 1:
                    out = ops.attention_decode(qn, cache.view(0), slots_t, lens, 512, 1.0, window)
                else:
                    out = ops.attention_extend(qn, cache.view(0), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                               torch.zeros(n, dtype=torch.int32, device=DEV),
                                               torch.arange(at, at + n, dtype=torch.int32, device=DEV), slots_t, lens, n, 1.0,
                                               window)
                rows.append(out.reshape(n, H, dv))
            got = torch.cat(rows).cpu().double()
            assert float((got - ref[first:first + 9]).abs().max()) <= tol * 9.0, f"portions of {portion}, key {spike}"


# --------------------------------------------------------------------------- the block's own kernels
def test_token_shift_reads_the_row_before_and_keeps_the_last():
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(11)
    W = 72
    for dtype in (torch.float32, torch.bfloat16):
        mix = torch.rand(W, generator=gen)
        seqs = [torch.randn(n, W, generator=gen).to(dtype) for n in (23, 9)]
        want = [P.token_shift(s.double(), mix.double()) for s in seqs]
        last = torch.full((4, 1, W), 3.0, dtype=torch.float32, device=DEV)
        last[[2, 0]] = 0.0
        slots = torch.tensor([2, -1, 0], dtype=torch.int32, device=DEV)
        got, at = [[], []], [0, 0]
        for n0, n1 in ((1, 2), (5, 1), (17, 6)):
            pad = torch.ones(3, W, dtype=dtype)
            h = torch.cat([seqs[0][at[0]:at[0] + n0], pad, seqs[1][at[1]:at[1] + n1]]).to(DEV).contiguous()
            cu = torch.tensor([0, n0, n0 + 3, n0 + 3 + n1], dtype=torch.int32, device=DEV)
            seq_of = torch.tensor([0] * n0 + [1] * 3 + [2] * n1, dtype=torch.int32, device=DEV)
            out = ops.token_shift(h, mix.to(DEV), last, cu, seq_of, slots).cpu().double()
            got[0].append(out[:n0])
            got[1].append(out[n0 + 3:])
            at = [at[0] + n0, at[1] + n1]
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        for b in range(2):
            assert float((torch.cat(got[b]) - want[b]).abs().max()) <= tol * float(want[b].abs().max())
        assert float((last[[1, 3]] - 3.0).abs().max()) == 0.0
        assert torch.equal(last[2, 0].cpu(), seqs[0][-1].float()) and torch.equal(last[0, 0].cpu(), seqs[1][-1].float())


def test_scaled_add_row_gate_gelu_gate_and_tanh():
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(12)
    x, y, f = torch.randn(7, 40, generator=gen), torch.randn(7, 40, generator=gen), torch.randn(40, generator=gen)
    got = ops.scaled_add_(x.clone().to(DEV), y.to(DEV), f.to(DEV)).cpu().double()
    assert float((got - (x.double() + f.double() * y.double())).abs().max()) < 1e-6
    for dtype, width in ((torch.float32, 40), (torch.bfloat16, 40), (torch.bfloat16, 1030)):
        xs, ys, fs = torch.randn(7, width, generator=gen), torch.randn(7, width, generator=gen), torch.randn(width, generator=gen)
        g = (1.0 + 0.2 * torch.randn(width, generator=gen)).to(dtype)
        stream = xs.clone().to(DEV)
        normed = ops.scaled_add_norm_(stream, ys.to(DEV), fs.to(DEV), g.to(DEV), 1e-5, dtype).cpu().double()
        summed = xs.double() + fs.double() * ys.double()
        assert float((stream.cpu().double() - summed).abs().max()) < 1e-6
        want = P.unit_rms(summed, 1e-5) * g.double()
        assert float((normed - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2)
    for dtype in (torch.float32, torch.bfloat16):
        h, w = torch.randn(7, 24, generator=gen).to(dtype), torch.randn(24, generator=gen)
        got = ops.row_gate_(y.clone().to(DEV), h.to(DEV), w.to(DEV)).cpu().double()
        want = y.double() * torch.sigmoid(h.double() @ w.double())[:, None]
        assert float((got - want).abs().max()) < 1e-5
    both = torch.randn(5, 48, generator=gen) * 3.0
    for block in (8, 24):
        gate = both.reshape(5, 24 // block, 2, block)[:, :, 0].reshape(5, 24).double()
        up = both.reshape(5, 24 // block, 2, block)[:, :, 1].reshape(5, 24).double()
        want = P.gelu_tanh(gate) * up
        got = ops.gelu_tanh_mul(both.to(DEV), block).cpu().double()
        assert float((got - want).abs().max()) < 1e-5
        got = ops.gelu_tanh_mul(both.to(DEV), block, out_dtype=torch.bfloat16).cpu().double()
        assert float((got - want).abs().max()) < 1e-2 * float(want.abs().max())
    got = ops.tanh_columns(both.to(DEV), 5, 11, torch.float32).cpu().double()
    assert float((got - torch.tanh(both.double()[:, 5:16])).abs().max()) < 1e-6


@pytest.mark.parametrize("T,E,top,groups,scale", [(5, 6, 2, (3, 2), 2.5), (70, 8, 4, (4, 3), 1.5), (3, 4, 4, None, 1.0),
                                                  (300, 24, 3, (6, 2), 0.5), (9, 5, 1, (5, 1), 3.0)])
def test_router_renormalizes_with_its_epsilon_and_scales(T, E, top, groups, scale):
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(T + E)
    width = 64
    x = torch.randn(T, width, generator=gen)
    w = torch.randn(E, width, generator=gen) * 0.3
    f = dict(router=dict(experts=E, top=top, scale=scale))
    if groups is not None:
        f["router"]["groups"] = dict(count=groups[0], keep=groups[1])
    ids, weights = P.route(x.double(), f, {"router": w.double()}, "")
    scoring = ops.Scoring(None, groups[0] if groups else 1, groups[1] if groups else 1, True, 1e-20, scale)
    got_ids, got_w = ops.moe_router(x.to(DEV), w.to(DEV), None, top, scoring)
    order = got_ids.cpu().long().sort(-1)
    want = ids.sort(-1)
    assert torch.equal(order.values, want.values)
    assert float((got_w.cpu().double().gather(1, order.indices) - weights.gather(1, want.indices)).abs().max()) < 1e-5
    logits = (x @ w.T).to(DEV).contiguous()
    got_ids, got_w = ops.moe_route_scored(logits, top, scoring)
    order = got_ids.cpu().long().sort(-1)
    assert torch.equal(order.values, want.values)
    assert float((got_w.cpu().double().gather(1, order.indices) - weights.gather(1, want.indices)).abs().max()) < 1e-5


def test_norm_with_one_number_for_a_weight(engine):
    from llama_rs_metal_b200.parts.norm import RMSNorm
    from llama_rs_metal_b200.runtime import Runtime

    class Ctx:
        runtime = Runtime(engine.device, torch.float32)

        @staticmethod
        def take_pending():
            return None
    norm = RMSNorm(72, 1e-5, scalar=True)
    assert norm.tensors()["weight"].shape == ()
    norm.bind({"weight": torch.tensor(1.7, device=DEV)}, Ctx.runtime)
    x = torch.randn(6, 72, generator=torch.Generator().manual_seed(1))
    got = norm.forward(x.to(DEV), Ctx).cpu().double()
    assert float((got - P.scalar_norm(x.double(), torch.tensor(1.7, dtype=F64), 1e-5)).abs().max()) < 1e-5

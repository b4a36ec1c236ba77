"""The Norevik decoder through the engine, compared with the plain implementation (plain_norevik.py).

Model level, on three tiny configurations (helpers.NOREVIK): whole prompts, the residual stream
layer by layer, prefill against token-by-token decoding in unequal batches, portions down to two
tokens, company in the batch, slots and pages that are freed and used again, long decoding through
captured steps, greedy generation through Session.generate, a replay through bin/trace_run,
configurations drawn at random. Mechanism level, on models of one layer whose weights are made so
that a fault shows: each mixer and each feed-forward alone, a far key that must win and a sink that
must take its share (in a prompt, in portions, in decoding, across a page's border), rotation of
neighbouring pairs far from the start, a state-space head that remembers its first token, the
convolution's tail under portions of one and two tokens, the matrix memory's first tokens (a
maximum that starts at zero) and saturated gates, routing with negative choice scores inside kept
groups, identity experts, and the norm behind a sublayer.
"""
import numpy as np
import pytest
import torch

import helpers
import plain_norevik as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ["N1", "N2", "N3"]
F64 = torch.float64


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> folder; the bfloat16 comparisons run on the folder with steady routing."""
    out = {}
    for n in NAMES:
        out[n, "float32"] = helpers.make_norevik_dir(str(tmp_path_factory.mktemp(f"norevik_{n}")), n)
        out[n, "bfloat16"] = helpers.make_norevik_dir(str(tmp_path_factory.mktemp(f"norevik_{n}_steady")), n,
                                                      steady_routing=True)
    return out


@pytest.fixture(scope="module")
def plain(folders):
    return {key: P.read_model(path) for key, path in folders.items()}


class Ref:
    """Reference logits [rows, vocab] with, per row, how far the plain model's logits move when only
    the inputs of its sublayers and of its head are rounded to bfloat16, or moved at random by up to
    2^-7 of their size (the largest of three such trials, as a fraction of the largest logit).
    Indexing keeps the two together."""

    def __init__(self, logits, moved):
        self.logits, self.moved = np.asarray(logits), np.asarray(moved)

    def __getitem__(self, key):
        return Ref(self.logits[key], self.moved[key])

    def numpy(self):
        return self.logits

    @staticmethod
    def stack(refs):
        return Ref(np.stack([r.logits for r in refs]), np.stack([r.moved for r in refs]))


_REFS = {}


def reference(plain, which, tokens):
    """The plain implementation's logits for `tokens` on the folder of `which` = (name, dtype)."""
    key = (which, tuple(tokens))
    if key not in _REFS:
        config, tensors = plain[which]
        logits = P.forward(config, tensors, tokens)
        gen = torch.Generator().manual_seed(len(tokens))

        def jitter(t):   # the size of a bfloat16 rounding on top of an input that is itself half a percent off
            return t * (1.0 + 2.0 ** -7 * (2.0 * torch.rand(t.shape, generator=gen, dtype=F64) - 1.0))
        moved = torch.zeros(len(tokens), dtype=F64)
        for seen in (lambda t: t.to(torch.bfloat16).to(F64), jitter, jitter):
            other = P.forward(config, tensors, tokens, seen=seen)
            moved = torch.maximum(moved, (other - logits).abs().max(dim=-1).values / logits.abs().max())
        _REFS[key] = Ref(logits.numpy(), moved.numpy())
    return _REFS[key]


# Allowed error of a row of logits as a fraction of the largest reference logit. float32: sums in
# another order than the plain implementation's float64, and recurrences that feed back what they
# add up. bfloat16: activations are rounded between kernels; a fault of any mechanism is far above.
# A norm stands behind every sublayer, so a row whose sublayer output nearly cancels is scaled up
# again together with its rounding: in these tiny random models such a row's error is tens of times
# the median's in both types (in float32 still below the tolerance). Against a Ref, a bfloat16 row
# may therefore be off by three times what the rounding of the inputs alone moves that row of the
# plain model, where that is more than the tolerance. Against plain arrays one row in twenty may be
# up to six times over while the median stays below a third; `strict` compares every row.
TOLERANCE = {"float32": 5e-5, "bfloat16": 5e-2}


def close(got, ref, dtype, what, factor=1.0, strict=False):
    moved = None
    if isinstance(ref, Ref):
        ref, moved = ref.logits, np.atleast_1d(ref.moved)
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got.reshape(1, -1), ref.reshape(1, -1)
    assert got.shape == ref.shape and np.all(np.isfinite(got)), what
    err = np.abs(got - ref).max(axis=-1) / max(float(np.abs(ref).max()), 1e-30)
    allowed = np.full(len(err), factor * TOLERANCE[dtype])
    if moved is not None and dtype == "bfloat16":
        allowed = np.maximum(allowed, 3.0 * moved)
    worst = int((err / allowed).argmax())
    report = (f"{what}: row {worst} off by {err[worst]:.3e} of the largest logit (allowed {allowed[worst]:.0e}); "
              f"first such row {int(np.argmax(err > allowed))}; {int((err > allowed).sum())} of {len(err)} rows over; "
              f"median {np.median(err):.3e}")
    if dtype == "bfloat16" and moved is None and not strict and len(err) >= 8:
        assert (err > allowed).sum() <= max(1, len(err) // 20) and err[worst] <= 6 * allowed[worst] \
            and np.median(err) <= allowed[worst] / 3, report
    else:
        assert err[worst] <= allowed[worst], report


def vocab_of(name):
    return helpers.NOREVIK[name]["config"]["vocab"]


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


# --------------------------------------------------------------------------- whole prompts
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
def test_every_layer_matches_the_plain_residual_stream(engine, folders, plain, name):
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
    assert len(seen) == len(streams)
    for i, (got, want) in enumerate(zip(seen, streams)):
        err = float((got[:len(tokens)] - want).abs().max() / want.abs().max())
        assert err < 2e-5, f"{name}: the stream after layer {i} is off by {err:.2e}"


# --------------------------------------------------------------------------- prefill against decoding
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_decoding_in_an_unequal_batch(engine, folders, plain, name, dtype):
    """Prompts of unequal lengths in one step, then one token each per step, past a page's border;
    the shorter requests end earlier and the batch shrinks."""
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
@pytest.mark.parametrize("name", ["N1", "N2"])
def test_a_prompt_geometry_that_comes_again_is_captured_and_replayed(engine, folders, plain, name, dtype):
    """The same shape of batch four times with other tokens, in slots that were used before: states,
    tails and running maxima must start from zero each time, also under a captured graph's replay."""
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
    close(np.stack(following), Ref.stack(expected), dtype, f"{name}: the token after each prompt")
    runner.check_device_status()


@pytest.mark.parametrize("sizes", [[2], [3, 64, 5], [1, 70, 2], [64], [17]])
@pytest.mark.parametrize("name", ["N1", "N2"])
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
    name = "N2"
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
    limit = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(alone - together).max() <= limit * np.abs(alone).max()
    close(together, reference(plain, (name, dtype), mine), dtype, "in company")


def test_a_freed_slot_and_its_pages_start_from_nothing(engine, folders, plain):
    """States, tails and running maxima of a slot are cleared when it is taken again, and the pages
    a sequence gave back hold another sequence's latents when they are used again."""
    name = "N1"
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
    """300 tokens one by one from the very first: several pages pass by, the states are carried
    through hundreds of captured steps."""
    name = "N1"
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    tokens = helpers.random_tokens(9, 300, vocab_of(name))
    ref = reference(plain, (name, dtype), tokens)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens]
    close(np.concatenate(rows), ref, dtype, "token by token from the start", factor=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_session(engine, folders, plain, dtype):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    name = "N2"
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
    name = "N1"
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
        ref = Ref.stack([refs[rid.split(":")[-1]][pos] for rid, pos in rows])
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
            return helpers._plain_ff(int(pick(24, 64, 100)))
        count = int(pick(1, 2, 3))
        size = int(pick(1, 2, 4))                       # outputs per group
        outputs = count * size
        identity = int(rng.integers(0, min(3, outputs)))
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, keep * size + 1))
        return helpers._experts(int(pick(8, 24, 40)), outputs - identity, top, identity=identity,
                                groups=(count, keep) if rng.integers(3) else None, shared=pick(None, 16, 48))
    width = int(pick(40, 64, 88, 136))
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = pick("mamba2", "latent_attention", "mlstm")
        if kind == "mamba2":
            groups = int(pick(1, 2, 3))
            heads, vdim = groups * int(pick(1, 2)), int(pick(4, 8, 20, 64))
            parts = [p for p in (1, 2, 3, 4, 5) if (heads * vdim) % p == 0]
            mixer = helpers._ssm(heads, vdim, int(pick(4, 16, 24, 64, 128)), groups, int(pick(1, 2, 4, 5)), int(pick(*parts)))
        elif kind == "latent_attention":
            mixer = helpers._sink_latent(int(pick(1, 2, 5)), int(pick(4, 16, 24)), int(pick(2, 8, 16)), int(pick(8, 12, 32)),
                                         int(pick(8, 24, 40)), float(pick(0.1, 0.4)), float(pick(30.0, 10000.0)))
        else:
            mixer = helpers._memory(int(pick(1, 2, 3)), int(pick(4, 16, 40)), int(pick(3, 8, 16, 63)), float(pick(2.0, 10.0, 30.0)))
        layers.append(dict(type=kind, mixer=mixer, mlp=feed_forward()))
    config = dict(architecture="Norevik", vocab=int(pick(97, 256, 333)), width=width, norm=dict(eps=float(pick(1e-6, 1e-4))),
                  embedding=dict(scale=float(pick(0.5, 1.0, 6.0))), layers=layers)
    return dict(config=config, seed=2000 + seed, std=float(pick(0.08, 0.15)))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(engine, tmp_path, seed):
    """Other sizes, orders of layers and constants than the fixed configurations: a prompt whole,
    then tokens one by one, a second sequence beside it in portions."""
    spec = drawn_configuration(seed)
    for dtype in ("float32", "bfloat16"):
        folder = helpers.make_norevik_dir(str(tmp_path / dtype), spec, steady_routing=dtype == "bfloat16")
        plain = {("drawn", dtype): P.read_model(folder)}
        V = spec["config"]["vocab"]
        a, b = helpers.random_tokens(seed, 150, V), helpers.random_tokens(seed + 50, 100, V)
        ref_a, ref_b = reference(plain, ("drawn", dtype), a), reference(plain, ("drawn", dtype), b)
        _REFS.pop((("drawn", dtype), tuple(a)))          # the next seed's folder is another model
        _REFS.pop((("drawn", dtype), tuple(b)))
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

"""The Tarupel decoder as a plan of parts.

Every layer is pre-norm with norms whose weight is one number: x <- x + m * s1 * mixer(shift(norm1(x))),
then x <- x + m * s2 * ff(norm2(x)) (or nothing), with one factor m for the model, stored factors s1,
s2 per channel, and `shift` the mix of a token's normalized row with the previous token's. Three
kinds of mixer: `general_delta`, a generalized delta rule with a decay and a removal rate per key
channel; `attention`, grouped-query attention with biased projections, a short convolution on q, k
and v, a split-half rotation of part of each head, unit RMS per head behind it, and keys visible
inside the query's chunk of positions; `attention_2`, grouped-query attention with biased
projections, a weighted RMS norm over the whole query row and the whole key row, a rotation of
neighbouring dimensions, and a sliding window. The feed-forward is dense (a GELU gate, tanh form)
or a mixture of gated SiLU experts: scores from the softmax over all router outputs, the choice
inside the best groups of neighbours, the chosen scores renormalized and scaled, and a shared
expert under a sigmoid gate per token. A run of layers may loop: it runs several times in a row with
the same weights, every pass with cache entries of its own; before each pass but the first the
embedding's output is added to the stream, and before each pass a vector of the table `loop.step`.
The embedding is scaled; the head is a matrix of its own behind the model's last norm.

Checkpoint names: `embed`, `head`, `final.norm`, `loop.step`, and per layer i `l<i>.norm1`,
`l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`, `l<i>.shift`, `l<i>.mix.*`, `l<i>.mlp.*`; an expert's tensors are
`l<i>.mlp.e<j>.{gate,up,down}`, the shared expert's `l<i>.mlp.shared.*` with its gate `.sg`; a bias is
its matrix's name + `.b`, a convolution's taps + `.conv`, a row norm's weight + `.norm`.
"""
from __future__ import annotations

import math

from ..config.tarupel import TarupelConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20          # the design names no limit
DECAY_SCALE = math.exp(-0.5)     # the decay is exp(-DECAY_SCALE * sigmoid(.)): never below exp(-e^-1/2)
UNIT_EPS = 1e-6                  # under the root of the unit key
RENORMALIZE_EPS = 1e-20          # added to the sum the chosen scores are divided by


def _general_delta(config: TarupelConfig, m, p: str) -> PartSpec:
    names = {f"{own}_proj.weight": p + own for own in ("r", "k", "v", "g", "a", "o")}
    names.update({"a_proj.bias": p + "a.b", "d_down.weight": p + "w1", "d_up.weight": p + "w2", "d_bias": p + "w0",
                  "norm.weight": p + "norm"})
    return PartSpec("generalized_delta_rule", dict(
        hidden_size=config.width, num_heads=m.heads, head_dim=m.dim, value_dim=m.dim, eps=config.eps,
        decay_scale=DECAY_SCALE, decay_rank=m.decay_rank, unit_eps=UNIT_EPS), names=names)


def _attention_names(p: str) -> dict:
    names = {f"{own}_proj.weight": p + own for own in ("q", "k", "v", "o")}
    names.update({f"{own}_proj.bias": p + own + ".b" for own in ("q", "k", "v")})
    return names


def _rotation(m, adjacent: bool):
    if not m.rot_dims:
        return None
    return PartSpec("rope", dict(head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base, adjacent_pairs=adjacent))


def _chunked_attention(config: TarupelConfig, m, p: str) -> PartSpec:
    names = _attention_names(p)
    names.update({f"{own}_conv.weight": p + own + ".conv" for own in ("q", "k", "v")})
    return PartSpec("attention", dict(
        hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
        position=_rotation(m, False), scale=m.scale, bias=True, conv_taps=m.conv, head_norm_eps=config.eps,
        chunk=m.span), names=names)


def _window_attention(config: TarupelConfig, m, p: str) -> PartSpec:
    names = _attention_names(p)
    names.update({"q_norm.weight": p + "q.norm", "k_norm.weight": p + "k.norm"})
    return PartSpec("attention", dict(
        hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
        position=_rotation(m, True), scale=m.scale, bias=True, row_norm_eps=config.eps, window=m.span), names=names)


MIXERS = {"general_delta": _general_delta, "attention": _chunked_attention, "attention_2": _window_attention}


def _gated_names(p: str) -> dict:
    return {"gate_proj.weight": p + "gate", "up_proj.weight": p + "up", "down_proj.weight": p + "down"}


def _feed_forward(config: TarupelConfig, f, p: str) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("gated_mlp", dict(hidden_size=config.width, intermediate_size=f.ff, activation="gelu_tanh"),
                        names=_gated_names(p))
    names = {"router.weight": p + "router"}
    for e in range(f.experts):
        names.update({f"experts.{e}.{own}": full for own, full in _gated_names(f"{p}e{e}.").items()})
    shared = None
    if f.shared_ff is not None:
        shared = PartSpec("gated_mlp", dict(hidden_size=config.width, intermediate_size=f.shared_ff, activation="silu"))
        names.update({"shared." + own: full for own, full in _gated_names(p + "shared.").items()})
        names["shared.gate"] = p + "shared.sg"
    return PartSpec("moe", dict(
        hidden_size=config.width, intermediate_size=f.ff, num_experts=f.experts, top=f.top, activation="silu",
        router_bias=False, scoring="softmax_all", correction=False, groups=f.groups, renormalize=True,
        renormalize_eps=RENORMALIZE_EPS, weight_scale=f.scale, shared=shared, shared_gate=shared is not None),
        names=names)


def layer_runs(config: TarupelConfig):
    """[(layer, pass number or None)] in the order the layers run: the pass number stands at the
    first layer of each pass of the looped run."""
    n = len(config.layers)
    if not config.loops:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(config.loop_start)]
    for t in range(config.loop_times):
        runs += [(i, t if i == config.loop_start else None) for i in range(config.loop_start, config.loop_stop)]
    return runs + [(i, None) for i in range(config.loop_stop, n)]


def tarupel_plan(config: TarupelConfig) -> ModelPlan:
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", dict(size=config.width, eps=config.eps, scalar=True), names={"weight": name})

    layers = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        parts = dict(mixer=MIXERS[layer.kind](config, layer.mixer, p + "mix."), mixer_norm=norm(p + "norm1"))
        names = {"mixer_scale": p + "ls1", "shift": p + "shift"}
        if layer.mlp is not None:
            parts.update(feed_forward=_feed_forward(config, layer.mlp, p + "mlp."), feed_forward_norm=norm(p + "norm2"))
            names["feed_forward_scale"] = p + "ls2"
        layers.append(LayerSpec("scaled_pre_norm" if layer.mlp is not None else "scaled_pre_norm_mixer", parts=parts,
                                options=dict(hidden_size=config.width, residual_mult=config.residual_mult,
                                             layer_scale=True, token_shift=True), names=names))
    schedule = tuple(ScheduleEntry(layer=i, cache=n, add_offset=t, add_embedding=t is not None and t > 0)
                     for n, (i, t) in enumerate(layer_runs(config)))
    return ModelPlan(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), schedule=schedule,
        final_norm=norm("final.norm"), head_name="head",
        embedding_scale=config.embedding_scale if config.embedding_scale != 1.0 else None,
        stream_offsets=("loop.step", config.loop_times) if config.loops else None)


register_architecture("Tarupel", TarupelConfig, tarupel_plan, model_types=("tarupel",))

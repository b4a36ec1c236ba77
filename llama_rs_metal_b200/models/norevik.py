"""The Norevik decoder as a plan of parts.

Every layer has a norm only behind each sublayer, and the sublayers read the residual stream
itself: x <- x + norm_1(mixer(x)), then x <- x + norm_2(feed_forward(x)) (or nothing); the norms
are layer norms with weight and bias. Three kinds of mixer: `mamba2`, a state-space mixer with a
scalar decay per head and token behind a short convolution, gated and then normalized part by
part; `latent_attention`, causal attention whose keys and values are unfolded from a small cached
latent, with rotary positions (neighbouring dimensions paired) on a key part all heads share, a
per-head sink in the softmax and a sigmoid gate per head and value dimension; `mlstm`, a matrix
memory with capped exponential gates under a running maximum. The feed-forward is dense (squared
ReLU, no gate) or a mixture of gated SiLU experts: scores from the softmax over all router
outputs, the choice made on corrected scores within the best groups of neighbours, weights not
renormalized, identity experts without matrices, and a shared expert for every token. The
embedding is scaled; the head is a matrix of its own behind the model's last norm.

Checkpoint names: `embed`, `head`, `final.norm` (+ `.b`), and per layer i `l<i>.norm1`, `l<i>.norm2`
(each + `.b` for the bias), `l<i>.mix.*`, `l<i>.mlp.*`; an expert's tensors are `l<i>.mlp.e<j>.{gate,
up,down}`, the shared expert's `l<i>.mlp.shared.*`; a bias is its matrix's or table's name + `.b`.
"""
from __future__ import annotations

from ..config.norevik import NorevikConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20  # the design names no limit
FLOOR_EPS = 1e-6         # added to the matrix memory's denominator


def _state_space(config: NorevikConfig, m, p: str) -> PartSpec:
    names = {"in_proj.weight": p + "in", "conv.weight": p + "conv", "conv.bias": p + "conv.b", "dt_bias": p + "dt_bias",
             "A_log": p + "A_log", "D": p + "D", "norm.weight": p + "norm", "o_proj.weight": p + "o"}
    return PartSpec("state_space_duality", dict(
        hidden_size=config.width, num_heads=m.heads, value_dim=m.vdim, state_size=m.state, groups=m.groups,
        conv_taps=m.conv, norm_parts=m.norm_groups, eps=config.eps), names=names)


def _latent_attention(config: NorevikConfig, m, p: str) -> PartSpec:
    names = {"q_proj.weight": p + "q", "kv_down.weight": p + "dkv", "kv_down.norm": p + "dkv.norm",
             "k_up.weight": p + "uk", "v_up.weight": p + "uv", "sinks": p + "sink", "gate.weight": p + "g",
             "o_proj.weight": p + "o"}
    position = PartSpec("rope", dict(head_dim=m.rot_dim, rotary_dim=m.rot_dim, theta=m.rot_base, adjacent_pairs=True))
    return PartSpec("latent_attention", dict(
        hidden_size=config.width, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
        kv_rank=m.kv_rank, q_rank=None, eps=config.eps, scale=m.scale, position=position, window=None,
        sinks=True, gate="per_dim"), names=names)


def _matrix_memory(config: NorevikConfig, m, p: str) -> PartSpec:
    names = {"q_proj.weight": p + "q", "k_proj.weight": p + "k", "v_proj.weight": p + "v", "g_proj.weight": p + "g",
             "i_gate.weight": p + "i", "i_gate.bias": p + "i.b", "f_gate.weight": p + "f", "f_gate.bias": p + "f.b",
             "norm.weight": p + "norm", "o_proj.weight": p + "o"}
    return PartSpec("matrix_memory", dict(
        hidden_size=config.width, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, gate_cap=m.gate_cap,
        eps=config.eps, floor_eps=FLOOR_EPS), names=names)


MIXERS = {"mamba2": _state_space, "latent_attention": _latent_attention, "mlstm": _matrix_memory}


def _gated_names(p: str) -> dict:
    return {"gate_proj.weight": p + "gate", "up_proj.weight": p + "up", "down_proj.weight": p + "down"}


def _feed_forward(config: NorevikConfig, f, p: str) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("mlp", dict(hidden_size=config.width, intermediate_size=f.ff, activation="relu_squared"),
                        names={"up_proj.weight": p + "up", "down_proj.weight": p + "down"})
    names = {"router.weight": p + "router", "router.correction": p + "correction"}
    for e in range(f.experts):
        names.update({f"experts.{e}.{own}": full for own, full in _gated_names(f"{p}e{e}.").items()})
    shared = None
    if f.shared_ff is not None:
        shared = PartSpec("gated_mlp", dict(hidden_size=config.width, intermediate_size=f.shared_ff, activation="silu"))
        names.update({"shared." + own: full for own, full in _gated_names(p + "shared.").items()})
    return PartSpec("moe", dict(
        hidden_size=config.width, intermediate_size=f.ff, num_experts=f.experts, top=f.top, activation="silu",
        router_bias=False, scoring="softmax_all", correction=True, groups=f.groups, renormalize=False,
        identity=f.identity, shared=shared), names=names)


def norevik_plan(config: NorevikConfig) -> ModelPlan:
    def norm(name: str) -> PartSpec:
        return PartSpec("layer_norm", dict(size=config.width, eps=config.eps), names={"weight": name, "bias": name + ".b"})

    layers, schedule = [], []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        parts = dict(mixer=MIXERS[layer.kind](config, layer.mixer, p + "mix."), mixer_post_norm=norm(p + "norm1"))
        if layer.mlp is not None:
            parts.update(feed_forward=_feed_forward(config, layer.mlp, p + "mlp."),
                         feed_forward_post_norm=norm(p + "norm2"))
        layers.append(LayerSpec("post_norm" if layer.mlp is not None else "post_norm_mixer", parts=parts))
        schedule.append(ScheduleEntry(layer=i, cache=i))
    return ModelPlan(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("final.norm"), head_name="head",
        embedding_scale=config.embedding_scale if config.embedding_scale != 1.0 else None)


register_architecture("Norevik", NorevikConfig, norevik_plan, model_types=("norevik",))

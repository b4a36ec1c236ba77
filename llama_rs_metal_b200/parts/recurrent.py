"""Mixers whose memory is a matrix of fixed size per sequence and head.

Both keep S [head_dim, value_dim] in float32 per (sequence, head) in the cache's state storage,
update it token by token and read it out with the query (csrc/recurrent_scan.cu):

* `retention`: S <- a_h S + k v^T with one fixed decay a_h per head, no softmax and no
  denominator; rotary positions on q and k; the read-out is normalized per head and gated.
* `gated_delta_rule`: S <- diag(g) S; S <- S + k (b (v - S^T k))^T with decays g per key channel
  and step sizes b computed from the input; q, k, v pass a short causal convolution first.

* `generalized_delta_rule`: S <- diag(g) S - (a * u) (u^T S) + k v^T with a decay g and a removal rate
  a per key channel, both computed from the input, u the unit key, both terms reading the old S
  (csrc/general_delta.cu prepares its inputs).

A third keeps one number per channel (csrc/gated_recurrence.cu):

* `gated_linear_recurrence`: S <- a S + sqrt(1 - a^2) (i u) with a decay a and an input gate i
  computed from the input, block by block of channels; u passes a short causal convolution first.

Two more decay S by one number per head and token, S <- a_t S + k (b_t v)^T, on the same scan
(csrc/scalar_gated_state.cu prepares their inputs and reads them out):

* `state_space_duality`: a_t = exp(-exp(A_log_h) dt_t), b_t = dt_t with a step size dt computed from
  the input; x, B (the keys) and C (the queries) pass a short causal convolution first; the read-out
  is gated, then normalized part by part.
* `matrix_memory`: exponential input and forget gates under a running maximum, a normalizer n
  beside S, the read-out divided by max(|n . q|, exp(-m)).

A step of any size (a prompt, a portion, one token) runs the same scan from the state the
steps before left, so nothing depends on how a sequence was cut into steps.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..errors import InvalidError, UnsupportedError
from ..kernels import ops
from ..registry import POSITION_ENCODINGS, build_part, register_mixer
from ..weights.loader import TensorSpec
from .base import CompositeRequest, Mixer, PartSpec, StateRequest
from .linear import LinearWeight


def _needs_own_state(ctx) -> None:
    if not ctx.entry.writes_cache:
        raise UnsupportedError("a mixer with a fixed-size state cannot read another layer's state")


@register_mixer("retention")
class Retention(Mixer):
    """o_t = S_t^T q_t, S_t = a_h S_(t-1) + k_t v_t^T per head, with q and k rotated by position
    (`position`: a rotary PartSpec, or None) and k multiplied by `key_scale` (default
    head_dim^-1/2) after the rotation. Each head's o is divided by its root mean square
    (`eps`, no weight), the heads are concatenated, multiplied by silu(W_g x) and projected."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float],
                 eps: float, position: Optional[PartSpec] = None, key_scale: Optional[float] = None,
                 output_scale: float = 1.0):
        if num_heads <= 0 or head_dim <= 0 or value_dim <= 0 or len(decay) != num_heads:
            raise InvalidError("retention needs one decay per head")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.decay = [float(a) for a in decay]
        self.eps, self.output_scale = float(eps), float(output_scale)
        self.key_scale = float(key_scale) if key_scale is not None else head_dim ** -0.5
        self.position = build_part(POSITION_ENCODINGS, position, "position encoding") \
            if position is not None else None
        self.fused: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None
        self.head_decay: Optional[torch.Tensor] = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def tensors(self) -> Dict[str, TensorSpec]:
        qk, v, h = self.num_heads * self.head_dim, self.num_heads * self.value_dim, self.hidden_size
        return {"q_proj.weight": TensorSpec((qk, h)), "k_proj.weight": TensorSpec((qk, h)),
                "v_proj.weight": TensorSpec((v, h)), "g_proj.weight": TensorSpec((v, h)),
                "o_proj.weight": TensorSpec((h, v))}

    def bind(self, weights, runtime) -> None:
        # one matrix q | k | v | g: each output is the same dot product as with separate matrices
        self.fused = LinearWeight(torch.cat([weights["q_proj.weight"], weights["k_proj.weight"],
                                             weights["v_proj.weight"], weights["g_proj.weight"]], dim=0))
        self.out = LinearWeight(weights["o_proj.weight"])
        self.head_decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        if self.position is not None:
            self.position.bind({}, runtime)
            if self.position.rotary_table() is None:
                raise UnsupportedError("retention rotates q and k by a rotary table or not at all")

    def cache_request(self):
        return StateRequest((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        H, d, dv = self.num_heads, self.head_dim, self.value_dim
        projected = self.fused(x)
        inv_freq, rotary = self.position.rotary_table() if self.position is not None else (None, 0)
        q, k, v = ops.retention_prepare(projected, 0, H * d, 2 * H * d, H, d, dv, ctx.positions, inv_freq, rotary,
                                        self.key_scale)
        o = ops.linear_state_scan(q, k, v, cache.state, ctx.cu_seqlens, ctx.slots, head_decay=self.head_decay)
        mixed = ops.head_norm_gate(o, self.eps, projected.dtype, gate=projected, gate_column=2 * H * d + H * dv,
                                   gate_act=ops.GATE_SILU, out_scale=self.output_scale)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """q = W_q x, k = W_k x (kv_heads x head_dim), v = W_v x (heads x value_dim); each passes a
    causal convolution of `conv_taps` taps per channel (no bias, zeros before the start) and SiLU;
    q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times head_dim^-1/2.
    b = sigmoid(W_b x) per head; g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias)) per head
    and key channel. Per head, with q/k head h // (heads / kv_heads):
        S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q.
    o is divided by its root mean square over value_dim (`eps`), multiplied by a weight shared by
    the heads and by sigmoid(W_g2 (W_g1 x)), then projected. The inner ranks of the two low-rank
    products are the checkpoint's (`decay_rank`, `gate_rank` None) unless given.
    State: S in float32 and the last conv_taps - 1 convolution inputs of every channel."""

    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 conv_taps: int, eps: float, decay_rank: Optional[int] = None, gate_rank: Optional[int] = None,
                 unit_eps: float = 1e-6, output_scale: float = 1.0):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads or conv_taps <= 0:
            raise InvalidError("gated delta rule: heads must be a multiple of key heads, and taps positive")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.conv_taps = head_dim, value_dim, conv_taps
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.eps, self.unit_eps, self.output_scale = float(eps), float(unit_eps), float(output_scale)
        self.channels = 2 * num_kv_heads * head_dim + num_heads * value_dim
        self.fused: Optional[LinearWeight] = None
        self.low: Optional[LinearWeight] = None
        self.high: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        H, G, d, dv, h, n = (self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size,
                             self.conv_taps)
        return {"q_proj.weight": TensorSpec((G * d, h)), "k_proj.weight": TensorSpec((G * d, h)),
                "v_proj.weight": TensorSpec((H * dv, h)), "q_conv.weight": TensorSpec((G * d, n)),
                "k_conv.weight": TensorSpec((G * d, n)), "v_conv.weight": TensorSpec((H * dv, n)),
                "b_proj.weight": TensorSpec((H, h)), "A_log": TensorSpec((H,)), "dt_bias": TensorSpec((H * d,)),
                "a_down.weight": TensorSpec((self.decay_rank, h)), "a_up.weight": TensorSpec((H * d, self.decay_rank)),
                "g_down.weight": TensorSpec((self.gate_rank, h)), "g_up.weight": TensorSpec((H * dv, self.gate_rank)),
                "norm.weight": TensorSpec((dv,)), "o_proj.weight": TensorSpec((h, H * dv))}

    def bind(self, weights, runtime) -> None:
        H, d, dv = self.num_heads, self.head_dim, self.value_dim
        a_down, a_up, g_down, g_up = (weights[n + ".weight"] for n in ("a_down", "a_up", "g_down", "g_up"))
        ra, rg = a_down.shape[0], g_down.shape[0]
        if a_up.shape[1] != ra or g_up.shape[1] != rg:
            raise InvalidError("gated delta rule: the two halves of a low-rank product disagree on its rank")
        # q | k | v | b in one product; the two low-rank products share a first product
        # [a_down; g_down] and a second one with the block matrix [[a_up, 0], [0, g_up]]: the zero
        # blocks add exact zeros, so every output is the sum it would be with separate matrices
        self.fused = LinearWeight(torch.cat([weights["q_proj.weight"], weights["k_proj.weight"],
                                             weights["v_proj.weight"], weights["b_proj.weight"]], dim=0))
        self.low = LinearWeight(torch.cat([a_down, g_down], dim=0))
        high = torch.zeros((H * d + H * dv, ra + rg), dtype=a_up.dtype, device=a_up.device)
        high[: H * d, :ra] = a_up
        high[H * d:, ra:] = g_up
        self.high = LinearWeight(high)
        self.out = LinearWeight(weights["o_proj.weight"])
        f32 = torch.float32
        self.taps = torch.cat([weights["q_conv.weight"], weights["k_conv.weight"], weights["v_conv.weight"]],
                              dim=0).to(f32).contiguous()
        self.rate = torch.exp(weights["A_log"].to(f32)).contiguous()      # exp(A_log), float32
        self.dt_bias = weights["dt_bias"].to(f32).contiguous()
        self.norm_weight = weights["norm.weight"].to(f32).contiguous()

    def cache_request(self):
        return CompositeRequest((
            StateRequest((self.num_heads, self.head_dim, self.value_dim), torch.float32),
            StateRequest((self.conv_taps - 1, self.channels), torch.float32)))

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        H, G, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        state, tails = cache
        projected = self.fused(x)                                        # [T, q | k | v | b]
        both = self.high(self.low(x), out_dtype=torch.float32)           # [T, a (H d) | gate (H dv)], float32
        q, k, v, g, beta = ops.delta_prepare(projected, 0, self.channels, both, self.dt_bias, self.rate, self.taps,
                                             tails.state, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots, H, G, d, dv,
                                             self.unit_eps, d ** -0.5)
        o = ops.linear_state_scan(q, k, v, state.state, ctx.cu_seqlens, ctx.slots, g=g, beta=beta)
        mixed = ops.head_norm_gate(o, self.eps, projected.dtype, weight=self.norm_weight, gate=both,
                                   gate_column=H * d, gate_act=ops.GATE_SIGMOID, out_scale=self.output_scale)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_mixer("generalized_delta_rule")
class GeneralizedDeltaRule(Mixer):
    """r = W_r x, k = W_k x (heads x head_dim), v = W_v x (heads x value_dim). Per head and key channel
    a decay g = exp(-decay_scale * sigmoid(W_d2 tanh(W_d1 x) + d_bias)) and a removal rate
    a = sigmoid(W_a x + a_bias); with the unit key u = k / sqrt(sum k^2 + unit_eps) of each head,
        S <- diag(g) S - (a * u) (u^T S) + k v^T    (both terms read the state before the token),
        o = S^T r    (the state after it).
    o is divided by its root mean square over value_dim (`eps`), multiplied by a weight over all heads'
    columns and by sigmoid(W_g x), then projected. The inner rank of the decay's low-rank product is
    the checkpoint's (`decay_rank` None) unless given. Everything behind the projections (the tanh is
    rounded to the activation type where it enters the second product) is float32.
    State: S [heads, head_dim, value_dim] in float32."""

    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, eps: float,
                 decay_scale: float, decay_rank: Optional[int] = None, unit_eps: float = 1e-6):
        if min(num_heads, head_dim, value_dim) <= 0 or not decay_scale > 0:
            raise InvalidError("generalized delta rule: sizes and the decay's scale must be positive")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.eps, self.decay_scale, self.decay_rank, self.unit_eps = float(eps), float(decay_scale), decay_rank, float(unit_eps)
        self.fused: Optional[LinearWeight] = None
        self.high: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        H, d, dv, h = self.num_heads, self.head_dim, self.value_dim, self.hidden_size
        return {"r_proj.weight": TensorSpec((H * d, h)), "k_proj.weight": TensorSpec((H * d, h)),
                "v_proj.weight": TensorSpec((H * dv, h)), "g_proj.weight": TensorSpec((H * dv, h)),
                "a_proj.weight": TensorSpec((H * d, h)), "a_proj.bias": TensorSpec((H * d,)),
                "d_down.weight": TensorSpec((self.decay_rank, h)), "d_up.weight": TensorSpec((H * d, self.decay_rank)),
                "d_bias": TensorSpec((H * d,)), "norm.weight": TensorSpec((H * dv,)),
                "o_proj.weight": TensorSpec((h, H * dv))}

    def bind(self, weights, runtime) -> None:
        f32 = torch.float32
        down, up = weights["d_down.weight"], weights["d_up.weight"]
        if up.shape[1] != down.shape[0]:
            raise InvalidError("generalized delta rule: the two halves of the decay's product disagree on its rank")
        # r | k | v | g | a | the decay's first product, in one product
        self.fused = LinearWeight(torch.cat([weights[n + "_proj.weight"] for n in "rkvga"] + [down], dim=0))
        self.rank = down.shape[0]
        self.high = LinearWeight(up)
        self.out = LinearWeight(weights["o_proj.weight"])
        self.a_bias = weights["a_proj.bias"].to(f32).contiguous()
        self.d_bias = weights["d_bias"].to(f32).contiguous()
        self.norm_weight = weights["norm.weight"].to(f32).contiguous()

    def cache_request(self):
        return StateRequest((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        H, d, dv = self.num_heads, self.head_dim, self.value_dim
        projected = self.fused(x, out_dtype=torch.float32)               # [T, r | k | v | g | a | low], float32
        at_v, at_g, at_a, at_low = 2 * H * d, 2 * H * d + H * dv, 2 * H * d + 2 * H * dv, 3 * H * d + 2 * H * dv
        inner = ops.tanh_columns(projected, at_low, self.rank, x.dtype)
        z = self.high(inner, out_dtype=torch.float32)                    # [T, H d], float32
        r, k, v, g, look, put = ops.general_delta_prepare(projected, 0, H * d, at_v, at_a, z, self.d_bias, self.a_bias,
                                                          self.decay_scale, self.unit_eps, H, d, dv)
        o = ops.general_delta_scan(r, k, v, g, look, put, cache.state, ctx.cu_seqlens, ctx.slots)
        mixed = ops.head_norm_gate(o, self.eps, x.dtype, weight=self.norm_weight, gate=projected, gate_column=at_g,
                                   gate_act=ops.GATE_SIGMOID)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """Two branches of `channels` channels each: y = gelu_tanh(W_y x + b_y) and
    u = conv(W_x x + b_x), a causal convolution of `conv_taps` taps per channel with a bias (zeros
    before the start, no activation). The channels are cut into `blocks` equal blocks; per block,
    with square matrices of its own, r = sigmoid(A u + b_a) and i = sigmoid(B u + b_b). Then
        a = exp(-decay_factor * r * softplus(lam)),   S <- a S + sqrt(1 - a^2) (i u)
    per channel, from S = 0, and the output is W_o (S y). Gates, decays and the state are float32;
    the projections keep their float32 sums up to the biases.
    State: S [channels] in float32 and the last conv_taps - 1 convolution inputs of every channel."""

    graph_safe = True

    def __init__(self, hidden_size: int, channels: int, blocks: int, conv_taps: int, decay_factor: float = 8.0):
        if channels <= 0 or blocks <= 0 or channels % blocks or conv_taps <= 0:
            raise InvalidError("gated linear recurrence: channels must be a multiple of blocks, and taps positive")
        self.hidden_size, self.channels, self.blocks, self.conv_taps = hidden_size, channels, blocks, conv_taps
        self.decay_factor = float(decay_factor)
        self.fused: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        C, h, B, n = self.channels, self.hidden_size, self.blocks, self.conv_taps
        s = C // B
        return {"x_proj.weight": TensorSpec((C, h)), "x_proj.bias": TensorSpec((C,)),
                "y_proj.weight": TensorSpec((C, h)), "y_proj.bias": TensorSpec((C,)),
                "conv.weight": TensorSpec((C, n)), "conv.bias": TensorSpec((C,)),
                "decay_gate.weight": TensorSpec((B, s, s)), "decay_gate.bias": TensorSpec((B, s)),
                "input_gate.weight": TensorSpec((B, s, s)), "input_gate.bias": TensorSpec((B, s)),
                "lam": TensorSpec((C,)), "o_proj.weight": TensorSpec((h, C))}

    def bind(self, weights, runtime) -> None:
        f32 = torch.float32
        # x | y in one product; a block's two gate matrices one above the other in one block product
        self.fused = LinearWeight(torch.cat([weights["x_proj.weight"], weights["y_proj.weight"]], dim=0))
        self.in_bias = torch.cat([weights["x_proj.bias"], weights["y_proj.bias"]]).to(f32).contiguous()
        self.taps = weights["conv.weight"].to(f32).contiguous()
        self.conv_bias = weights["conv.bias"].to(f32).contiguous()
        self.gates = torch.cat([weights["decay_gate.weight"], weights["input_gate.weight"]], dim=1).contiguous()
        self.gate_bias = torch.cat([weights["decay_gate.bias"], weights["input_gate.bias"]], dim=1).to(f32).contiguous()
        self.rate = (self.decay_factor * torch.nn.functional.softplus(weights["lam"].to(f32))).contiguous()
        self.out = LinearWeight(weights["o_proj.weight"])

    def cache_request(self):
        return CompositeRequest((StateRequest((self.channels,), torch.float32),
                                 StateRequest((self.conv_taps - 1, self.channels), torch.float32)))

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        C = self.channels
        state, tails = cache
        projected = self.fused(x, out_dtype=torch.float32)                       # [T, x | y], float32
        u = ops.short_conv(projected, 0, C, self.in_bias[:C], self.taps, self.conv_bias, tails.state,
                           ctx.cu_seqlens, ctx.seq_of_token, ctx.slots, x.dtype)
        gates = ops.blockwise_linear(u, self.gates, bias=self.gate_bias, out_dtype=torch.float32)
        mixed = ops.gated_linear_scan(u, gates, projected, C, self.in_bias[C:], self.rate, state.state,
                                      ctx.cu_seqlens, ctx.slots, ctx.max_seq_len, self.blocks)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_mixer("state_space_duality")
class StateSpaceDuality(Mixer):
    """A state-space mixer with one scalar decay per head and token. With inner = heads * value_dim,
    N = state_size and G = groups, W_in x is [z: inner | x: inner | B: G N | C: G N | dt: heads];
    x, B and C pass a causal convolution of `conv_taps` taps per channel with a bias (zeros before
    the start) and SiLU; dt = softplus(dt + dt_bias), without a clamp. Per head h (which reads the
    B and C of group h // (heads / G)), with S [N, value_dim] from zero:
        S <- exp(-exp(A_log_h) dt) S + dt B x^T,    y = S^T C + D_h x.
    y (heads side by side) is multiplied by silu(z), then each of `norm_parts` equal parts of the
    row is divided by its own root mean square (`eps`) and multiplied by a weight: the gate comes
    before the norm. Then W_o. The projection keeps its float32 sums; decays, step sizes and the
    state are float32 (csrc/scalar_gated_state.cu, the per-token-decay scan of csrc/recurrent_scan.cu).
    State: S in float32 and the last conv_taps - 1 convolution inputs of every channel."""

    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state_size: int, groups: int,
                 conv_taps: int, norm_parts: int, eps: float):
        inner = num_heads * value_dim
        if min(num_heads, value_dim, state_size, groups, conv_taps, norm_parts) <= 0 or num_heads % groups \
                or inner % norm_parts:
            raise InvalidError("state-space mixer: heads must be a multiple of groups, and the inner width of the norm's parts")
        self.hidden_size, self.num_heads, self.value_dim, self.state_size = hidden_size, num_heads, value_dim, state_size
        self.groups, self.conv_taps, self.norm_parts, self.eps = groups, conv_taps, norm_parts, float(eps)
        self.inner = inner
        self.channels = inner + 2 * groups * state_size
        self.fused: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        H, h, C = self.num_heads, self.hidden_size, self.channels
        return {"in_proj.weight": TensorSpec((self.inner + C + H, h)), "conv.weight": TensorSpec((C, self.conv_taps)),
                "conv.bias": TensorSpec((C,)), "dt_bias": TensorSpec((H,)), "A_log": TensorSpec((H,)),
                "D": TensorSpec((H,)), "norm.weight": TensorSpec((self.inner,)),
                "o_proj.weight": TensorSpec((h, self.inner))}

    def bind(self, weights, runtime) -> None:
        f32 = torch.float32
        self.fused = LinearWeight(weights["in_proj.weight"])
        self.taps = weights["conv.weight"].to(f32).contiguous()
        self.conv_bias = weights["conv.bias"].to(f32).contiguous()
        self.dt_bias = weights["dt_bias"].to(f32).contiguous()
        self.rate = torch.exp(weights["A_log"].to(f32)).contiguous()      # exp(A_log), float32
        self.skip = weights["D"].to(f32).contiguous()
        self.norm_weight = weights["norm.weight"].to(f32).contiguous()
        self.out = LinearWeight(weights["o_proj.weight"])

    def cache_request(self):
        return CompositeRequest((
            StateRequest((self.num_heads, self.state_size, self.value_dim), torch.float32),
            StateRequest((self.conv_taps - 1, self.channels), torch.float32)))

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        H, G, N, dv = self.num_heads, self.groups, self.state_size, self.value_dim
        state, tails = cache
        projected = self.fused(x, out_dtype=torch.float32)               # [T, z | x | B | C | dt], float32
        q, k, v, xf, decay = ops.ssd_prepare(projected, self.inner, self.inner + self.channels, self.dt_bias, self.rate,
                                             self.taps, self.conv_bias, tails.state, ctx.cu_seqlens, ctx.seq_of_token,
                                             ctx.slots, H, G, N, dv)
        ops.conv_tail_update_(projected, self.inner, self.channels, self.conv_taps, tails.state, ctx.cu_seqlens,
                              ctx.slots)
        o = ops.linear_state_scan(q, k, v, state.state, ctx.cu_seqlens, ctx.slots, token_decay=decay)
        mixed = ops.skip_gate_part_norm(o, xf, self.skip, projected, 0, self.norm_weight, self.norm_parts, self.eps,
                                        x.dtype)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_mixer("matrix_memory")
class MatrixMemory(Mixer):
    """A matrix memory with exponential gates, stabilized by a running maximum. q = W_q x *
    head_dim^-1/2, k = W_k x (heads x head_dim), v = W_v x (heads x value_dim); per head a log input
    gate i = cap tanh((W_i x + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f x +
    b_f) / cap)) with cap = `gate_cap`. With S [head_dim, value_dim], n [head_dim] and m from zero:
        m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k alone;
        o = S^T q / (max(|n . q|, exp(-m')) + floor_eps).
    Each head's o is divided by its root mean square (`eps`), multiplied by a weight over all
    heads' columns and by sigmoid(W_g x), then W_o. The projection keeps its float32 sums; gates,
    the maximum, S and n are float32. n rides the scan as one more value column (csrc/
    scalar_gated_state.cu), so the state is S | n [head_dim, value_dim + 1, filled up to a multiple of
    four columns] and m per head."""

    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 floor_eps: float = 1e-6):
        if min(num_heads, head_dim, value_dim) <= 0 or not gate_cap > 0:
            raise InvalidError("matrix memory: sizes and the gates' cap must be positive")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.gate_cap, self.eps, self.floor_eps = float(gate_cap), float(eps), float(floor_eps)
        self.padded = (value_dim + 1 + 3) // 4 * 4
        self.fused: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        H, d, dv, h = self.num_heads, self.head_dim, self.value_dim, self.hidden_size
        return {"q_proj.weight": TensorSpec((H * d, h)), "k_proj.weight": TensorSpec((H * d, h)),
                "v_proj.weight": TensorSpec((H * dv, h)), "g_proj.weight": TensorSpec((H * dv, h)),
                "i_gate.weight": TensorSpec((H, h)), "i_gate.bias": TensorSpec((H,)),
                "f_gate.weight": TensorSpec((H, h)), "f_gate.bias": TensorSpec((H,)),
                "norm.weight": TensorSpec((H * dv,)), "o_proj.weight": TensorSpec((h, H * dv))}

    def bind(self, weights, runtime) -> None:
        f32 = torch.float32
        # q | k | v | g | i | f in one product
        self.fused = LinearWeight(torch.cat([weights[n + ".weight"] for n in
                                             ("q_proj", "k_proj", "v_proj", "g_proj", "i_gate", "f_gate")], dim=0))
        self.i_bias = weights["i_gate.bias"].to(f32).contiguous()
        self.f_bias = weights["f_gate.bias"].to(f32).contiguous()
        self.norm_weight = weights["norm.weight"].to(f32).contiguous()
        self.out = LinearWeight(weights["o_proj.weight"])

    def cache_request(self):
        return CompositeRequest((StateRequest((self.num_heads, self.head_dim, self.padded), torch.float32),
                                 StateRequest((self.num_heads,), torch.float32)))

    def forward(self, x, ctx, cache, residual):
        _needs_own_state(ctx)
        H, d, dv = self.num_heads, self.head_dim, self.value_dim
        state, top = cache
        projected = self.fused(x, out_dtype=torch.float32)               # [T, q | k | v | g | i | f], float32
        gates_at = 2 * H * d + 2 * H * dv
        decay, take, floor = ops.capped_gates(projected, gates_at, gates_at + H, self.i_bias, self.f_bias,
                                              self.gate_cap, top.state, ctx.cu_seqlens, ctx.slots)
        q, k, v = ops.memory_prepare(projected, 0, H * d, 2 * H * d, take, d ** -0.5, H, d, dv, self.padded)
        o = ops.linear_state_scan(q, k, v, state.state, ctx.cu_seqlens, ctx.slots, token_decay=decay)
        mixed = ops.head_norm_gate(o, self.eps, x.dtype, weight=self.norm_weight, gate=projected,
                                   gate_column=2 * H * d + H * dv, gate_act=ops.GATE_SIGMOID, value_dim=dv,
                                   floor=floor, floor_eps=self.floor_eps)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)

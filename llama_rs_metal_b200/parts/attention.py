"""Grouped-query attention over the paged key/value cache."""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

from ..errors import InvalidError, UnsupportedError
from ..kernels import ops
from ..registry import POSITION_ENCODINGS, build_part, register_mixer
from ..weights.loader import TensorSpec
from .base import CompositeRequest, KeyValueRequest, Mixer, PartSpec, StateRequest
from .linear import LinearWeight


@register_mixer("attention")
class Attention(Mixer):
    """q, k, v projections -> position encoding of q and k -> cache write ->
    causal attention with scale head_dim^-1/2 -> output projection, added to
    the residual stream (crates/model-runtime/src/execute.rs:45-112,196).

    A prompt attends to its own freshly projected keys; a decoded token, or a
    portion of several tokens appended to a started sequence, attends to the
    cache. `window` limits a query to the last `window` keys. Which kernels run
    is decided in kernels/attention_dispatch.py (`attend`); a variant mixer
    overrides `before_rotation` to transform q and k per head.

    Options: `value_dim`, the head width of values when it is not that of queries and keys;
    `bias`, the q, k and v projections have biases (added in float32 before rounding);
    `output_scale`, a factor on the mixer's output (a mixer that enters a weighted sum of
    mixers), applied to the mixed heads before the output projection. A position scheme that
    is a linear distance penalty (`distance_slopes`) is applied by the attention kernels.
    `values_are_keys`: there is no value projection, a token's key row is its value row too, and
    the cache keeps keys only; `sinks`: a learned number per query head (tensor `sinks`) whose
    exponential joins the softmax's denominator; `query_temperature` (coef, every): the query
    at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).

    Queries and keys shaped between projection and attention (any of these makes the layer take its
    float32 projection through csrc/shaped_qkv.cu, which then also rotates): `conv_taps` n, a causal
    convolution of n taps per channel on q, k and v right after the biased projection (tensors
    `q_conv.weight`, `k_conv.weight`, `v_conv.weight`, [channels, n]; the last n - 1 projections of a
    sequence are kept as state beside its keys and values); `row_norm_eps`, an RMS norm with weights
    over the whole query row and the whole key row before the rotation (`q_norm.weight`,
    `k_norm.weight`); `head_norm_eps`, each query and key head divided by its root mean square after
    the rotation, no weight. `chunk`: positions form chunks of this many counted from position 0 and a
    query sees the keys of its own chunk only; the cache then keeps a window of `chunk` keys.
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, value_dim: Optional[int] = None, bias: bool = False,
                 output_scale: float = 1.0, values_are_keys: bool = False, sinks: bool = False,
                 query_temperature: Optional[Sequence[float]] = None, conv_taps: int = 0,
                 row_norm_eps: Optional[float] = None, head_norm_eps: Optional[float] = None,
                 chunk: Optional[int] = None):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise InvalidError("attention heads must be a multiple of key/value heads")
        self.values_are_keys, self.has_sinks = bool(values_are_keys), bool(sinks)
        if self.values_are_keys and value_dim not in (None, head_dim):
            raise InvalidError("values that are the keys have the keys' width")
        self.query_temperature = None
        if query_temperature is not None:
            coef, every = float(query_temperature[0]), int(query_temperature[1])
            if every <= 0:
                raise InvalidError("a query temperature grows every so many positions: a positive number")
            self.query_temperature = (coef, every)
        self.extras = None
        self.conv_taps = int(conv_taps)
        self.row_norm_eps = None if row_norm_eps is None else float(row_norm_eps)
        self.head_norm_eps = None if head_norm_eps is None else float(head_norm_eps)
        self.chunk = int(chunk) if chunk else None
        if self.conv_taps < 0 or (self.chunk is not None and (self.chunk <= 0 or window is not None)):
            raise InvalidError("attention: taps cannot be negative, and a chunked layer has no window besides")
        self.shaped = bool(self.conv_taps) or self.row_norm_eps is not None or self.head_norm_eps is not None
        if self.shaped and (values_are_keys or sinks or query_temperature is not None):
            raise InvalidError("shaped queries and keys are not built together with sinks, a query temperature or keys as values")
        self.taps = self.row_norm = None
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.window = head_dim, window
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.has_bias, self.output_scale = bool(bias), float(output_scale)
        self.bias: Optional[torch.Tensor] = None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = build_part(POSITION_ENCODINGS, position, "position encoding") \
            if position is not None else None
        self.qkv: Optional[LinearWeight] = None
        self.q_only: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def tensors(self) -> Dict[str, TensorSpec]:
        q, kv, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        v, mixed = self.num_kv_heads * self.value_dim, self.num_heads * self.value_dim
        out = {"q_proj.weight": TensorSpec((q, h)), "k_proj.weight": TensorSpec((kv, h)),
               "v_proj.weight": TensorSpec((v, h)), "o_proj.weight": TensorSpec((h, mixed))}
        if self.values_are_keys:
            del out["v_proj.weight"]
        if self.has_sinks:
            out["sinks"] = TensorSpec((self.num_heads,))
        if self.has_bias:
            out.update({"q_proj.bias": TensorSpec((q,)), "k_proj.bias": TensorSpec((kv,))})
            if not self.values_are_keys:
                out["v_proj.bias"] = TensorSpec((v,))
        if self.conv_taps:
            out.update({"q_conv.weight": TensorSpec((q, self.conv_taps)), "k_conv.weight": TensorSpec((kv, self.conv_taps)),
                        "v_conv.weight": TensorSpec((v, self.conv_taps))})
        if self.row_norm_eps is not None:
            out.update({"q_norm.weight": TensorSpec((q,)), "k_norm.weight": TensorSpec((kv,))})
        if self.position is not None:
            out.update({"position." + n: s for n, s in self.position.tensors().items()})
        return out

    def bind(self, weights, runtime) -> None:
        # One [q + 2kv, h] matrix: rows of the three projections one after another,
        # so each output element is the same dot product as with separate matrices.
        q_weight, k_weight = weights["q_proj.weight"], weights["k_proj.weight"]
        # (a shaped layer's kernel rotates neighbouring pairs itself: nothing is reordered)
        order = self.position.head_permutation() if self.position is not None and not self.shaped else None
        if order is not None:
            # the position scheme wants each head's dimensions reordered: the same reordering of
            # the rows of the query and key projections leaves every score q.k as it was
            index = torch.tensor(order, dtype=torch.long, device=q_weight.device)
            q_weight = q_weight.view(self.num_heads, self.head_dim, -1)[:, index].reshape(q_weight.shape)
            k_weight = k_weight.view(self.num_kv_heads, self.head_dim, -1)[:, index].reshape(k_weight.shape)
        rows = [q_weight, k_weight] if self.values_are_keys else [q_weight, k_weight, weights["v_proj.weight"]]
        fused = torch.cat(rows, dim=0).contiguous()
        if self.has_sinks or self.query_temperature is not None:
            from ..kernels.attention_dispatch import Extras
            sinks = weights["sinks"].to(torch.float32).contiguous() if self.has_sinks else None
            self.extras = Extras(sinks, self.query_temperature)
        self.qkv = LinearWeight(fused)
        self.q_only = LinearWeight(fused[: self.num_heads * self.head_dim])
        self.out = LinearWeight(weights["o_proj.weight"])
        if self.has_bias:
            if order is not None:
                raise InvalidError("projection biases with a reordered head are not built")
            biases = ["q_proj.bias", "k_proj.bias"] + ([] if self.values_are_keys else ["v_proj.bias"])
            self.bias = torch.cat([weights[n] for n in biases]).to(torch.float32).contiguous()
        if self.position is not None:
            self.position.bind({n[len("position."):]: t for n, t in weights.items()
                                if n.startswith("position.")}, runtime)
        if self.conv_taps:
            # [taps, projection row]: the kernel reads one tap of many channels at a time
            self.taps = torch.cat([weights[n + "_conv.weight"] for n in "qkv"], dim=0).to(torch.float32).t().contiguous()
        if self.row_norm_eps is not None:
            self.row_norm = (weights["q_norm.weight"].to(torch.float32).contiguous(),
                             weights["k_norm.weight"].to(torch.float32).contiguous())
        if self.shaped and self.position is not None and self.position.rotary_table() is None:
            raise InvalidError("a shaped attention layer rotates by a rotary table or not at all")

    @property
    def projected_width(self) -> int:
        return self.num_heads * self.head_dim + self.num_kv_heads * (self.head_dim + self.value_dim)

    def cache_request(self):
        # a chunk never shows a key more than `chunk` - 1 positions back: the cache keeps that window
        keys = KeyValueRequest(self.num_kv_heads, self.head_dim, self.chunk or self.window,
                               None if self.value_dim == self.head_dim else self.value_dim,
                               values_in_keys=self.values_are_keys)
        if self.conv_taps > 1:
            return CompositeRequest((keys, StateRequest((self.conv_taps - 1, self.projected_width), torch.float32)))
        return keys

    def _shaped_forward(self, x, ctx, cache, residual):
        """Projection in float32, then bias, convolution, norms and rotation in one kernel that also
        splits and stores, then attention under the window or the chunk."""
        from ..kernels.attention_dispatch import Shaping
        entry = ctx.entry
        if not entry.writes_cache:
            raise UnsupportedError("a shaped attention layer reading another layer's cache is not built")
        keys, tails = cache if self.conv_taps > 1 else (cache, None)
        inv_freq, rotary, adjacent = None, 0, False
        if self.position is not None:
            rotary, adjacent = self.position.rotary_dim, self.position.adjacent_pairs
            inv_freq = self.position.inv_freq64
        shaping = Shaping(taps=self.taps, tails=tails, row_norm=self.row_norm, row_eps=self.row_norm_eps or 0.0,
                          inv_freq=inv_freq, rotary=rotary, adjacent_pairs=adjacent, head_norm_eps=self.head_norm_eps)
        mixed = ops.attend(self.qkv(x, out_dtype=torch.float32), q_heads=self.num_heads, kv_heads=self.num_kv_heads,
                           head_dim=self.head_dim, rotary=None, ctx=ctx, cache=keys, writes_cache=True,
                           cache_entry=entry.cache, scale=self.scale, window=self.chunk or self.window,
                           value_dim=self.value_dim, bias=self.bias, out_scale=self.output_scale, shaping=shaping,
                           chunk=self.chunk)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)

    def forward(self, x, ctx, cache, residual):
        if self.shaped:
            return self._shaped_forward(x, ctx, cache, residual)
        entry = ctx.entry
        weight = self.qkv if entry.writes_cache else self.q_only
        rotary = self.position.rotary_table() if self.position is not None else None
        slopes = self.position.distance_slopes() if self.position is not None else None
        if (self.has_bias or self.value_dim != self.head_dim or slopes is not None or self.output_scale != 1.0
                or self.values_are_keys or self.extras is not None or self.chunk):
            # the general form: projection, then a split that adds the biases and stores keys and
            # values, then the attention kernels that know the penalty and the value width
            bias = self.bias
            if bias is not None and not entry.writes_cache:
                bias = bias[: self.num_heads * self.head_dim]
            mixed = ops.attend(weight(x), q_heads=self.num_heads, kv_heads=self.num_kv_heads,
                               head_dim=self.head_dim, rotary=rotary, ctx=ctx, cache=cache,
                               writes_cache=entry.writes_cache, cache_entry=entry.cache, scale=self.scale,
                               window=self.window, value_dim=self.value_dim, bias=bias, slopes=slopes,
                               out_scale=self.output_scale, extras=self.extras,
                               values_are_keys=self.values_are_keys, chunk=self.chunk)
            return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)
        # Nothing stands between projection and rotation unless a variant mixer overrides the hook
        # or the position scheme is no rotary table: the kernels may then do both in one launch.
        direct = (type(self).before_rotation is Attention.before_rotation
                  and (self.position is None or rotary is not None) and x.dtype == weight.weight.dtype)
        projected = None if direct else self.before_rotation(weight(x), ctx, entry.writes_cache)
        mixed = ops.attend(projected, q_heads=self.num_heads, kv_heads=self.num_kv_heads,
                           head_dim=self.head_dim, rotary=rotary, ctx=ctx, cache=cache,
                           writes_cache=entry.writes_cache, cache_entry=entry.cache, scale=self.scale,
                           window=self.window, projection=(x, weight.weight) if direct else None)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)

    def before_rotation(self, projected, ctx, has_keys: bool):
        """Hook between the projection and the kernels: [T, (Hq + 2 Hk) d] when `has_keys`, else
        [T, Hq d] queries. A variant mixer transforms q and k per head here (a norm of each
        head, a bias) and returns the same layout. As built: a position scheme that is not a
        rotary table transforms q and k here."""
        if self.position is None or self.position.rotary_table() is not None:
            return projected
        T = projected.shape[0]
        nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        q = projected[:, :nq].reshape(T, self.num_heads, self.head_dim)
        if not has_keys:
            q, _ = self.position.apply(q, q[:, :0], ctx)
            return q.reshape(T, nq).contiguous()
        k = projected[:, nq:nq + nk].reshape(T, self.num_kv_heads, self.head_dim)
        q, k = self.position.apply(q, k, ctx)
        return torch.cat([q.reshape(T, nq), k.reshape(T, nk), projected[:, nq + nk:]], dim=1).contiguous()

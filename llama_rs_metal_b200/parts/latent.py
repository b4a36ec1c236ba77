"""Attention whose keys and values are unfolded from one small latent vector per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import InvalidError
from ..kernels import ops
from ..registry import POSITION_ENCODINGS, build_part, register_mixer
from ..weights.loader import TensorSpec
from .base import KeyValueRequest, Mixer, PartSpec
from .linear import LinearWeight


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Per token: cq = RMSnorm(W_dq x) w_q and q = W_uq cq, per head [head_dim plain | rot_dim
    rotated]; c = RMSnorm((W_dkv x)[:kv_rank]) w_c and one key part k_r = rotate((W_dkv x)[kv_rank:])
    shared by all heads. Per head h: key [W_uk_h c | k_r], value W_uv_h c,
        score = (q_plain . W_uk_h c + q_rot . k_r) * scale,
    softmax over the last `window` positions (all, when None), the head's output times
    sigmoid(W_g x)_h, then W_o.

    Only c and k_r are cached: one key head of width kv_rank + rot_dim whose first kv_rank columns
    are also the value row. The per-head matrices are folded onto the query side,
        q_plain . W_uk_h c = (W_uk_h^T q_plain) . c,    sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j),
    so attention runs as one key/value head of the latent's width for every phase, and W_uk, W_uv
    are applied to queries and outputs as block products (csrc/blockwise.cu). `owns_latent` False:
    the layer has no W_dkv and reads the cache entry another layer of the same kv_rank, rot_dim
    and rotation filled (the schedule entry names it, with writes_cache False); `cache_window` is
    then what that entry has to keep for its widest reader. `position` is a rotary PartSpec over
    rot_dim dimensions (a scheme that pairs neighbouring dimensions has the rotated rows of W_q and
    W_dkv reordered once, when they are bound).

    `q_rank` None: the queries have no latent, q = W_q x. `sinks`: a learned number per head whose
    exponential is added to the softmax's denominator (no key, no value, not scaled). `gate`
    "per_head": one sigmoid gate per head; "per_dim": one per head and value dimension, applied to
    the concatenated heads element by element."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 q_rank: Optional[int], eps: float, scale: float, position: Optional[PartSpec] = None,
                 window: Optional[int] = None, owns_latent: bool = True, cache_window: Optional[int] = None,
                 sinks: bool = False, gate: str = "per_head"):
        if min(num_heads, head_dim, value_dim, kv_rank, q_rank or 1) <= 0 or rot_dim < 0 or rot_dim % 2:
            raise InvalidError("latent attention: sizes must be positive and the rotated part even")
        if gate not in ("per_head", "per_dim"):
            raise InvalidError("latent attention: the gate is per_head or per_dim")
        if (rot_dim > 0) != (position is not None):
            raise InvalidError("latent attention: a rotated key part needs a position scheme, and the reverse")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.kv_rank, self.q_rank = value_dim, kv_rank, q_rank
        self.eps, self.scale, self.window, self.owns_latent = float(eps), float(scale), window, bool(owns_latent)
        self.cache_window = cache_window if owns_latent and cache_window is not None else window
        self.has_sinks, self.gates = bool(sinks), num_heads * (value_dim if gate == "per_dim" else 1)
        self.extras = None
        self.position = build_part(POSITION_ENCODINGS, position, "position encoding") if position is not None else None
        self.down: Optional[LinearWeight] = None
        self.up_q: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def tensors(self) -> Dict[str, TensorSpec]:
        H, d, r, dv, h = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.hidden_size
        out = {"k_up.weight": TensorSpec((H * d, self.kv_rank)), "v_up.weight": TensorSpec((H * dv, self.kv_rank)),
               "gate.weight": TensorSpec((self.gates, h)), "o_proj.weight": TensorSpec((h, H * dv))}
        if self.q_rank is not None:
            out.update({"q_down.weight": TensorSpec((self.q_rank, h)), "q_down.norm": TensorSpec((self.q_rank,)),
                        "q_up.weight": TensorSpec((H * (d + r), self.q_rank))})
        else:
            out["q_proj.weight"] = TensorSpec((H * (d + r), h))
        if self.has_sinks:
            out["sinks"] = TensorSpec((H,))
        if self.owns_latent:
            out.update({"kv_down.weight": TensorSpec((self.kv_rank + r, h)), "kv_down.norm": TensorSpec((self.kv_rank,))})
        return out

    def bind(self, weights, runtime) -> None:
        H, d, r, dv, f32 = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, torch.float32
        self.inv_freq, order = None, None
        if self.position is not None:
            self.position.bind({}, runtime)
            table = self.position.rotary_table()
            if table is None or table[1] != self.rot_dim:
                raise InvalidError("latent attention rotates its rot_dim dimensions by a rotary table")
            self.inv_freq = table[0]
            order = self.position.head_permutation()  # new rotated dimension j is old dimension order[j]
        queries = weights["q_up.weight"] if self.q_rank is not None else weights["q_proj.weight"]
        kv_down = weights["kv_down.weight"] if self.owns_latent else None
        if order is not None:
            index = torch.tensor(order, dtype=torch.long, device=queries.device)
            queries = queries.view(H, d + r, -1).clone()
            queries[:, d:] = queries[:, d:].index_select(1, index)
            queries = queries.view(H * (d + r), -1)
            if kv_down is not None:
                kv_down = torch.cat([kv_down[:self.kv_rank], kv_down[self.kv_rank:].index_select(0, index)], dim=0)
        # (q latent, or q itself) | (kv latent | shared key part) | gates in one product
        q_width = self.q_rank if self.q_rank is not None else H * (d + r)
        rows = [weights["q_down.weight"] if self.q_rank is not None else queries] + \
            ([kv_down] if self.owns_latent else []) + [weights["gate.weight"]]
        self.down = LinearWeight(torch.cat(rows, dim=0))
        self.q_width = q_width
        self.c_column = q_width if self.owns_latent else -1
        self.gate_column = q_width + (self.kv_rank + self.rot_dim if self.owns_latent else 0)
        self.q_norm = weights["q_down.norm"].to(f32).contiguous() if self.q_rank is not None else None
        self.c_norm = weights["kv_down.norm"].to(f32).contiguous() if self.owns_latent else None
        self.up_q = LinearWeight(queries) if self.q_rank is not None else None
        if self.has_sinks:
            from ..kernels.attention_dispatch import Extras
            self.extras = Extras(sinks=weights["sinks"].to(f32).contiguous())
        # W_uk_h^T as the [out = kv_rank, in = head_dim] matrix of head h; W_uv_h is [value_dim, kv_rank] as stored
        self.k_fold = weights["k_up.weight"].view(H, d, self.kv_rank).transpose(1, 2).contiguous()
        self.v_unfold = weights["v_up.weight"].view(H, dv, self.kv_rank).contiguous()
        self.out = LinearWeight(weights["o_proj.weight"])

    def cache_request(self):
        if not self.owns_latent:
            return None
        return KeyValueRequest(1, self.kv_rank + self.rot_dim, self.cache_window, self.kv_rank, values_in_keys=True)

    def forward(self, x, ctx, cache, residual):
        H, d, r, dv, kv = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        entry, prefill = ctx.entry, ctx.phase == "prefill"
        writes = self.owns_latent and entry.writes_cache
        projected = self.down(x, out_dtype=torch.float32)
        cq, rows, gate = ops.latent_prepare(
            projected, 0, self.q_norm, self.c_column, self.c_norm, r, ctx.positions, self.inv_freq, self.eps,
            self.gate_column, self.gates, x.dtype, kv=cache if writes else None,
            dest_rows=ctx.dest_rows[cache.group] if writes and cache is not None else None, keep_packed=prefill,
            q_width=self.q_width)
        if prefill:
            if writes:
                ctx.fresh_kv[entry.cache] = (rows, rows)
            rows = ctx.fresh_kv[entry.cache][0]
        q = self.up_q(cq) if self.up_q is not None else cq                  # [T, H (d + r)]
        T = q.shape[0]
        folded = torch.empty((T, H * (kv + r)), dtype=q.dtype, device=q.device)
        ops.blockwise_linear(q, self.k_fold, x_block=d + r, out=folded, out_block=kv + r)
        if r:
            ops.rope_heads(q, d, d + r, folded, kv, kv + r, ctx.positions, self.inv_freq, H)
        folded = folded.view(T, H, kv + r)
        if prefill:
            mixed = ops.attention_prefill(folded, rows.view(T, 1, kv + r), None, ctx.cu_seqlens, ctx.seq_of_token,
                                          ctx.max_seq_len, self.scale, self.window, value_dim=kv, extras=self.extras)
        elif ctx.phase == "decode":
            mixed = ops.attention_decode(folded, cache, ctx.slots, ctx.kv_lens, ctx.max_kv_len, self.scale, self.window,
                                         extras=self.extras)
        else:
            mixed = ops.attention_extend(folded, cache, ctx.cu_seqlens, ctx.seq_of_token, ctx.positions, ctx.slots,
                                         ctx.kv_lens, ctx.max_seq_len, self.scale, self.window, extras=self.extras)
        heads = ops.blockwise_linear(mixed, self.v_unfold, row_scale=gate, out_dtype=x.dtype)   # [T, H dv]
        return self.out(heads, epilogue=ops.ADD, out=residual, ctx=ctx)

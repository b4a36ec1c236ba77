"""Mixture of experts: a router picks a few small gated feed-forwards per token."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..errors import InvalidError, UnsupportedError
from ..kernels import ops
from ..registry import FEED_FORWARDS, build_part, register_feed_forward
from ..weights.loader import TensorSpec
from .base import FeedForward, PartSpec
from .linear import LinearWeight


@register_feed_forward("moe")
class MixtureOfExperts(FeedForward):
    """z = W_r x (+ b_r) in float32; the `top` experts with the largest z are chosen and weighted
    by the softmax over the chosen z only; the output is the weighted sum of their outputs,
    added to the residual stream.

    An expert (activation "clamped_gate"): g = min(W_gate x, limit), u = clamp(W_up x, -limit,
    limit), y = g sigmoid(alpha g) (u + 1), output W_down y; no biases.

    The router's matrix is kept in float32 whatever the runtime, so its product runs on the
    float32 kernel. The experts' matrices are stacked, gate_up [E, 2 ff, h] and down [h, E, ff],
    and serve two ways of computing (csrc/moe.cu). Token by token (decoding, float32, many
    experts per choice): one launch reads, for every token, only the experts it chose; their
    outputs come back as float32 planes that are added to the stream in a fixed order (by the
    next norm where it folds them). All experts at once (bfloat16 steps of DENSE_ROWS tokens and
    more when at most DENSE_RATIO experts exist per chosen one): two tensor-core products over
    every expert, with the weights of the experts a token did not choose set to zero between
    them.

    Options beyond that router and that expert. `activation` "silu": an expert is W_down (silu(W_gate
    x) * (W_up x)). `scoring` "softmax_all": the scores are s = softmax(z) over all outputs; the
    choice is made on s + correction (`correction` True: a stored vector), the weights are the
    chosen s (divided by their sum with `renormalize`). `groups` (count, keep): the outputs form
    `count` equal groups of neighbours, a group counts by its largest choice score, and only the
    outputs of the `keep` best groups can be chosen. `identity` n: the router has n more outputs
    than there are experts; the last n are identity experts without matrices, whose output is the
    layer's input itself (the float32 stream where the block gives it) times the weight. `shared`
    (a PartSpec of a feed-forward): a part that runs for every token and is added; with `shared_gate`
    it is first multiplied by sigmoid(w . x), one number per token (tensor `shared.gate`, [1, hidden],
    kept and applied in float32). `renormalize_eps` is added to the sum the chosen scores are divided
    by, `weight_scale` multiplies the weights afterwards."""

    graph_safe = True
    ROUTER_ROWS = 256  # up to this many tokens the router always runs as one launch, a CTA per token
    DENSE_ROWS = 64   # from this many tokens on a step is a prompt: the tensor-core products pay
    DENSE_RATIO = 4   # experts per chosen expert up to which computing all of them is the faster way

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 activation: str = "clamped_gate", limit: float = 7.0, alpha: float = 1.702,
                 router_bias: bool = True, scoring: str = "softmax_chosen", correction: bool = False,
                 groups: Optional[Tuple[int, int]] = None, renormalize: bool = False, identity: int = 0,
                 shared: Optional[PartSpec] = None, weight_scale: float = 1.0, renormalize_eps: float = 0.0,
                 shared_gate: bool = False):
        if activation not in ("clamped_gate", "silu"):
            raise UnsupportedError(f"expert activation {activation!r}")
        if scoring not in ("softmax_chosen", "softmax_all"):
            raise UnsupportedError(f"router scoring {scoring!r}")
        outputs = num_experts + identity
        if num_experts <= 0 or identity < 0 or not 0 < top <= outputs:
            raise InvalidError("the router chooses between 1 and all of the experts")
        count, keep = groups if groups is not None else (1, 1)
        if (shared_gate and shared is None) or (scoring == "softmax_chosen" and (weight_scale != 1.0 or renormalize_eps)):
            raise UnsupportedError("a gate needs a shared part; weight scale and epsilon belong to the softmax_all router")
        self.weight_scale, self.renormalize_eps, self.shared_gate = float(weight_scale), float(renormalize_eps), bool(shared_gate)
        self.shared_gate_weight: Optional[torch.Tensor] = None
        if scoring == "softmax_chosen" and (correction or groups is not None or identity or renormalize):
            raise UnsupportedError("corrections, groups and identity experts belong to the softmax_all router")
        if count <= 0 or outputs % count or not 0 < keep <= count or top > keep * (outputs // count):
            raise InvalidError("router groups must divide its outputs, and the kept groups hold at least `top` of them")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top, self.identity, self.outputs = num_experts, top, identity, outputs
        self.limit, self.alpha = float(limit), float(alpha)
        self.act = ops.ACT_SILU if activation == "silu" else ops.ACT_CLAMPED_GATE
        self.scored, self.has_correction = scoring == "softmax_all", bool(correction)
        self.router_bias = bool(router_bias) and not self.scored
        self.groups, self.keep, self.renormalize = count, keep, bool(renormalize)
        self.shared = build_part(FEED_FORWARDS, shared, "feed-forward") if shared is not None else None
        self._shared_spec = shared
        self.router: Optional[LinearWeight] = None
        self.bias: Optional[torch.Tensor] = None
        self.scoring: Optional[ops.Scoring] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        h, f = self.hidden_size, self.intermediate_size
        out = {"router.weight": TensorSpec((self.outputs, h))}
        if self.router_bias:
            out["router.bias"] = TensorSpec((self.num_experts,))
        if self.has_correction:
            out["router.correction"] = TensorSpec((self.outputs,))
        if self.shared is not None:
            for own, spec in self.shared.tensors().items():
                out["shared." + own] = spec
            if self.shared_gate:
                out["shared.gate"] = TensorSpec((1, h))
        for e in range(self.num_experts):
            out[f"experts.{e}.gate_proj.weight"] = TensorSpec((f, h))
            out[f"experts.{e}.up_proj.weight"] = TensorSpec((f, h))
            out[f"experts.{e}.down_proj.weight"] = TensorSpec((h, f))
        return out

    def bind(self, weights, runtime) -> None:
        self.router = LinearWeight(weights["router.weight"].to(torch.float32))
        self.bias = weights["router.bias"].to(torch.float32).contiguous() if self.router_bias else None
        if self.scored:
            correction = weights["router.correction"].to(torch.float32).contiguous() if self.has_correction else None
            self.scoring = ops.Scoring(correction, self.groups, self.keep, self.renormalize, self.renormalize_eps,
                                       self.weight_scale)
        if self.shared is not None:
            self.shared.bind({own: weights["shared." + own] for own in self.shared.tensors()}, runtime)
            if self.shared_gate:
                self.shared_gate_weight = weights["shared.gate"].to(torch.float32).reshape(-1).contiguous()
        E, f, h = self.num_experts, self.intermediate_size, self.hidden_size
        self.gate_up = torch.stack([torch.cat([weights[f"experts.{e}.gate_proj.weight"],
                                               weights[f"experts.{e}.up_proj.weight"]]) for e in range(E)]).contiguous()
        self.down = torch.stack([weights[f"experts.{e}.down_proj.weight"] for e in range(E)], dim=1).contiguous()
        # the same storage seen as two plain matrices, for the products over every expert
        self.gate_up_all = LinearWeight(self.gate_up.view(E * 2 * f, h))
        self.down_all = LinearWeight(self.down.view(h, E * f))

    def route(self, x):
        """(expert ids int32 [T, top], weights float32 [T, top]). One launch per step; steps of
        many tokens make the logits with the float32 matrix kernel first when there are many
        experts to a token's CTA."""
        routed = ops.moe_router(x, self.router.weight, self.bias, self.top, self.scoring) \
            if x.shape[0] <= self.ROUTER_ROWS or self.outputs <= 16 else None
        if routed is None:
            logits = self.router(x, out_dtype=torch.float32)
            routed = ops.moe_route_scored(logits, self.top, self.scoring) if self.scored \
                else ops.moe_route(logits, self.bias, self.top)
        return routed

    def forward(self, x, ctx, residual):
        ids, weights = self.route(x)
        # identity experts pass the input on: the float32 stream itself where x is its rounding
        x32 = ctx.stream if self.identity and x.dtype != torch.float32 else None
        dense = (x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16 and x.shape[0] >= self.DENSE_ROWS
                 and self.num_experts <= self.DENSE_RATIO * self.top)
        if residual is None:
            # a block that puts a norm between this part and the stream: the shared part's float32
            # output (or the all-experts product's) is what everything else is added to
            out = self.shared.forward(x, ctx, residual=None) if self.shared is not None else None
            if self.shared_gate and not dense:
                # the gate on the shared part and the experts' planes beside it in one pass
                planes = ops.moe_experts_rows(x, self.gate_up, self.down, ids, weights, self.limit, self.alpha, self.act, x32)
                return ops.row_gate_(out, x, self.shared_gate_weight, planes)
            if self.shared_gate:
                ops.row_gate_(out, x, self.shared_gate_weight)
            if dense:
                both = self.gate_up_all(x, out_dtype=torch.float32)
                y = ops.moe_dense_gate(both, ids, weights, self.num_experts, self.limit, self.alpha, out_dtype=x.dtype,
                                       act=self.act)
                out = self.down_all(y, epilogue=ops.ADD, out=out)
                if self.identity:
                    ops.moe_identity_add_(out, x32 if x32 is not None else x, ids, weights, self.num_experts)
                return out
            planes = ops.moe_experts_rows(x, self.gate_up, self.down, ids, weights, self.limit, self.alpha, self.act, x32)
            if out is None:
                out, planes = planes[0], planes[1:]
            return ops.add_planes_(out, planes) if planes.shape[0] else out
        if self.shared_gate:
            gated = ops.row_gate_(self.shared.forward(x, ctx, residual=None), x, self.shared_gate_weight)
            ctx.settle(residual)
            ops.add_(residual, gated)
        elif self.shared is not None:
            residual = self.shared.forward(x, ctx, residual=residual)
            ctx.settle(residual)
        if dense:
            # gate and up stay float32 up to the activation, as they do token by token
            both = self.gate_up_all(x, out_dtype=torch.float32)
            y = ops.moe_dense_gate(both, ids, weights, self.num_experts, self.limit, self.alpha, out_dtype=x.dtype,
                                   act=self.act)
            if self.identity:
                ctx.settle(residual)
                ops.moe_identity_add_(residual, x32 if x32 is not None else x, ids, weights, self.num_experts)
            return self.down_all(y, epilogue=ops.ADD, out=residual, ctx=ctx)
        planes = ops.moe_experts_rows(x, self.gate_up, self.down, ids, weights, self.limit, self.alpha, self.act, x32)
        if ctx.may_defer:
            ctx.settle(residual)  # at most one set of partial sums is pending at a time
            ctx.pending = planes
            return residual
        return ops.add_planes_(residual, planes)

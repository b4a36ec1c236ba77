"""Norms: RMSNorm, layer norm with weight and bias, and the plain rounding of the stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import UnsupportedError
from ..kernels import ops
from ..registry import register_norm
from ..weights.loader import TensorSpec
from .base import Norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * (offset + w), statistics in float32
    (crates/metal-backend/src/shaders/elementwise.metal:31-46; no +1 offset for Llama).
    `offset` 1 is for checkpoints that keep a norm's weight as its difference from 1; the sum is made once, in float32, when the
    weights are bound. `scalar`: the stored weight is one number (a tensor without dimensions) that
    multiplies every coordinate; it is spread over the row once, when the weights are bound."""

    graph_safe = True
    folds_pending = True

    def __init__(self, size: int, eps: float, offset: float = 0.0, scalar: bool = False):
        self.size = size
        self.eps = float(eps)
        self.offset = float(offset)
        self.scalar = bool(scalar)
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec(() if self.scalar else (self.size,))}

    def bind(self, weights, runtime) -> None:
        weight = weights["weight"]
        if self.scalar:
            weight = weight.reshape(1).expand(self.size)
        if self.offset != 0.0:
            weight = weight.to(torch.float32) + self.offset
        self.weight = weight.contiguous()

    def forward(self, hidden, ctx, rows=None):
        # partial sums a product left for the residual stream are added in the same pass
        pending = ctx.take_pending()
        return ops.rms_norm(hidden, self.weight, self.eps, ctx.runtime.dtype, rows=rows, partials=pending)

    def add_into(self, hidden, y, ctx, mult=1.0, then=None):
        # one pass: the sublayer's output is normalized, scaled and added to the stream, and the
        # updated row goes through the next sublayer's norm while it is still in registers
        fused = isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype
        out = ops.rms_norm_add_(hidden, y, self.weight, self.eps, mult,
                                then.weight if fused else None, then.eps if fused else None,
                                ctx.runtime.dtype if fused else None)
        if then is not None and not fused:
            out = then.forward(hidden, ctx)
        return out


@register_norm("cast")
class StreamCast(Norm):
    """No norm at all: the stream itself in the activation type (the float32 stream as it is under
    float32 activations, its rounding under bfloat16). It stands where a block wants "the norm in
    front of the sublayer" of an arrangement whose sublayers read the stream itself."""

    graph_safe = True

    def forward(self, hidden, ctx, rows=None):
        if rows is not None:
            raise UnsupportedError("the plain rounding of the stream is not made for chosen rows")
        return ops.cast(hidden, ctx.runtime.dtype)


@register_norm("layer_norm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(variance + eps) * w + b over a row, with the variance the mean of the
    squared deviations; statistics, weight and bias in float32. The bias is the tensor `bias`."""

    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, float(eps)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,)), "bias": TensorSpec((self.size,))}

    def bind(self, weights, runtime) -> None:
        self.weight = weights["weight"].to(torch.float32).contiguous()
        self.bias = weights["bias"].to(torch.float32).contiguous()

    def forward(self, hidden, ctx, rows=None):
        return ops.layer_norm(hidden, self.weight, self.bias, self.eps, ctx.runtime.dtype, rows=rows)

    def add_into(self, hidden, y, ctx, mult=1.0, then=None):
        # the pass that adds the normed output also writes the updated row in the activation type
        # when the next sublayer reads the stream itself
        if isinstance(then, StreamCast):
            if ctx.runtime.dtype == torch.float32:
                ops.layer_norm_add_(hidden, y, self.weight, self.bias, self.eps, mult)
                return hidden
            return ops.layer_norm_add_(hidden, y, self.weight, self.bias, self.eps, mult, cast_dtype=ctx.runtime.dtype)
        ops.layer_norm_add_(hidden, y, self.weight, self.bias, self.eps, mult)
        return then.forward(hidden, ctx) if then is not None else None

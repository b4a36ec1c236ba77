"""Dense feed-forwards: gated, and plain (one matrix up, an activation, one matrix down)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import UnsupportedError
from ..kernels import ops
from ..registry import register_feed_forward
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import LinearWeight

GATE_BLOCK = 8  # rows of gate and up alternate in blocks of this many in the fused matrix


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """down( act(x Wg^T) * (x Wu^T) ), added to the residual stream
    (crates/model-runtime/src/execute.rs:251-267). The reference builds SiLU only
    (crates/model-format/src/mlx/config.rs:58-64). Activation "clamped_gate" is the gate of the
    mixture of experts as a dense layer: g = min(x Wg^T, limit), u = clamp(x Wu^T, -limit, limit),
    down(g sigmoid(alpha g) (u + 1)); gate and up keep their float32 sums up to the activation.
    Activation "gelu_tanh": act(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), likewise from
    float32 sums."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 limit: float = 7.0, alpha: float = 1.702):
        if activation not in ("silu", "clamped_gate", "gelu_tanh"):
            raise UnsupportedError(f"feed-forward activation {activation!r}")
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up: Optional[LinearWeight] = None
        self.down: Optional[LinearWeight] = None
        self.block = GATE_BLOCK if intermediate_size % GATE_BLOCK == 0 else intermediate_size

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def bind(self, weights, runtime) -> None:
        # Blocks of `block` gate rows alternate with the matching up rows, so a
        # product's epilogue finds both halves of a gated pair in one tile.
        g, u = weights["gate_proj.weight"], weights["up_proj.weight"]
        i, h, b = self.intermediate_size, self.hidden_size, self.block
        fused = torch.stack([g.reshape(i // b, b, h), u.reshape(i // b, b, h)], dim=1).reshape(2 * i, h)
        self.gate_up = LinearWeight(fused)
        self.down = LinearWeight(weights["down_proj.weight"])

    def forward(self, x, ctx, residual):
        if self.activation == "clamped_gate":
            both = self.gate_up(x, out_dtype=torch.float32)
            gated = ops.clamped_gate_mul(both, self.block, self.limit, self.alpha, out_dtype=x.dtype)
            return self.down(gated, epilogue=ops.ADD, out=residual, ctx=ctx)
        if self.activation == "gelu_tanh":
            gated = ops.gelu_tanh_mul(self.gate_up(x, out_dtype=torch.float32), self.block, out_dtype=x.dtype)
            return self.down(gated, epilogue=ops.ADD, out=residual, ctx=ctx)
        if self.block == GATE_BLOCK and self.gate_up.supports_fused_gate(x.dtype):
            gated = self.gate_up(x, epilogue=ops.SILU_GATE)
        else:
            gated = ops.silu_mul(self.gate_up(x), self.block)
        return self.down(gated, epilogue=ops.ADD, out=residual, ctx=ctx)


@register_feed_forward("mlp")
class PlainMLP(FeedForward):
    """down( act(x Wu^T) ) without a gate; activation "relu_squared": act(z) = max(z, 0)^2. The
    first product keeps its float32 sums up to the activation (squaring doubles a rounding's
    relative size)."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu_squared"):
        if activation != "relu_squared":
            raise UnsupportedError(f"feed-forward activation {activation!r}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.up: Optional[LinearWeight] = None
        self.down: Optional[LinearWeight] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {"up_proj.weight": TensorSpec((i, h)), "down_proj.weight": TensorSpec((h, i))}

    def bind(self, weights, runtime) -> None:
        self.up = LinearWeight(weights["up_proj.weight"])
        self.down = LinearWeight(weights["down_proj.weight"])

    def forward(self, x, ctx, residual):
        inner = ops.relu_squared(self.up(x, out_dtype=torch.float32), x.dtype)
        return self.down(inner, epilogue=ops.ADD, out=residual, ctx=ctx)

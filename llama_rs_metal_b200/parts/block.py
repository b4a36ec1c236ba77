"""Arrangements of a layer's parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import InvalidError
from ..kernels import ops
from ..registry import register_block
from ..weights.loader import TensorSpec
from .base import Block, CompositeRequest, StateRequest
from .norm import StreamCast

STREAM_ITSELF = StreamCast()  # what a block whose sublayers read the stream itself has for an entry norm


@register_block("pre_norm")
class PreNormBlock(Block):
    """hidden += mixer(norm(hidden)); hidden += feed_forward(norm(hidden))
    (crates/model-runtime/src/execute.rs:24,196-199,236)."""

    graph_safe = True

    @property
    def folds_pending_on_entry(self) -> bool:
        return self.mixer_norm.folds_pending

    def forward(self, hidden, ctx, cache):
        after = ctx.next_folds_pending  # what comes after this block (the model says)
        x = self.mixer_norm.forward(hidden, ctx)
        # the mixer's output goes straight into the second norm: if that norm adds pending
        # partial sums itself, the mixer's last product may leave its K slices unadded
        ctx.may_defer = self.feed_forward_norm.folds_pending
        hidden = self.mixer.forward(x, ctx, cache, residual=hidden)
        ctx.may_defer = False
        x = self.feed_forward_norm.forward(hidden, ctx)
        ctx.may_defer = after
        hidden = self.feed_forward.forward(x, ctx, residual=hidden)
        ctx.may_defer = False
        return hidden


@register_block("pre_norm_mixer")
class PreNormMixerBlock(Block):
    """hidden += mixer(norm(hidden)): a layer without a feed-forward."""

    graph_safe = True
    roles = {"mixer": "mixer", "mixer_norm": "norm"}

    @property
    def folds_pending_on_entry(self) -> bool:
        return self.mixer_norm.folds_pending

    def forward(self, hidden, ctx, cache):
        after = ctx.next_folds_pending
        x = self.mixer_norm.forward(hidden, ctx)
        ctx.may_defer = after
        hidden = self.mixer.forward(x, ctx, cache, residual=hidden)
        ctx.may_defer = False
        return hidden


class _ScaledPreNormBlock(Block):
    """Pre-norm sublayers whose outputs enter the stream under a factor per channel:
    hidden += mult * scale * sublayer(norm(hidden)), with `scale` a stored vector per sublayer
    (`layer_scale`; tensors `mixer_scale`, `feed_forward_scale`) and `mult` one number for the model.
    A sublayer's output stays float32 up to the addition. With `token_shift` the mixer reads
    h + (h' - h) * shift instead of its norm's output h, h' being the previous token's h (zeros for
    a sequence's first token; tensor `shift`); the last h of every sequence is state of the layer,
    kept beside the mixer's own. The pass that adds a sublayer's output also applies the norm that
    comes next (the feed-forward's, or the next block's first norm when that block takes it, handed
    over through StepContext.normed)."""

    graph_safe = True

    def __init__(self, hidden_size: int, residual_mult: float = 1.0, layer_scale: bool = False,
                 token_shift: bool = False, **parts):
        super().__init__(**parts)
        self.hidden_size, self.residual_mult = int(hidden_size), float(residual_mult)
        self.layer_scale, self.token_shift = bool(layer_scale), bool(token_shift)
        self.factors: Dict[str, torch.Tensor] = {}
        self.shift: Optional[torch.Tensor] = None

    @property
    def folds_pending_on_entry(self) -> bool:
        return self.mixer_norm.folds_pending

    def tensors(self) -> Dict[str, TensorSpec]:
        out = {}
        if self.layer_scale:
            out.update({role + "_scale": TensorSpec((self.hidden_size,)) for role in ("mixer", "feed_forward")
                        if role in self.parts})
        if self.token_shift:
            out["shift"] = TensorSpec((self.hidden_size,))
        return out

    def bind(self, weights, runtime) -> None:
        for role in ("mixer", "feed_forward"):
            if role in self.parts:
                scale = weights[role + "_scale"].to(torch.float32) if self.layer_scale else \
                    torch.ones(self.hidden_size, dtype=torch.float32, device=runtime.device)
                self.factors[role] = (scale * self.residual_mult).contiguous()
        if self.token_shift:
            self.shift = weights["shift"].to(torch.float32).contiguous()

    def cache_request(self):
        request = self.mixer.cache_request()
        if not self.token_shift:
            return request
        return CompositeRequest((request, StateRequest((1, self.hidden_size), torch.float32)))

    @property
    def entry_norm(self):
        return self.mixer_norm

    def _add(self, hidden, y, role, then, ctx):
        """hidden += factor * y; returns then.forward(hidden) of the updated stream (None without `then`)."""
        from .norm import RMSNorm
        if isinstance(then, RMSNorm) and then.weight is not None and ctx.pending is None:
            return ops.scaled_add_norm_(hidden, y, self.factors[role], then.weight, then.eps, ctx.runtime.dtype)
        ops.scaled_add_(hidden, y, self.factors[role])
        return then.forward(hidden, ctx) if then is not None else None

    def _mixer_half(self, hidden, ctx, cache, then):
        x = ctx.take_normed(self.mixer_norm)
        if x is None:
            x = self.mixer_norm.forward(hidden, ctx)
        if self.token_shift:
            if cache is None or not ctx.entry.writes_cache:
                raise InvalidError("a layer with token shift keeps state of its own")
            cache, last = cache
            x = ops.token_shift(x, self.shift, last.state, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots)
        y = self.mixer.forward(x, ctx, cache, residual=None)
        return self._add(hidden, y, "mixer", then, ctx)


@register_block("scaled_pre_norm")
class ScaledPreNormBlock(_ScaledPreNormBlock):
    """A mixer and a feed-forward, each behind a norm, each added under its factor."""

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        x = self._mixer_half(hidden, ctx, cache, self.feed_forward_norm)
        y = self.feed_forward.forward(x, ctx, residual=None)
        normed = self._add(hidden, y, "feed_forward", following, ctx)
        ctx.normed = (following, normed) if following is not None else None
        return hidden


@register_block("scaled_pre_norm_mixer")
class ScaledPreNormMixerBlock(_ScaledPreNormBlock):
    """The same for a layer without a feed-forward."""

    roles = {"mixer": "mixer", "mixer_norm": "norm"}

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        normed = self._mixer_half(hidden, ctx, cache, following)
        ctx.normed = (following, normed) if following is not None else None
        return hidden


class _SandwichBlock(Block):
    """Norms on both sides of every sublayer, and a factor on what a sublayer adds:
    hidden += mult * post_norm(sublayer(pre_norm(hidden))). The sublayer's output stays float32
    up to its norm. The post-norm's pass also applies the norm that comes next (the
    feed-forward's pre-norm, or the next block's first norm when that block takes it)."""

    graph_safe = True

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    @property
    def entry_norm(self):
        return self.mixer_norm

    def _mixer_half(self, hidden, ctx, cache, then):
        x = ctx.take_normed(self.mixer_norm)
        if x is None:
            x = self.mixer_norm.forward(hidden, ctx)
        y = self.mixer.forward(x, ctx, cache, residual=None)
        return self.mixer_post_norm.add_into(hidden, y, ctx, self.residual_mult, then)


@register_block("sandwich_norm")
class SandwichNormBlock(_SandwichBlock):
    """A mixer and a feed-forward, each between two norms."""

    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward_post_norm": "norm"}

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        x = self._mixer_half(hidden, ctx, cache, self.feed_forward_norm)
        y = self.feed_forward.forward(x, ctx, residual=None)
        normed = self.feed_forward_post_norm.add_into(hidden, y, ctx, self.residual_mult, following)
        ctx.normed = (following, normed) if following is not None else None
        return hidden


@register_block("sandwich_norm_mixer")
class SandwichNormMixerBlock(_SandwichBlock):
    """A mixer between two norms: a layer without a feed-forward."""

    roles = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm"}

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        normed = self._mixer_half(hidden, ctx, cache, following)
        ctx.normed = (following, normed) if following is not None else None
        return hidden


class _PostNormBlock(Block):
    """A norm on each sublayer's output only, and a factor on what it adds:
    hidden += mult * post_norm(sublayer(hidden)). The sublayers read the stream itself (its rounding
    under bfloat16 activations, which the pass of the norm before writes beside the float32 row);
    a sublayer's output stays float32 up to its norm. While a sublayer runs, ctx.stream is the
    float32 stream its input is the rounding of."""

    graph_safe = True

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    @property
    def entry_norm(self):
        return STREAM_ITSELF

    def _mixer_half(self, hidden, ctx, cache, then):
        x = ctx.take_normed(STREAM_ITSELF)
        if x is None:
            x = STREAM_ITSELF.forward(hidden, ctx)
        ctx.stream = hidden
        y = self.mixer.forward(x, ctx, cache, residual=None)
        return self.mixer_post_norm.add_into(hidden, y, ctx, self.residual_mult, then)


@register_block("post_norm")
class PostNormBlock(_PostNormBlock):
    """A mixer and a feed-forward, each with a norm behind it."""

    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_post_norm": "norm",
             "feed_forward_post_norm": "norm"}

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        x = self._mixer_half(hidden, ctx, cache, STREAM_ITSELF)
        y = self.feed_forward.forward(x, ctx, residual=None)
        normed = self.feed_forward_post_norm.add_into(hidden, y, ctx, self.residual_mult, following)
        ctx.stream = None
        ctx.normed = (following, normed) if following is not None else None
        return hidden


@register_block("post_norm_mixer")
class PostNormMixerBlock(_PostNormBlock):
    """A mixer with a norm behind it: a layer without a feed-forward."""

    roles = {"mixer": "mixer", "mixer_post_norm": "norm"}

    def forward(self, hidden, ctx, cache):
        following = ctx.next_entry_norm
        normed = self._mixer_half(hidden, ctx, cache, following)
        ctx.stream = None
        ctx.normed = (following, normed) if following is not None else None
        return hidden

"""Configuration of the Tarupel decoder, read from its own config.json keys.

    {"architecture": "Tarupel", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "residual_mult": m, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "general_delta" | "attention" | "attention_2", "mixer": {...}, "mlp": {...} | null}, ...]}

A general_delta mixer: heads, dim (and, for random weights only, decay_rank: the checkpoint's
tensors give it otherwise). An attention mixer: heads, kv_heads, dim, vdim, scale, conv (taps),
rot {dims, base}, mask {size} (the chunk). An attention_2 mixer: heads, kv_heads, dim, vdim, scale,
rot {dims, base}, mask {size} (the window); without rot nothing is rotated, without mask every
earlier key is seen. A feed-forward is {"kind": "dense", "ff"} or {"kind":
"moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "shared":
{"ff"}}; scale, groups and shared may be absent, and so may loop, embedding and residual_mult.
Every size and every constant that can differ between models comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import InvalidError, UnsupportedError
from .base import read_int
from .kikalix import _positive, _real, _table


@dataclass(frozen=True)
class GeneralDeltaConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "GeneralDeltaConfig":
        rank = read_int(m, "decay_rank", None)
        return cls(_positive(m, "heads", where), _positive(m, "dim", where), rank if rank else None)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out


@dataclass(frozen=True)
class MaskedAttentionConfig:
    """Both attention mixers: `conv` is None for attention_2 (which has no convolution), and `span` is
    the chunk's size for attention, the window's for attention_2."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    span: Optional[int]
    conv: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str, with_conv: bool) -> "MaskedAttentionConfig":
        heads, kv_heads, dim, vdim = (_positive(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim"))
        if heads % kv_heads:
            raise InvalidError(f"config.{where}heads must be a multiple of kv_heads")
        rot = m.get("rot") if isinstance(m.get("rot"), Mapping) else {}
        dims, base = read_int(rot, "dims", 0), 10000.0
        if dims:
            base = _real(rot, "base", where + "rot.")
        if dims % 2 or dims > dim or base <= 0:
            raise InvalidError(f"config.{where}rot: dims must be even and at most dim, base positive")
        span = _positive(m["mask"], "size", where + "mask.") if isinstance(m.get("mask"), Mapping) else None
        conv = _positive(m, "conv", where) if with_conv else None
        return cls(heads, kv_heads, dim, vdim, _real(m, "scale", where), dims, base, span, conv)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "rot": {"dims": self.rot_dims, "base": self.rot_base}}
        if self.span is not None:
            out["mask"] = {"size": self.span}
        if self.conv is not None:
            out["conv"] = self.conv
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                       # "dense" | "moe"
    ff: int                         # inner width (of one expert, for "moe")
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    groups: Optional[Tuple[int, int]] = None   # (count, keep)
    shared_ff: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = m.get("kind")
        if kind == "dense":
            return cls("dense", _positive(m, "ff", where))
        if kind != "moe":
            raise UnsupportedError(f"config.{where}kind {kind!r}: built are \"dense\" and \"moe\"")
        ff = _positive(_table(m, "expert", where), "ff", where + "expert.")
        router = _table(m, "router", where)
        experts, top = _positive(router, "experts", where + "router."), _positive(router, "top", where + "router.")
        scale = _real(router, "scale", where + "router.") if "scale" in router else 1.0
        groups = None
        if isinstance(router.get("groups"), Mapping):
            g = router["groups"]
            groups = (_positive(g, "count", where + "router.groups."), _positive(g, "keep", where + "router.groups."))
            if experts % groups[0] or groups[1] > groups[0]:
                raise InvalidError(f"config.{where}router.groups: count must divide experts, keep at most count")
        reachable = experts if groups is None else groups[1] * (experts // groups[0])
        if top > reachable:
            raise InvalidError(f"config.{where}router.top exceeds the experts that can be chosen")
        shared = m.get("shared")
        shared_ff = _positive(shared, "ff", where + "shared.") if isinstance(shared, Mapping) else None
        return cls("moe", ff, experts, top, scale, groups, shared_ff)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXERS = {"general_delta": lambda m, where: GeneralDeltaConfig.read(m, where),
          "attention": lambda m, where: MaskedAttentionConfig.read(m, where, True),
          "attention_2": lambda m, where: MaskedAttentionConfig.read(m, where, False)}


@dataclass(frozen=True)
class TarupelLayer:
    kind: str  # a key of MIXERS
    mixer: Any
    mlp: Optional[FeedForwardConfig]

    def to_dict(self) -> dict:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class TarupelConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[TarupelLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    architecture: str = "Tarupel"

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "TarupelConfig":
        vocab, width = _positive(root, "vocab", ""), _positive(root, "width", "")
        eps = _real(_table(root, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise InvalidError("config.norm.eps must be positive")
        listed = root.get("layers")
        if not isinstance(listed, list) or not listed or len(listed) > 1024:
            raise InvalidError("config.layers must list 1 to 1024 layers")
        layers = []
        for i, item in enumerate(listed):
            where = f"layers[{i}]."
            if not isinstance(item, Mapping):
                raise InvalidError(f"config.layers[{i}] must be an object")
            kind = item.get("type")
            if kind not in MIXERS:
                raise UnsupportedError(f"config.{where}type {kind!r}: built are {', '.join(sorted(MIXERS))}")
            mixer = MIXERS[kind](_table(item, "mixer", where), where + "mixer.")
            mlp = item.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise InvalidError(f"config.{where}mlp must be an object or null")
            layers.append(TarupelLayer(kind, mixer, FeedForwardConfig.read(mlp, where + "mlp.") if mlp is not None else None))
        embedding = root.get("embedding")
        scale = _real(embedding, "scale", "embedding.") if isinstance(embedding, Mapping) and "scale" in embedding else 1.0
        mult = _real(root, "residual_mult", "") if "residual_mult" in root else 1.0
        start, stop, times = 0, 0, 1
        loop = root.get("loop")
        if isinstance(loop, Mapping):
            start, stop = read_int(loop, "start"), read_int(loop, "stop")
            times = _positive(loop, "times", "loop.")
            if not 0 <= start <= stop <= len(layers) or times > 1024:
                raise InvalidError("config.loop: 0 <= start <= stop <= number of layers, times at most 1024")
        return cls(vocab, width, eps, scale, mult, tuple(layers), start, stop, times)

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.loops:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

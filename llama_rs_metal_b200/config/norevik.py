"""Configuration of the Norevik decoder, read from its own config.json keys.

    {"architecture": "Norevik", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "mamba2" | "latent_attention" | "mlstm", "mixer": {...}, "mlp": {...} | null}, ...]}

A mamba2 mixer: heads, vdim, state, groups, conv (taps), norm_groups. A latent_attention mixer:
heads, dim, rot_dim, vdim, kv_rank, scale, rot {dims, base}. An mlstm mixer: heads, dim, vdim,
gate_cap. A feed-forward is {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router":
{"experts", "top", "identity", "groups": {"count", "keep"}}, "shared": {"ff"}}; identity, groups and
shared may be absent. Every size and every constant that can differ between models comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import InvalidError, UnsupportedError
from .base import read_int
from .kikalix import _positive, _real, _table


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "StateSpaceConfig":
        heads, vdim, state, groups, conv = (_positive(m, k, where) for k in ("heads", "vdim", "state", "groups", "conv"))
        norm_groups = read_int(m, "norm_groups", 1)
        if heads % groups:
            raise InvalidError(f"config.{where}heads must be a multiple of groups")
        if norm_groups <= 0 or (heads * vdim) % norm_groups:
            raise InvalidError(f"config.{where}norm_groups must divide heads * vdim")
        return cls(heads, vdim, state, groups, conv, norm_groups)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class SinkLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "SinkLatentConfig":
        heads, dim, rot_dim, vdim, kv_rank = (_positive(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        rot = _table(m, "rot", where)
        if read_int(rot, "dims", rot_dim) != rot_dim or rot_dim % 2:
            raise InvalidError(f"config.{where}rot.dims must equal rot_dim, an even number")
        base = _real(rot, "base", where + "rot.")
        if base <= 0:
            raise InvalidError(f"config.{where}rot.base must be positive")
        return cls(heads, dim, rot_dim, vdim, kv_rank, _real(m, "scale", where), base)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"dims": self.rot_dim, "base": self.rot_base}}


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "MatrixMemoryConfig":
        heads, dim, vdim = (_positive(m, k, where) for k in ("heads", "dim", "vdim"))
        cap = _real(m, "gate_cap", where)
        if cap <= 0:
            raise InvalidError(f"config.{where}gate_cap must be positive")
        return cls(heads, dim, vdim, cap)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                       # "dense" | "moe"
    ff: int                         # inner width (of one expert, for "moe")
    experts: int = 0
    top: int = 0
    identity: int = 0
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
        identity = read_int(router, "identity", 0)
        outputs = experts + identity
        groups = None
        if isinstance(router.get("groups"), Mapping):
            g = router["groups"]
            groups = (_positive(g, "count", where + "router.groups."), _positive(g, "keep", where + "router.groups."))
            if outputs % groups[0] or groups[1] > groups[0]:
                raise InvalidError(f"config.{where}router.groups: count must divide experts + identity, keep at most count")
        reachable = outputs if groups is None else groups[1] * (outputs // groups[0])
        if top > reachable:
            raise InvalidError(f"config.{where}router.top exceeds the experts that can be chosen")
        shared = m.get("shared")
        shared_ff = _positive(shared, "ff", where + "shared.") if isinstance(shared, Mapping) else None
        return cls("moe", ff, experts, top, identity, groups, shared_ff)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top, "identity": self.identity}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXERS = {"mamba2": StateSpaceConfig, "latent_attention": SinkLatentConfig, "mlstm": MatrixMemoryConfig}


@dataclass(frozen=True)
class NorevikLayer:
    kind: str  # a key of MIXERS
    mixer: Any
    mlp: Optional[FeedForwardConfig]

    def to_dict(self) -> dict:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class NorevikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[NorevikLayer, ...]
    architecture: str = "Norevik"

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "NorevikConfig":
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
            mixer = MIXERS[kind].read(_table(item, "mixer", where), where + "mixer.")
            mlp = item.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise InvalidError(f"config.{where}mlp must be an object or null")
            layers.append(NorevikLayer(kind, mixer, FeedForwardConfig.read(mlp, where + "mlp.") if mlp is not None else None))
        embedding = root.get("embedding")
        scale = _real(embedding, "scale", "embedding.") if isinstance(embedding, Mapping) and "scale" in embedding else 1.0
        return cls(vocab, width, eps, scale, tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "layers": [layer.to_dict() for layer in self.layers]}

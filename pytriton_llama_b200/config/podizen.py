"""Typed configuration of the Podizen decoder, read from its config.json.

A Podizen model is a list of layers of two types.  ``attention`` is grouped-query softmax attention
without any rotation: a bias that grows with the distance between query and key is taken off the
scores, a sliding window limits the keys, and the heads pass a sigmoid gate before the output
projection.  ``parallel`` runs two mixers on the same input and takes the mean of their outputs,
each normed over the model width: on the left softmax attention with a per-head query and key norm,
a rotation of half-split pairs and a sliding window behind which every whole block of ``mask.pool``
positions is seen as one mean key and mean value; on the right retention, linear attention with one
fixed decay per head.  A layer's feed-forward is a routed mixture of gated experts (softmax scores,
experts chosen among the best groups of neighbours, weights renormalised) with an optional shared
expert, or absent.  Every sub-layer has a norm before and a norm after it, and what a layer hands on
is a learned weighted sum of the embedding output and all layer results so far.  Keys of the file:

    architecture, vocab, width, norm.eps,
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp (null, or {kind: moe, expert.ff,
    router.experts, router.top, router.groups.{count, keep}, shared.ff})
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

from .lilenex import _optional_int
from .llama import ConfigError
from .tibepel import _need, _positive_int


@dataclass(frozen=True)
class HalfRotation:
    """Entry i of the first ``dims`` of a head is paired with entry i + dims/2; the pair turns by
    position * base^(-2i/dims)."""
    dims: int
    base: float

    @classmethod
    def from_dict(cls, d, where, head_dim) -> Optional["HalfRotation"]:
        if d is None:
            return None
        dims = _positive_int(d, "dims", where)
        if dims % 2 or dims > head_dim:
            raise ConfigError(f"{where}dims={dims} must be even and at most the head size {head_dim}")
        base = float(_need(d, "base", where))
        if not base > 0:
            raise ConfigError(f"{where}base must be positive, got {base}")
        return cls(dims, base)

    def to_dict(self):
        return {"base": self.base, "dims": self.dims}


def _heads(d, where) -> Tuple[int, int]:
    heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"{where}heads={heads} is no multiple of kv_heads={kv}")
    return heads, kv


@dataclass(frozen=True)
class GatedAttentionConfig:
    """Mixer of an ``attention`` layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                 # 0: every earlier position is seen

    @classmethod
    def from_dict(cls, d, where) -> "GatedAttentionConfig":
        heads, kv = _heads(d, where)
        return cls(heads, kv, _positive_int(d, "dim", where), _positive_int(d, "vdim", where), float(_need(d, "scale", where)),
                   _optional_int(d.get("mask") or {}, "size", where + "mask."))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class PooledAttentionConfig:
    """Left member of a ``parallel`` layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                 # 0: every earlier position is seen (and no block is pooled)
    pool: int                   # 0: what the window has passed is not seen at all
    rot: Optional[HalfRotation]

    @classmethod
    def from_dict(cls, d, where) -> "PooledAttentionConfig":
        heads, kv = _heads(d, where)
        dim = _positive_int(d, "dim", where)
        mask = d.get("mask") or {}
        return cls(heads, kv, dim, _positive_int(d, "vdim", where), float(_need(d, "scale", where)),
                   _optional_int(mask, "size", where + "mask."), _optional_int(mask, "pool", where + "mask."),
                   HalfRotation.from_dict(d.get("rot"), where + "rot.", dim))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            d["mask"] = {"size": self.window, **({"pool": self.pool} if self.pool else {})}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class RetentionConfig:
    """Right member of a ``parallel`` layer."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]    # one per head
    rot: Optional[HalfRotation]

    @classmethod
    def from_dict(cls, d, where) -> "RetentionConfig":
        heads, dim = _positive_int(d, "heads", where), _positive_int(d, "dim", where)
        decay = _need(d, "decay", where)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"{where}decay must list one number for each of the {heads} heads")
        decay = tuple(float(x) for x in decay)
        if not all(0.0 <= x <= 1.0 for x in decay):
            raise ConfigError(f"{where}decay must lie in [0, 1]")
        return cls(heads, dim, _positive_int(d, "vdim", where), decay, HalfRotation.from_dict(d.get("rot"), where + "rot.", dim))

    def to_dict(self):
        d = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: PooledAttentionConfig
    right: RetentionConfig

    @classmethod
    def from_dict(cls, d, where) -> "ParallelMixerConfig":
        return cls(PooledAttentionConfig.from_dict(_need(d, "left", where), where + "left."),
                   RetentionConfig.from_dict(_need(d, "right", where), where + "right."))

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class GroupedMoeConfig:
    ff: int
    experts: int
    top: int
    groups: int                 # 1: no groups
    keep: int                   # groups whose experts may be chosen
    shared_ff: int              # 0: no shared expert

    @classmethod
    def from_dict(cls, d, where) -> Optional["GroupedMoeConfig"]:
        if d is None:
            return None
        kind = _need(d, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}kind={kind!r} is not supported (known: moe)")
        router = _need(d, "router", where)
        experts, top = _positive_int(router, "experts", where + "router."), _positive_int(router, "top", where + "router.")
        grp = router.get("groups") or {}
        groups = _optional_int(grp, "count", where + "router.groups.", 1) or 1
        keep = _optional_int(grp, "keep", where + "router.groups.", groups) or groups
        if experts % groups:
            raise ConfigError(f"{where}router.experts={experts} is no multiple of router.groups.count={groups}")
        if keep > groups:
            raise ConfigError(f"{where}router.groups.keep={keep} exceeds router.groups.count={groups}")
        if top > keep * (experts // groups):
            raise ConfigError(f"{where}router.top={top} exceeds the {keep * (experts // groups)} experts of the kept groups")
        shared = d.get("shared")
        return cls(_positive_int(_need(d, "expert", where), "ff", where + "expert."), experts, top, groups, keep,
                   _positive_int(shared, "ff", where + "shared.") if shared else 0)

    def to_dict(self):
        router = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        d = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class PodizenLayerConfig:
    type: str
    mixer: Union[GatedAttentionConfig, ParallelMixerConfig]
    mlp: Optional[GroupedMoeConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


_MIXERS = {"attention": GatedAttentionConfig, "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class PodizenConfig:
    vocab: int
    width: int
    layers: Tuple[PodizenLayerConfig, ...]
    norm_eps: float
    initializer_range: float = 0.02
    eos_token_id: Union[None, int, List[int]] = None

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "PodizenConfig":
        raw_layers = _need(data, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = _need(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type={kind!r} is not supported (known: {sorted(_MIXERS)})")
            layers.append(PodizenLayerConfig(kind, _MIXERS[kind].from_dict(_need(L, "mixer", where), where + "mixer."),
                                             GroupedMoeConfig.from_dict(L.get("mlp"), where + "mlp.")))
        eps = float(_need(_need(data, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        eos = data.get("eos_token_id")
        return cls(vocab=_positive_int(data, "vocab", ""), width=_positive_int(data, "width", ""), layers=tuple(layers),
                   norm_eps=eps, initializer_range=float(data.get("initializer_range", 0.02)),
                   eos_token_id=[int(e) for e in eos] if isinstance(eos, (list, tuple)) else eos)

    @classmethod
    def from_folder(cls, folder: Union[str, Path]) -> "PodizenConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": "Podizen", "layers": [L.to_dict() for L in self.layers], "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width, "initializer_range": self.initializer_range}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    @property
    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        return [self.eos_token_id] if isinstance(self.eos_token_id, int) else list(self.eos_token_id)

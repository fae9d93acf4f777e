"""Typed configuration of the Sogalix decoder, read from its config.json.

A Sogalix model is a list of layers of three types.  ``general_delta`` is a linear-attention mixer
whose matrix state decays per key channel and loses, per key channel, a learned share of what it
holds along the new key before the new value is written.  ``attention`` is grouped-query softmax
attention without rotation whose denominator has one more term of score zero and whose queries
grow with the logarithm of their position in steps.  ``latent_attention`` projects queries and
keys/values through small latents: only the key/value latent and one rotated key part shared by all
heads are kept per position, and a layer may read what an earlier layer keeps (``kv_from``).  A
layer's feed-forward is dense with the xIELU activation, or absent.  Every norm of the residual
stream is a layer norm with weight and bias; the embedding passes one too.  Keys of the file:

    architecture, vocab, width, norm.eps, layers[i].type, layers[i].mixer.{...},
    layers[i].mlp (null, or {kind: dense, ff})
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

from .lilenex import PairRotation, _optional_int
from .llama import ConfigError
from .tibepel import _need, _positive_int


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    rank: int = 0           # inner size of the decay projection for weights drawn at random (0: 16); a checkpoint's tensors say their own

    @classmethod
    def from_dict(cls, d, where) -> "DeltaMixerConfig":
        return cls(_positive_int(d, "heads", where), _positive_int(d, "dim", where), _optional_int(d, "rank", where))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads}
        if self.rank:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class QueryTemperature:
    """Queries at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)."""
    coef: float
    every: int

    @classmethod
    def from_dict(cls, d, where) -> Optional["QueryTemperature"]:
        if d is None:
            return None
        return cls(float(_need(d, "coef", where)), _positive_int(d, "every", where))

    def to_dict(self):
        return {"coef": self.coef, "every": self.every}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[QueryTemperature]

    @classmethod
    def from_dict(cls, d, where) -> "SinkAttentionConfig":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}heads={heads} is no multiple of kv_heads={kv}")
        return cls(heads, kv, _positive_int(d, "dim", where), _positive_int(d, "vdim", where), float(_need(d, "scale", where)),
                   QueryTemperature.from_dict(d.get("q_temp"), where + "q_temp."))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.q_temp is not None:
            d["q_temp"] = self.q_temp.to_dict()
        return d


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                    # entries of a query/key head that are not rotated
    rot_dim: int                # rotated entries of a query head; the one rotated key part that all heads share
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: PairRotation
    kv_from: Optional[int]      # the layer whose latent and rotated key part this one reads instead of its own

    @classmethod
    def from_dict(cls, d, where) -> "LatentAttentionConfig":
        rot_dim = _positive_int(d, "rot_dim", where)
        rot = PairRotation.from_dict(_need(d, "rot", where), where + "rot.", rot_dim)
        if rot.scaling is not None:
            raise ConfigError(f"{where}rot.scaling is not part of this design")
        src = d.get("kv_from")
        if src is not None and (isinstance(src, bool) or int(src) != src or int(src) < 0):
            raise ConfigError(f"{where}kv_from must name a layer, got {src!r}")
        return cls(_positive_int(d, "heads", where), _positive_int(d, "dim", where), rot_dim, _positive_int(d, "vdim", where),
                   _positive_int(d, "kv_rank", where), _positive_int(d, "q_rank", where), float(_need(d, "scale", where)), rot,
                   None if src is None else int(src))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot": self.rot.to_dict(),
             "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


def _mlp_from_dict(d, where):
    if d is None:
        return None
    kind = _need(d, "kind", where)
    if kind != "dense":
        raise ConfigError(f"{where}kind={kind!r} is not supported (known: dense)")
    return DenseMlpConfig(_positive_int(d, "ff", where))


@dataclass(frozen=True)
class SogalixLayerConfig:
    type: str
    mixer: Union[DeltaMixerConfig, SinkAttentionConfig, LatentAttentionConfig]
    mlp: Optional[DenseMlpConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


_MIXERS = {"general_delta": DeltaMixerConfig, "attention": SinkAttentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class SogalixConfig:
    vocab: int
    width: int
    layers: Tuple[SogalixLayerConfig, ...]
    norm_eps: float
    initializer_range: float = 0.02
    eos_token_id: Union[None, int, List[int]] = None

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "SogalixConfig":
        raw_layers = _need(data, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = _need(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type={kind!r} is not supported (known: {sorted(_MIXERS)})")
            layers.append(SogalixLayerConfig(kind, _MIXERS[kind].from_dict(_need(L, "mixer", where), where + "mixer."),
                                             _mlp_from_dict(L.get("mlp"), where + "mlp.")))
        for i, L in enumerate(layers):
            src = getattr(L.mixer, "kv_from", None)
            if src is None:
                continue
            where = f"layers[{i}].mixer."
            if src >= i or layers[src].type != "latent_attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"{where}kv_from={src} must name an earlier latent_attention layer that keeps a latent of its own")
            a, b = L.mixer, layers[src].mixer
            if (a.kv_rank, a.rot_dim, a.rot) != (b.kv_rank, b.rot_dim, b.rot):
                raise ConfigError(f"{where}kv_rank, rot_dim and rot must equal those of layer {src}")
        eps = float(_need(_need(data, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        eos = data.get("eos_token_id")
        return cls(vocab=_positive_int(data, "vocab", ""), width=_positive_int(data, "width", ""), layers=tuple(layers),
                   norm_eps=eps, initializer_range=float(data.get("initializer_range", 0.02)),
                   eos_token_id=[int(e) for e in eos] if isinstance(eos, (list, tuple)) else eos)

    @classmethod
    def from_folder(cls, folder: Union[str, Path]) -> "SogalixConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": "Sogalix", "layers": [L.to_dict() for L in self.layers], "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width, "initializer_range": self.initializer_range}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    @property
    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        return [self.eos_token_id] if isinstance(self.eos_token_id, int) else list(self.eos_token_id)

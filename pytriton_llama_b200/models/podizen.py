"""The Podizen decoder (architecture name "Podizen") as a ``ModelSpec``.

Layer i (tensors ``l<i>.*``) has a norm before and after each sub-layer (``norm1``, ``norm1b`` around
the mixer, ``norm2``, ``norm2b`` around the feed-forward) and hands on a weighted sum of the embedding
output and all layer results so far (``dwa`` [i + 2]).  The mixer is a windowed softmax attention with
a distance bias and a sigmoid gate (``attention``), or the mean of the normed outputs of a windowed
attention that sees pooled blocks behind its window and of a retention (``parallel``).  The
feed-forward is a routed mixture of gated experts with grouped softmax routing and a shared expert, or
absent.  The logits come from the embedding table.
"""
from __future__ import annotations

from ..config.podizen import (GatedAttentionConfig, GroupedMoeConfig, HalfRotation, ParallelMixerConfig, PodizenConfig,
                              PooledAttentionConfig, RetentionConfig)
from ..parts.base import PartSpec
from .spec import ModelSpec, RunEntry

DISTANCE_BIAS_EXPONENT = 8.0      # head h of H takes slope 2^(-8 (h + 1) / H) times the distance off its scores


def _names(prefix: str, *locals_: str):
    return {n: prefix + n for n in locals_}


def _rotation(rot: HalfRotation, head_dim: int):
    if rot is None:
        return {}
    return {"position": PartSpec("rope", {"head_dim": head_dim, "theta": rot.base, "scaling": None, "rotary_dim": rot.dims})}


def _gated_attention(width: int, m: GatedAttentionConfig, p: str) -> PartSpec:
    return PartSpec("window_attention",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "scale": m.scale, "window": m.window, "qk_norm_eps": 0.0, "own_kv": True,
                     "distance_bias": DISTANCE_BIAS_EXPONENT, "gate": "sigmoid"},
                    _names(p, "q", "k", "v", "g", "o"), {"position": PartSpec("none")})


def _pooled_attention(width: int, m: PooledAttentionConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("window_attention",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "scale": m.scale, "window": m.window, "pool": m.pool, "qk_norm_eps": eps, "qk_norm": "per_head",
                     "own_kv": True},
                    _names(p, "q", "k", "v", "q.norm", "k.norm", "o"),
                    _rotation(m.rot, m.dim) or {"position": PartSpec("none")})


def _retention(width: int, m: RetentionConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("retention", {"hidden": width, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim,
                                  "decay": list(m.decay), "norm_eps": eps},
                    _names(p, "q", "k", "v", "g", "o"), _rotation(m.rot, m.dim))


def _parallel(width: int, m: ParallelMixerConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("parallel", {"hidden": width, "combine": "normed_mean", "norm_eps": eps},
                    {"left.out": p + "left.out", "right.out": p + "right.out"},
                    {"left": _pooled_attention(width, m.left, p + "left.", eps), "right": _retention(width, m.right, p + "right.", eps)})


def _feed_forward(width: int, m: GroupedMoeConfig, p: str) -> PartSpec:
    names = ["router"] + [f"e{i}.{w}" for i in range(m.experts) for w in ("gate", "up", "down")]
    if m.shared_ff:
        names += ["shared.gate", "shared.up", "shared.down"]
    return PartSpec("routed_experts", {"hidden": width, "inter": m.ff, "experts": m.experts, "top": m.top,
                                       "shared_inter": m.shared_ff, "scale_input": False, "score": "softmax",
                                       "groups": m.groups, "keep_groups": m.keep, "renormalise": True}, _names(p, *names))


def podizen_spec(cfg: PodizenConfig, norm_init: str = "ones") -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def norm(weight: str):
        return PartSpec("rmsnorm", {"width": W, "eps": eps, "init": norm_init}, {"weight": weight})

    layers, run_order = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        if isinstance(L.mixer, GatedAttentionConfig):
            mixer = _gated_attention(W, L.mixer, p + "mix.")
        else:
            mixer = _parallel(W, L.mixer, p + "mix.", eps)
        parts = {"norm1": norm(p + "norm1"), "mixer": mixer, "norm1b": norm(p + "norm1b")}
        if L.mlp is not None:
            parts.update({"norm2": norm(p + "norm2"), "ffn": _feed_forward(W, L.mlp, p + "mlp."), "norm2b": norm(p + "norm2b")})
        layers.append(PartSpec("sandwich_depth_average", {"index": i, "layers": len(cfg.layers), "width": W}, {"depth": p + "dwa"}, parts))
        run_order.append(RunEntry(layer=i, cache=i, write=True))
    return ModelSpec(architecture="Podizen", hidden_size=W, vocab_size=cfg.vocab, embedding="embed", layers=layers,
                     run_order=run_order, final_norm=norm("final.norm"), lm_head=None,
                     initializer_range=cfg.initializer_range, eos_token_ids=cfg.eos_token_ids)

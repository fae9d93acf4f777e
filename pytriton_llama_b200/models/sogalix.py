"""The Sogalix decoder (architecture name "Sogalix") as a ``ModelSpec``.

The stream starts as the layer norm (``embed.norm``) of embed[token].  Layer i (tensors ``l<i>.*``) is a
pre-norm block with layer norms that have a weight and a bias (``norm1``, ``norm1.b``, ...): a mixer,
then a dense feed-forward with the xIELU activation (absent where the layer has none).  The mixer is
a generalized delta rule (type ``general_delta``), a softmax attention without rotation that has a
sink term in its denominator and a query temperature (``attention``), or an attention through
latents that keeps one latent and one rotated key part per position (``latent_attention``; with
``kv_from`` it reads the cache entry of an earlier layer).  The logits come from ``final.norm`` and
the table ``head``.
"""
from __future__ import annotations

from ..config.sogalix import (DeltaMixerConfig, LatentAttentionConfig, SinkAttentionConfig, SogalixConfig)
from ..parts.base import PartSpec
from .spec import ModelSpec, RunEntry


def _names(prefix: str, *locals_: str):
    return {n: prefix + n for n in locals_}


def _general_delta(width: int, m: DeltaMixerConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("general_delta_rule",
                    {"hidden": width, "heads": m.heads, "head_dim": m.dim, "norm_eps": eps, "unit_eps": 1e-6, "decay_rank": m.rank},
                    _names(p, "r", "k", "v", "g", "a", "a.b", "w1", "w2", "w0", "norm", "o"))


def _sink_attention(width: int, m: SinkAttentionConfig, p: str) -> PartSpec:
    return PartSpec("window_attention",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "scale": m.scale, "window": 0, "keep_first": 0, "qk_norm_eps": 0.0, "own_kv": True, "sink": True,
                     "q_temp": None if m.q_temp is None else m.q_temp.to_dict()},
                    _names(p, "q", "k", "v", "o"))


def _latent_attention(width: int, m: LatentAttentionConfig, p: str, eps: float) -> PartSpec:
    own = m.kv_from is None
    names = ["dq", "dq.norm", "uq", "uk", "uv", "g", "o"] + (["dkv", "dkv.norm"] if own else [])
    position = PartSpec("rotary_pairs", {"head_dim": m.rot_dim, "dims": m.rot.dims, "base": m.rot.base, "scaling": None})
    return PartSpec("latent_attention",
                    {"hidden": width, "heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                     "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": eps, "own_kv": own},
                    _names(p, *names), {"position": position})


def sogalix_spec(cfg: SogalixConfig, norm_init: str = "ones") -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"width": W, "eps": eps, "init": norm_init}, {"weight": name, "bias": name + ".b"})

    layers, run_order = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        cache, write = i, True
        if isinstance(L.mixer, DeltaMixerConfig):
            mixer = _general_delta(W, L.mixer, p + "mix.", eps)
        elif isinstance(L.mixer, SinkAttentionConfig):
            mixer = _sink_attention(W, L.mixer, p + "mix.")
        else:
            mixer = _latent_attention(W, L.mixer, p + "mix.", eps)
            if L.mixer.kv_from is not None:
                cache, write = L.mixer.kv_from, False
        parts = {"norm1": norm(p + "norm1"), "mixer": mixer}
        if L.mlp is not None:
            parts["norm2"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("xielu_mlp", {"hidden": W, "inter": L.mlp.ff}, _names(p + "mlp.", "up", "down", "act"))
        layers.append(PartSpec("pre_norm", parts=parts))
        run_order.append(RunEntry(layer=i, cache=cache, write=write))
    return ModelSpec(architecture="Sogalix", hidden_size=W, vocab_size=cfg.vocab, embedding="embed", layers=layers,
                     run_order=run_order, final_norm=norm("final.norm"), lm_head="head", embedding_norm=norm("embed.norm"),
                     initializer_range=cfg.initializer_range, eos_token_ids=cfg.eos_token_ids)

"""Grouped-query softmax attention behind a sliding window that keeps the first positions, over the
paged cache.

q = W_q h, k = W_k h, v = W_v h.  With ``qk_norm_eps`` > 0 the whole query projection (all heads at
once) and the whole key projection are divided by their root mean square and multiplied by a weight
of their own size.  The nested ``position`` part then turns neighbouring pairs of every head
(``rotary_pairs``) or leaves them alone (``none``).  Query i sees key j <= i if i - j < ``window``
or j < ``keep_first`` (``window`` 0: every j <= i); a kept key was rotated by its own position like any other.
score = (q . k) * scale, softmax, heads of ``value_dim`` concatenated, W_o.

Two options change the scores.  ``sink``: the softmax has one more term of score 0 in its denominator
(a key that every query sees and that has no value), p_j = exp(s_j) / (1 + sum exp(s_j)).
``q_temp`` = {coef, every}: the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1);
the factor is applied to the float32 scores, which is the same thing.

Further options.  ``qk_norm`` "per_head": the norm runs over every head by itself with one weight of the
head's size for all query heads and one for all key heads.  A ``position`` part that turns the pairs (i, i + rot/2)
(``rope``) goes with the per-head norm or with none.  ``distance_bias`` = c > 0: slope_h * (i - j) is taken off the
score of query i and key j, slope_h = 2^(-c (h + 1) / heads) for head h = 0 ..  ``gate`` "sigmoid": the concatenated
heads are multiplied by sigmoid(W_g h) before W_o.  ``pool`` = P > 0 (with a window of n): beside the window's keys,
query i sees one key and one value for every block b of P positions with bP + P - 1 <= i - n, the means of the
block's keys (as the cache holds them) and values, in the same softmax; positions that the window has passed and
whose block is not complete behind it are not seen.  The means are kept in pages of their own
(``CacheNeed.pool_block``), written in the step that brings a block's last position.

With ``own_kv`` False the layer has no key and value tensors: it attends, with its own queries and
its own window, over the cache entry that another layer writes (``RunEntry.write`` False).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, register_part


def yarn_pair_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(float64 frequency of pair i [dims/2], factor on cos and sin).  ``scaling``: None or {factor, original, fast,
    slow}: pairs that turn more than ``fast`` times within ``original`` positions keep their frequency, those that
    turn fewer than ``slow`` times are slowed by ``factor``, a linear ramp over the pair index lies between."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@register_part("position", "rotary_pairs")
class RotaryPairs(Part):
    """Rotation of the pairs (2i, 2i+1) of the first ``dims`` entries of every head by position * f_i.
    params: ``head_dim``, ``dims``, ``base``, ``scaling`` (None or the YaRN block)."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.head_dim, self.dims = int(p["head_dim"]), int(p["dims"])
        if self.dims % 2 or self.dims > self.head_dim:
            raise ValueError(f"rotary width {self.dims} must be even and at most the head size {self.head_dim}")
        f, self.amplitude = yarn_pair_frequencies(self.dims, float(p["base"]), p.get("scaling"))
        self.freq = f.to(torch.float32).to(runtime.device)

    def rotary_table(self):
        return None                      # not the split-halves rotation the fused cache-write kernels apply

    def pair_table(self):
        return self.freq, self.dims, self.amplitude


@register_part("mixer", "window_attention")
class WindowAttention(Part):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``window``, ``keep_first``,
    ``qk_norm_eps``, ``own_kv``, ``sink``, ``q_temp``, ``qk_norm`` ("whole" | "per_head"), ``distance_bias``, ``gate`` (None | "sigmoid"),
    ``pool``.  Nested part ``position`` (none: no encoding).  Tensors: ``q`` [heads*d, hidden], ``o`` [hidden,
    heads*value_dim], ``q.norm`` [heads*d]; with ``own_kv`` ``k`` [kv_heads*d, hidden], ``v`` [kv_heads*value_dim,
    hidden], ``k.norm`` [kv_heads*d]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.d, self.dv = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.d))
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        self.qk_norm_eps = float(p.get("qk_norm_eps") or 0.0)
        self.own_kv = bool(p.get("own_kv", True))
        self.sink = bool(p.get("sink", False))
        temp = p.get("q_temp") or {}
        self.temp_coef, self.temp_every = float(temp.get("coef", 0.0)), int(temp.get("every", 1))
        self.per_head_norm = (p.get("qk_norm") or "whole") == "per_head"
        if (p.get("qk_norm") or "whole") not in ("whole", "per_head"):
            raise ValueError(f"qk_norm={p.get('qk_norm')!r} (known: whole, per_head)")
        self.distance_bias = float(p.get("distance_bias") or 0.0)
        self.gate = p.get("gate") or None
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"gate={self.gate!r} (known: sigmoid)")
        self.pool = int(p.get("pool") or 0) if self.window else 0
        if self.pool and (self.keep_first or not self.own_kv or self.sink):
            raise ValueError("pooled blocks go with neither kept first positions, a sink, nor another layer's keys")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        self.position = build_part("position", spec.parts["position"], runtime) if "position" in spec.parts else None
        self.w_in = self.w_o = self.q_norm = self.k_norm = None

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, G, d, dv = self.heads, self.kv_heads, self.d, self.dv
        out = {"q": TensorSpec((H * d, self.hidden)), "o": TensorSpec((self.hidden, H * dv))}
        if self.own_kv:
            out.update({"k": TensorSpec((G * d, self.hidden)), "v": TensorSpec((G * dv, self.hidden))})
        if self.qk_norm_eps > 0:
            out["q.norm"] = TensorSpec((d if self.per_head_norm else H * d,), "ones_jitter")
            if self.own_kv:
                out["k.norm"] = TensorSpec((d if self.per_head_norm else G * d,), "ones_jitter")
        if self.gate:
            out["g"] = TensorSpec((H * dv, self.hidden))
        return out

    def load(self, t) -> None:
        rows = [t["q"], t["k"], t["v"]] if self.own_kv else [t["q"]]
        self.gate_column = sum(int(r.shape[0]) for r in rows)
        self.w_in = self._to_compute(torch.cat(rows + ([t["g"]] if self.gate else []), dim=0))
        self.w_o = self._to_compute(t["o"])
        if self.qk_norm_eps > 0:
            self.q_norm = self._to_f32(t["q.norm"])
            self.k_norm = self._to_f32(t["k.norm"]) if self.own_kv else None

    def cache_need(self) -> CacheNeed:
        # (a block's mean is made in the step that brings its last position, from keys that must still be held then)
        return CacheNeed(kind="window" if self.window else "full", kv_heads=self.kv_heads, head_dim=self.d,
                         window=max(self.window, self.pool), value_dim=self.dv if self.dv != self.d else 0,
                         keep_first=self.keep_first if self.window else 0, pool_block=self.pool)

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        g = cache.group
        if self.own_kv != bool(cache.write):
            raise ValueError("a layer with keys and values of its own writes its cache entry, one without reads another's")
        proj = ops.linear(x, self.w_in)                   # [T, q (| k | v) (| gate)]
        table = self.position.rotary_table() if self.position is not None and hasattr(self.position, "rotary_table") else (None, 0)
        if table is not None and table[1] and hasattr(self.position, "rotary_table64") and (self.per_head_norm or self.qk_norm_eps <= 0):
            table = self.position.rotary_table64()
        G = self.kv_heads if self.own_kv else 0
        if table is not None and (self.per_head_norm or self.qk_norm_eps <= 0):
            # halves of a head turned against each other (or nothing turned), a norm per head (or none)
            inv_freq, rot = table
            ops.head_norm_rotate_store(proj, self.heads, G, self.d, self.dv, self.q_norm, self.k_norm, self.qk_norm_eps,
                                       ctx.positions, inv_freq, rot, g.slots if self.own_kv else None,
                                       cache.kv if self.own_kv else None, g.page_size)
        elif self.per_head_norm:
            raise ValueError("the per-head norm goes with a rotation of half-split pairs or with none")
        else:
            freq, dims, amplitude = self.position.pair_table() if hasattr(self.position, "pair_table") else (None, 0, 1.0)
            ops.qk_norm_rotate_store(proj, self.heads, G, self.d, self.dv, self.q_norm, self.k_norm,
                                     self.qk_norm_eps, ctx.positions, freq, dims, amplitude,
                                     g.slots if self.own_kv else None, cache.kv if self.own_kv else None, g.page_size)
        extra = {}
        if self.pool:
            sg = cache.summary_group
            if sg is None or cache.summary is None:
                raise ValueError("pooled blocks need the cache entry's pages of block means")
            ops.pool_blocks(cache.kv, g.block_table, ctx.tok_req, ctx.positions, sg.slots, cache.summary, self.kv_heads,
                            self.d, self.dv, g.page_size, self.pool)
            extra.update(pool=self.pool, summary=cache.summary, summary_table=sg.block_table)
        if self.distance_bias:
            extra["distance_bias"] = self.distance_bias
        if self.gate:
            extra["gate_column"] = self.gate_column
        o = ops.window_attention(proj, cache.kv, g.block_table, ctx.tok_req, ctx.positions, self.heads, self.kv_heads, self.d,
                                 self.dv, g.page_size, self.scale, window=self.window, keep_first=self.keep_first,
                                 splits=ctx.attn_splits, hints=ctx, sink=self.sink, temp_coef=self.temp_coef,
                                 temp_every=self.temp_every, **extra)
        return ops.linear(o, self.w_o)

"""Generalized delta rule: a linear-attention mixer whose state decays per key channel and, along
the new key, loses a learned share of what it holds before the new value is written.

With h the mixer's input: r = W_r h, k = W_k h, v = W_v h (heads x head_dim each).  Per head and key
channel the decay is w = exp(-``decay_limit`` * sigmoid(z)), z = W_w2 tanh(W_w1 h) + w0, and the
removal rate a = sigmoid(W_a h + a_b).  With u = k / sqrt(sum k^2 + ``unit_eps``), per head

    S <- diag(w) S - (a * u) (u^T S) + k v^T        o = S^T r

where both products on the right read the old S.  o is divided by its root mean square per head,
multiplied by ``norm`` (one weight per channel of every head) and by sigmoid(W_g h), and projected
by W_o.  S [heads, head_dim, head_dim] is per-request state: float32, zero before position 0.  The
projections run in the compute type (those that feed the decay and the removal rate give float32);
tanh, the second decay product, the sigmoids, exponentials, the unit key, the state and the
read-out are float32.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("mixer", "general_delta_rule")
class GeneralDeltaRule(Part):
    """params: ``hidden``, ``heads``, ``head_dim``, ``norm_eps``; optional ``unit_eps`` (1e-6), ``decay_limit``
    (exp(-1/2): no channel decays faster than exp(-decay_limit) per token) and ``decay_rank`` (the inner size of the
    decay projection when weights are drawn at random; a checkpoint's own size is taken as it is).
    Tensors: ``r``, ``k``, ``v``, ``g``, ``a`` [heads*head_dim, hidden], ``a.b``, ``w0``, ``norm`` [heads*head_dim],
    ``w1`` [rank, hidden], ``w2`` [heads*head_dim, rank], ``o`` [hidden, heads*head_dim]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.d = int(p["hidden"]), int(p["heads"]), int(p["head_dim"])
        self.norm_eps = float(p["norm_eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.decay_limit = float(p.get("decay_limit", math.exp(-0.5)))
        self.rank = int(p.get("decay_rank") or 16)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, W = self.heads * self.d, self.hidden
        mat = TensorSpec((n, W))
        return {"r": mat, "k": mat, "v": mat, "g": mat, "a": mat, "a.b": TensorSpec((n,), "uniform", lo=-2.0, hi=2.0),
                "w1": TensorSpec((-self.rank, W)), "w2": TensorSpec((n, -self.rank)),
                "w0": TensorSpec((n,), "uniform", lo=-4.0, hi=3.0), "norm": TensorSpec((n,), "ones"), "o": TensorSpec((W, n))}

    def load(self, t) -> None:
        if t["w1"].shape[0] != t["w2"].shape[1]:
            raise ValueError(f"the decay projections do not fit: w1 is {list(t['w1'].shape)}, w2 is {list(t['w2'].shape)}")
        self.w_rkvg = self._to_compute(torch.cat([t["r"], t["k"], t["v"], t["g"]], dim=0))
        self.w_a_w1 = self._to_compute(torch.cat([t["a"], t["w1"]], dim=0))      # one product gives the removal's and the decay's inner inputs
        self.w_w2 = self._to_f32(t["w2"])           # the second, small product runs in float32 on the float32 tanh of the first
        self.a_bias, self.w_bias, self.norm_w = self._to_f32(t["a.b"]), self._to_f32(t["w0"]), self._to_f32(t["norm"])
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", states=(("S", (self.heads, self.d, self.d)),))

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        H, d = self.heads, self.d
        n = H * d
        proj = ops.linear(x, self.w_rkvg)                                     # [T, r | k | v | gate]
        aw = ops.linear(x, self.w_a_w1, out_dtype=torch.float32)              # float32 [T, removal's input | decay's inner input]
        z = ops.lowrank_tanh_linear(aw, n, self.w_w2)                         # float32 [T, heads*head_dim], before the bias
        o = ops.general_delta_scan(proj, aw, self.a_bias, z, self.w_bias, self.decay_limit, cache.states["S"], ctx, H, d,
                                   self.unit_eps)
        out = ops.empty((proj.shape[0], n), self.rt.dtype)
        ops.gated_head_norm(o, self.norm_w, self.norm_eps, proj, 3 * n, H, d, out, 0, 1.0, gate_kind="sigmoid", weight_per_head=True)
        return ops.linear(out, self.w_o)

"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

With h the mixer's input: q = W_q h, k = W_k h (heads x head_dim), v = W_v h (heads x value_dim).  The
nested ``position`` part turns the half-split pairs of q and k; k is then multiplied by
head_dim^(-1/2).  Per head, with the head's decay a from the list ``decay``,

    S <- a S + k v^T        o = S^T q

o is divided by its root mean square per head (no weight); the heads are concatenated, multiplied by
silu(W_g h) and projected by W_o.  S [heads, head_dim, value_dim] is per-request state: float32, zero
before position 0.  The projections run in the compute type; angles, the state and the read-out are
float32.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, register_part


@register_part("mixer", "retention")
class Retention(Part):
    """params: ``hidden``, ``heads``, ``head_dim``, ``value_dim``, ``decay`` (one per head), ``norm_eps``.  Nested part
    ``position`` (``rope`` or none).  Tensors: ``q``, ``k`` [heads*head_dim, hidden], ``v``, ``g`` [heads*value_dim,
    hidden], ``o`` [hidden, heads*value_dim]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.d, self.dv = int(p["head_dim"]), int(p["value_dim"])
        self.norm_eps = float(p["norm_eps"])
        decay = [float(a) for a in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.position = build_part("position", spec.parts["position"], runtime) if "position" in spec.parts else None
        self.ones = torch.ones(self.dv, dtype=torch.float32, device=runtime.device)

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, d, dv, W = self.heads, self.d, self.dv, self.hidden
        return {"q": TensorSpec((H * d, W)), "k": TensorSpec((H * d, W)), "v": TensorSpec((H * dv, W)), "g": TensorSpec((H * dv, W)),
                "o": TensorSpec((W, H * dv))}

    def load(self, t) -> None:
        self.w_qkvg = self._to_compute(torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0))
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", states=(("S", (self.heads, self.d, self.dv)),))

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        H, d, dv = self.heads, self.d, self.dv
        proj = ops.linear(x, self.w_qkvg)                                     # [T, q | k | v | gate]
        inv_freq, rot = (None, 0) if self.position is None else \
            self.position.rotary_table64() if hasattr(self.position, "rotary_table64") else self.position.rotary_table()
        if rot:
            # q and k are 2 * heads heads of the same size side by side; nothing is normed or stored
            ops.head_norm_rotate_store(proj, 2 * H, 0, d, dv, None, None, 0.0, ctx.positions, inv_freq, rot, None, None, 1)
        o = ops.gla_scan(proj, None, None, 1.0, cache.states["S"], ctx, H, d, dv, 1.0, head_decay=self.decay, k_scale=d ** -0.5)
        out = ops.empty((proj.shape[0], H * dv), self.rt.dtype)
        ops.gated_head_norm(o, self.ones, self.norm_eps, proj, 2 * H * d + H * dv, H, dv, out, 0, 1.0)
        return ops.linear(out, self.w_o)

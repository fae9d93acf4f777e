"""Attention whose queries, keys and values pass small latents; only the key/value latent and one
rotated key part shared by all heads are kept per position.

With h the mixer's input: c_q = rmsnorm(W_dq h) * dq.norm, q = W_uq c_q, laid out head by head as
[``head_dim`` plain | ``rot_dim`` rotated].  W_dkv h gives ``kv_rank`` + ``rot_dim`` entries: the first
``kv_rank``, RMS-normed with dkv.norm, are the latent c; the rest, rotated by the position (the nested
``position`` part turns neighbouring pairs), is the one rotated key part k_r.  Head n has the plain
key W_uk[n] c and the value W_uv[n] c.  score = (q_plain . W_uk[n] c + q_rot . k_r) * scale, causal
softmax, head n's output times sigmoid(W_g h)_n, W_o on the concatenated heads.

The cache keeps [c | k_r] per position as the key of one key head and no values.  Attention runs on
the latent: q_plain is carried through W_uk[n]^T once per query (q_c = W_uk[n]^T q_plain, so that
q_plain . W_uk[n] c = q_c . c), the kernel scores [q_c | q_rot] against [c | k_r] and sums the
weighted latents (the value of a key is its first ``kv_rank`` entries), and W_uv[n] is applied to
that sum.  Nothing per head is ever made for a cached position.

With ``own_kv`` False the layer has no W_dkv: it attends, with its own queries and its own W_uk and
W_uv, over the cache entry that another layer writes (``RunEntry.write`` False).
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: ``hidden``, ``heads``, ``head_dim``, ``rot_dim``, ``value_dim``, ``kv_rank``, ``q_rank``, ``scale``,
    ``norm_eps``, ``own_kv``.  Nested part ``position`` (kind ``rotary_pairs`` over ``rot_dim`` entries).
    Tensors: ``dq`` [q_rank, hidden], ``dq.norm`` [q_rank], ``uq`` [heads*(head_dim+rot_dim), q_rank], ``uk`` [heads*head_dim,
    kv_rank], ``uv`` [heads*value_dim, kv_rank], ``g`` [heads, hidden], ``o`` [hidden, heads*value_dim]; with ``own_kv``
    ``dkv`` [kv_rank+rot_dim, hidden], ``dkv.norm`` [kv_rank]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.d, self.n, self.dv = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["norm_eps"])
        self.own_kv = bool(p.get("own_kv", True))
        self.position = build_part("position", spec.parts["position"], runtime)
        # in bfloat16 the operator works prompt portions as matrix products laid out by the step's own lengths
        self.portions_by_host_lengths = runtime.dtype == torch.bfloat16

    def children(self):
        return {"position": self.position}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, d, n, e, R, Q, W = self.heads, self.d, self.n, self.dv, self.kv_rank, self.q_rank, self.hidden
        out = {"dq": TensorSpec((Q, W)), "dq.norm": TensorSpec((Q,), "ones_jitter"), "uq": TensorSpec((H * (d + n), Q)),
               "uk": TensorSpec((H * d, R)), "uv": TensorSpec((H * e, R)), "g": TensorSpec((H, W)), "o": TensorSpec((W, H * e))}
        if self.own_kv:
            out.update({"dkv": TensorSpec((R + n, W)), "dkv.norm": TensorSpec((R,), "ones_jitter")})
        return out

    def load(self, t) -> None:
        H, d, e, R = self.heads, self.d, self.dv, self.kv_rank
        rows = [t["dq"]] + ([t["dkv"]] if self.own_kv else []) + [t["g"]]
        self.w_in = self._to_compute(torch.cat(rows, dim=0))                  # [q latent (| kv latent | rotated key part) | gates]
        self.q_norm = self._to_f32(t["dq.norm"])
        self.kv_norm = self._to_f32(t["dkv.norm"]) if self.own_kv else None
        self.w_uq = self._to_compute(t["uq"])
        self.w_uk_t = self._to_compute(t["uk"].reshape(H, d, R).transpose(1, 2))      # [H, R, d]: q_c = W_uk[n]^T q_plain
        self.w_uv = self._to_compute(t["uv"].reshape(H, e, R))                        # [H, e, R]
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="full", kv_heads=1, head_dim=self.kv_rank + self.n, value_dim=self.kv_rank, shared_values=True)

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        g = cache.group
        if self.own_kv != bool(cache.write):
            raise ValueError("a layer with a latent of its own writes its cache entry, one without reads another's")
        H, d, n, e, R, Q = self.heads, self.d, self.n, self.dv, self.kv_rank, self.q_rank
        T = x.shape[0]
        proj = ops.linear(x, self.w_in)
        freq, dims, _ = self.position.pair_table()
        # the two latents are normed, the rotated key part is turned, and [c | k_r] goes to the token's slot of the cache
        cq = ops.latent_norm_store(proj, Q, self.q_norm, R if self.own_kv else 0, self.kv_norm, n if self.own_kv else 0,
                                   self.eps, ctx.positions, freq, dims, g.slots if self.own_kv else None,
                                   cache.kv if self.own_kv else None, g.page_size)
        q = ops.linear(cq, self.w_uq)                                         # [T, H, plain | rotated]
        ql = ops.empty((T, H * (R + n)), self.rt.dtype)                        # [T, H, q_c | rotated]
        ops.head_linear(q, d + n, 0, self.w_uk_t, ql, R + n, 0, H)             # q_c = W_uk[n]^T q_plain
        ops.rotate_head_part(q, d + n, d, ql, R + n, R, H, n, ctx.positions, freq, dims)
        o = ops.latent_attention(ql, cache.kv, g.block_table, ctx, H, R, n, g.page_size, self.scale)   # [T, H, R]: weighted latents
        out = ops.empty((T, H * e), self.rt.dtype)
        ops.head_linear(o, R, 0, self.w_uv, out, e, 0, H, gate=proj, gate_column=proj.shape[1] - H)    # W_uv[n], times sigmoid(gate n)
        return ops.linear(out, self.w_o)

"""A block with a norm before and a norm after each sub-layer, whose result joins a weighted sum over
depth.

With x the stream a layer receives:

    u = x + norm1b(mixer(norm1(x)))          X = u + norm2b(ffn(norm2(u)))

X is the layer's result.  What goes on to the next layer (and, after the last one, to the model's final
norm) is  sum_j c[j] * X_j  over the embedding output X_0 and the results X_1 .. of all layers up to this
one, with the layer's own coefficients ``depth`` [index + 2].  The results of a step are kept in one
float32 buffer [layers + 1, T, width] that the first block makes and hands on through the step's
context.

The norm after a sub-layer, the residual sum, the sum over depth and the norm before the next sub-layer
are one operator (``ops.post_norm_add``).  A mixer that is the mean of its members' normed outputs
(``ParallelMixers`` with ``combine`` "normed_mean") hands over the members' outputs and that mean is
taken in the same operator.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, build_part, register_part


class _Normed:
    """The next block's first norm, already applied (what ``RMSNorm.forward`` passes through untouched)."""

    def __init__(self, y: torch.Tensor, weight: torch.Tensor):
        self.y, self.weight = y, weight

    def materialise(self) -> torch.Tensor:
        return self.y


@register_part("block", "sandwich_depth_average")
class SandwichDepthAverageBlock(Part):
    """params: ``index`` (the layer's number from 0), ``layers`` (how many the model has), ``width``.  Nested parts:
    ``norm1``, ``mixer``, ``norm1b``; ``norm2``, ``ffn``, ``norm2b`` (all three or none).  Tensor: ``depth``
    [index + 2]."""

    KEY = "depth_results"

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.index, self.layers, self.width = int(p["index"]), int(p["layers"]), int(p["width"])
        self.norm1 = build_part("norm", spec.parts["norm1"], runtime)
        self.mixer = build_part("mixer", spec.parts["mixer"], runtime)
        self.norm1b = build_part("norm", spec.parts["norm1b"], runtime)
        have = [k in spec.parts for k in ("norm2", "ffn", "norm2b")]
        if any(have) != all(have):
            raise ValueError("a block has norm2, ffn and norm2b, or none of them")
        self.norm2 = build_part("norm", spec.parts["norm2"], runtime) if have[0] else None
        self.ffn = build_part("ffn", spec.parts["ffn"], runtime) if have[0] else None
        self.norm2b = build_part("norm", spec.parts["norm2b"], runtime) if have[0] else None
        self.depth = None

    takes_next_norm = True

    def children(self):
        parts = {"norm1": self.norm1, "mixer": self.mixer, "norm1b": self.norm1b, "norm2": self.norm2, "ffn": self.ffn,
                 "norm2b": self.norm2b}
        return {k: v for k, v in parts.items() if v is not None}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        # drawn at random: about an even share of every result, so that each of them matters
        n = self.index + 2
        return {"depth": TensorSpec((n,), "uniform", lo=0.5 / n, hi=1.5 / n)}

    def load(self, tensors) -> None:
        self.depth = self._to_f32(tensors["depth"])

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, residual, ctx, cache, next_norm=None):
        ops = self.rt.ops
        first = residual is None
        y, residual = self.norm1.forward(x, residual)
        if hasattr(y, "materialise"):
            y = y.materialise()
        if first:
            results = ops.empty((self.layers + 1, residual.shape[0], self.width), torch.float32)
            results[0].copy_(residual)
            ctx.scratch[self.KEY] = results
        results = ctx.scratch[self.KEY]
        if getattr(self.mixer, "normed", False):
            members = self.mixer.member_outputs(y, ctx, cache)
            outs, weights = [o for o, _ in members], [w for _, w in members]
        else:
            outs, weights = [self.mixer.forward(y, ctx, cache)], None
        eps = self.norm1b.eps
        following = next_norm.weight if next_norm is not None and getattr(next_norm, "deferrable", False) else None
        depth = dict(results=results, index=self.index + 1, coeffs=self.depth, next_weight=following)
        if self.ffn is None:
            y, residual = ops.post_norm_add(outs, weights, self.norm1b.weight, eps, residual, dtype=self.rt.dtype, **depth)
        else:
            y, residual = ops.post_norm_add(outs, weights, self.norm1b.weight, eps, residual, dtype=self.rt.dtype,
                                            next_weight=self.norm2.weight)
            y, residual = ops.post_norm_add([self.ffn.forward(y)], None, self.norm2b.weight, eps, residual, dtype=self.rt.dtype,
                                            **depth)
        return (_Normed(y, following) if following is not None else None), residual

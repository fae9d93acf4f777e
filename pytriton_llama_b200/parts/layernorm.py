"""Layer norm with weight and bias, the residual add fused in.

The sub-layer's output is added to the float32 residual first and the sum becomes the new
residual; then y = (s - mean(s)) / sqrt(var(s) + eps) * weight + bias, var being the mean of the
squared deviations from the mean.  Sum, mean, variance and y are float32 in every compute type;
y is rounded once.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """params: ``width``, ``eps``; optional ``init`` (how random-weights mode draws the weight).
    Tensors: ``weight`` [width], ``bias`` [width]."""

    deferrable = False      # no product's epilogue prepares this norm's input

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.width,), init=self.spec.params.get("init", "ones")),
                "bias": TensorSpec((self.width,), init="zeros_jitter")}

    def load(self, tensors) -> None:
        self.weight, self.bias = self._to_f32(tensors["weight"]), self._to_f32(tensors["bias"])

    def forward(self, x, residual, rows=None, bias=None):
        """``bias`` (float32 [width]) is added together with ``x``: the bias of the projection that
        made ``x``, where that projection left it out."""
        if hasattr(x, "materialise"):       # a prepared input of another norm: its sum is in the residual already
            x = None
        return self.rt.ops.add_layernorm(x, residual, self.weight, self.bias, self.eps, rows=rows, dtype=self.rt.dtype, add_bias=bias)

    def start_stream(self, x) -> torch.Tensor:
        """The normed ``x`` as a new float32 residual stream (the norm an embedding passes)."""
        y, _ = self.rt.ops.add_layernorm(x, None, self.weight, self.bias, self.eps, dtype=torch.float32, keep_sum=False)
        return y

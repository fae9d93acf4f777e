"""Dense feed-forwards with one hidden layer, W_down act(W_up h), the activation worked out in float32.

``gelu_mlp``: the tanh form of gelu, gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
``xielu_mlp``: xIELU with two learned numbers (p, q) per layer: for z > 0, softplus(p) z^2 + z / 2; for z <= 0,
(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
from __future__ import annotations

import math
from typing import Dict

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("ffn", "gelu_mlp")
class GeluMLP(Part):
    """params: ``hidden``, ``inter``.  Tensors: ``up`` [inter, hidden], ``down`` [hidden, inter]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.hidden, self.inter = int(spec.params["hidden"]), int(spec.params["inter"])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"up": TensorSpec((self.inter, self.hidden)), "down": TensorSpec((self.hidden, self.inter))}

    def load(self, t) -> None:
        self.w_up, self.w_down = self._to_compute(t["up"]), self._to_compute(t["down"])

    def forward(self, x):
        ops = self.rt.ops
        return ops.linear(ops.gelu_tanh(ops.linear(x, self.w_up)), self.w_down)


@register_part("ffn", "xielu_mlp")
class XieluMLP(GeluMLP):
    """params: ``hidden``, ``inter``.  Tensors: ``up`` [inter, hidden], ``down`` [hidden, inter], ``act`` [2] = (p, q)."""

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {**super().tensor_specs(), "act": TensorSpec((2,), "uniform", lo=-1.0, hi=1.0)}

    def load(self, t) -> None:
        super().load(t)
        softplus = lambda v: max(v, 0.0) + math.log1p(math.exp(-abs(v)))
        p, q = (float(v) for v in t["act"].to("cpu", dtype=__import__("torch").float64))
        self.pos_factor, self.neg_factor = softplus(p), 0.5 + softplus(q)     # worked out once, in float64

    def forward(self, x):
        ops = self.rt.ops
        return ops.linear(ops.xielu(ops.linear(x, self.w_up), self.pos_factor, self.neg_factor), self.w_down)

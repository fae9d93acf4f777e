"""Mixture of gated experts with a router, and optionally an expert that every token uses.

Router: z = W_router h in float32, score = sigmoid(z); each token takes the ``top`` experts with the
largest scores, weighted by those scores as they are (not renormalised).  An expert is
W_down (silu(W_gate u) * (W_up u)); with ``scale_input`` its input is u = weight * h and the outputs
are summed, otherwise u = h and the outputs are summed with the weights.  The shared expert (same
form, its own inner size) sees h itself and is added.

Options of the router.  ``score`` "softmax": score = softmax(z) over all experts.  ``groups`` > 1: the experts form
that many groups of neighbours, a group's score is its largest score, and only experts of the ``keep_groups`` groups
with the largest scores can be chosen.  ``renormalise``: the weights are the chosen scores divided by their sum
(+ 1e-20).

The experts' weights are kept as stacks [experts, ...]; the tokens of a step are sorted by expert on
the device (no count ever comes back to the host, so a step can be captured in a CUDA graph) and one
grouped product per projection walks tiles of tokens of one expert each.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("ffn", "routed_experts")
class RoutedExperts(Part):
    """params: ``hidden``, ``inter``, ``experts``, ``top``, ``shared_inter`` (0: none), ``scale_input``, ``score`` ("sigmoid" |
    "softmax"), ``groups``, ``keep_groups``, ``renormalise``.
    Tensors: ``router`` [experts, hidden]; per expert i ``e<i>.gate``, ``e<i>.up`` [inter, hidden], ``e<i>.down``
    [hidden, inter]; ``shared.gate``, ``shared.up`` [shared_inter, hidden], ``shared.down`` [hidden, shared_inter]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.inter, self.experts, self.top = int(p["hidden"]), int(p["inter"]), int(p["experts"]), int(p["top"])
        self.shared_inter = int(p.get("shared_inter") or 0)
        self.scale_input = bool(p.get("scale_input", True))
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top={self.top} of {self.experts} experts")
        self.score = p.get("score") or "sigmoid"
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"score={self.score!r} (known: sigmoid, softmax)")
        self.groups = int(p.get("groups") or 1)
        self.keep_groups = int(p.get("keep_groups") or self.groups)
        self.renormalise = bool(p.get("renormalise", False))
        if self.experts % self.groups or not 1 <= self.keep_groups <= self.groups:
            raise ValueError(f"{self.experts} experts in {self.groups} groups of which {self.keep_groups} are kept")
        if self.top > self.keep_groups * (self.experts // self.groups):
            raise ValueError(f"top={self.top} exceeds the experts of {self.keep_groups} groups")
        self.routing = {}
        if self.score != "sigmoid" or self.groups > 1 or self.renormalise:
            self.routing = dict(score=self.score, groups=self.groups, keep_groups=self.keep_groups, renormalise=self.renormalise)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out = {"router": TensorSpec((self.experts, self.hidden))}
        for i in range(self.experts):
            out.update({f"e{i}.gate": TensorSpec((self.inter, self.hidden)), f"e{i}.up": TensorSpec((self.inter, self.hidden)),
                        f"e{i}.down": TensorSpec((self.hidden, self.inter))})
        if self.shared_inter:
            out.update({"shared.gate": TensorSpec((self.shared_inter, self.hidden)), "shared.up": TensorSpec((self.shared_inter, self.hidden)),
                        "shared.down": TensorSpec((self.hidden, self.shared_inter))})
        return out

    def load(self, t) -> None:
        E = range(self.experts)
        self.w_router = self._to_compute(t["router"])
        # per expert the gate rows, then the up rows: one grouped product feeds the activation
        self.w_gate_up = self._to_compute(torch.stack([torch.cat([t[f"e{i}.gate"], t[f"e{i}.up"]], dim=0) for i in E]))
        self.w_down = self._to_compute(torch.stack([t[f"e{i}.down"] for i in E]))
        if self.shared_inter:
            # the shared expert is a dense gated feed-forward: where the operator set's product applies silu(gate) * up
            # in its epilogue, gate and up rows alternate (as in parts/swiglu.py)
            ops = self.rt.ops
            self.alternating = bool(ops is not None and hasattr(ops, "fused_ffn_layout")
                                    and ops.fused_ffn_layout(self.rt.dtype, self.hidden, self.shared_inter))
            if self.alternating:
                gu = torch.stack([t["shared.gate"], t["shared.up"]], dim=1).reshape(2 * self.shared_inter, self.hidden)
            else:
                gu = torch.cat([t["shared.gate"], t["shared.up"]], dim=0)
            self.w_shared_gate_up = self._to_compute(gu)
            self.w_shared_down = self._to_compute(t["shared.down"])

    def forward(self, x):
        ops = self.rt.ops
        shared = None
        if self.shared_inter:
            inner = ops.gate_up_silu(x, self.w_shared_gate_up) if self.alternating else ops.silu_mul(ops.linear(x, self.w_shared_gate_up))
            shared = ops.linear(inner, self.w_shared_down)
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        return ops.routed_experts(x, logits, self.w_gate_up, self.w_down, self.top, self.scale_input, shared, **self.routing)

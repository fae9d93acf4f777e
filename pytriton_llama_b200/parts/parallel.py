"""Several mixers side by side on the same input, added with fixed scales:
y = sum_m scale_m * mixer_m(h); or (``combine`` "normed_mean") each output first divided by its root mean
square over the model width and multiplied by a weight of its own, y = (1 / M) sum_m rmsnorm_m(mixer_m(h)).

Each member writes the input of its output projection, already multiplied by its scale, into its
columns of one buffer, and one product with the members' output weights side by side gives the sum
(the members' output biases, scaled, are added by the caller: ``output_bias``).  At most one member
may keep keys and values in pages; the per-request states of all members are kept under
"<member>.<name>".

On a CUDA device the members run side by side in time as well: the first on the launching stream,
every other one on a stream of its own that starts after the input is ready and is joined before
the output product (a member that walks its tokens in order fills few SMs for long; the others'
kernels take the rest).  A step that is captured in a CUDA graph keeps the fork as branches of the
graph.  ``PTL_PARALLEL_STREAMS=0`` runs the members one after another.
"""
from __future__ import annotations

import os
from dataclasses import replace

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixers(Part):
    """params: ``hidden``, ``scales`` {member: factor}.  Nested parts: the members, by name; each has
    ``inner_width``, ``write_inner``, ``w_o`` and ``output_bias``.  With ``combine`` "normed_mean" (and ``norm_eps``)
    the members only need ``forward``; tensors ``<member>.out`` [hidden]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.members = {name: build_part("mixer", s, runtime) for name, s in spec.parts.items()}
        self.combine = spec.params.get("combine") or "joint_projection"
        if self.combine not in ("joint_projection", "normed_mean"):
            raise ValueError(f"combine={self.combine!r} (known: joint_projection, normed_mean)")
        self.normed = self.combine == "normed_mean"
        self.out_weights = {}
        self.columns, at = {}, 0
        if self.normed:
            self.hidden, self.norm_eps = int(spec.params["hidden"]), float(spec.params["norm_eps"])
            self.scales = {name: 1.0 / len(self.members) for name in self.members}
        else:
            self.scales = {name: float(spec.params["scales"][name]) for name in self.members}
            for name, m in self.members.items():
                self.columns[name] = at
                at += m.inner_width
        self.inner_width = at
        self.output_bias_spec = any(getattr(m, "output_bias_spec", False) for m in self.members.values())
        self.w_o = self.output_bias = None
        self._streams = None

    def children(self):
        return dict(self.members)

    def tensor_specs(self):
        if not self.normed:
            return {}
        return {f"{name}.out": TensorSpec((self.hidden,), "ones_jitter") for name in self.members}

    def load(self, tensors) -> None:
        for name in self.members:
            self.out_weights[name] = self._to_f32(tensors[f"{name}.out"])

    def after_load(self) -> None:
        if self.normed:
            return
        self.w_o = torch.cat([m.w_o for m in self.members.values()], dim=1).contiguous()
        for m in self.members.values():
            m.w_o = None            # the joint weight is the one that is used
        biases = [m.output_bias * self.scales[name] for name, m in self.members.items() if m.output_bias is not None]
        self.output_bias = sum(biases[1:], biases[0]).contiguous() if biases else None

    def cache_need(self) -> CacheNeed:
        needs = {name: m.cache_need() for name, m in self.members.items()}
        paged = [n for n in needs.values() if n.kind != "none"]
        if len(paged) > 1:
            raise ValueError("only one member of a parallel mixer may keep pages of keys and values")
        states = tuple((f"{name}.{s}", shape) for name, n in needs.items() for s, shape in n.states)
        if any(n.state_shape is not None for n in needs.values()):
            raise ValueError("members of a parallel mixer name their states")
        base = paged[0] if paged else CacheNeed()
        return replace(base, states=states)

    def member_outputs(self, x, ctx, cache):
        """``combine`` "normed_mean": [(output [T, hidden], its norm weight)] of the members, side by side in time."""
        names = list(self.members)
        outs = {}
        side_by_side = (self.rt.device.type == "cuda" and len(names) > 1 and isinstance(x, torch.Tensor)
                        and os.environ.get("PTL_PARALLEL_STREAMS", "1") != "0")
        if not side_by_side:
            for name in names:
                outs[name] = self.members[name].forward(x, ctx, cache.member(name))
        else:
            if self._streams is None:
                self._streams = [torch.cuda.Stream(self.rt.device) for _ in names[1:]]
            main = torch.cuda.current_stream(self.rt.device)
            ready = torch.cuda.Event()
            ready.record(main)
            for name, stream in zip(names[1:], self._streams):
                stream.wait_event(ready)
                with torch.cuda.stream(stream):
                    outs[name] = self.members[name].forward(x, ctx, cache.member(name))
            outs[names[0]] = self.members[names[0]].forward(x, ctx, cache.member(names[0]))
            for stream in self._streams:
                main.wait_stream(stream)
        return [(outs[name], self.out_weights[name]) for name in names]

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        if self.normed:
            return ops.mean_of_normed(self.member_outputs(x, ctx, cache), self.norm_eps, self.rt.dtype)
        joint = ops.empty((x.shape[0], self.inner_width), self.rt.dtype)
        names = list(self.members)
        side_by_side = (self.rt.device.type == "cuda" and len(names) > 1 and isinstance(x, torch.Tensor)
                        and os.environ.get("PTL_PARALLEL_STREAMS", "1") != "0")
        if not side_by_side:
            for name in names:
                self.members[name].write_inner(x, ctx, cache.member(name), joint, self.columns[name], self.scales[name])
            return ops.linear(joint, self.w_o)
        if self._streams is None:
            self._streams = [torch.cuda.Stream(self.rt.device) for _ in names[1:]]
        main = torch.cuda.current_stream(self.rt.device)
        ready = torch.cuda.Event()
        ready.record(main)
        for name, stream in zip(names[1:], self._streams):
            stream.wait_event(ready)
            with torch.cuda.stream(stream):
                self.members[name].write_inner(x, ctx, cache.member(name), joint, self.columns[name], self.scales[name])
        self.members[names[0]].write_inner(x, ctx, cache.member(names[0]), joint, self.columns[names[0]], self.scales[names[0]])
        for stream in self._streams:
            main.wait_stream(stream)
        return ops.linear(joint, self.w_o)

"""Interfaces and registry of the parts a decoder layer is put together from.

A part is one of six categories: ``mixer`` (attention, a selective scan, a delta rule, or several
side by side), ``ffn``, ``norm``, ``position``, ``token_input`` (a term that depends on the
token itself, added to the stream inside a layer) and ``block`` (how the others are arranged
around the residual stream).  A part is described
by a ``PartSpec`` (kind + its sizes and constants + where its tensors are in the checkpoint) and
built by ``build_part``; it never sees the model's configuration and does not know which model
it is in.  New kinds are added with ``register_part`` from anywhere, tests included.

Contracts (``T`` = tokens of the step, all tensors on the runtime's device):

* every part: ``tensor_specs() -> {local name: TensorSpec}``, ``load(tensors)`` with the same
  local names (tensors in the checkpoint's stored element type, on the CPU);
* norm: ``forward(x, residual, rows=None) -> (y, residual)`` -- adds ``x`` ([T, H], or None when
  the sub-layer before already added its output) into the float32 ``residual`` (None at the first
  layer), returns the normed sum in the compute type;
* position: ``rotary_table() -> (inv_freq float32 [rot/2], rot)`` when it is a rotation of the
  (j, j + rot/2) pairs of every head by position * inv_freq[j], which the kernels apply while they
  write the cache; ``(None, 0)`` for no encoding at all; ``None`` for anything else, and then the
  mixer calls ``apply(qk, positions, heads, head_dim)`` on the projected q and k before they are
  stored (in place; ``qk`` is the [T, heads*head_dim] view of the projection's q and k columns,
  whose rows are not contiguous);
* mixer: ``cache_need() -> CacheNeed``; ``forward(x, ctx, cache) -> [T, H]`` where ``ctx`` is the
  step's ``StepContext`` and ``cache`` the ``LayerCacheView`` of the cache entry this run of the
  layer uses (``cache.write`` tells whether this run stores its keys and values);
* ffn: ``forward(x) -> [T, H]``;
* a mixer or ffn may leave the bias of its last projection un-added and name it in
  ``output_bias`` (float32 [H] or None): whoever adds the output into the stream adds it too;
* token_input: ``apply(residual, x, bias, ctx)`` adds ``x`` (+ ``bias``), then its own term, into
  the float32 ``residual`` in place;
* a mixer or ffn with the class attribute ``fuses_residual = True`` is called with
  ``residual=<float32 [T, H]>`` as well and may add its output into it and return None;
* block: ``forward(x, residual, ctx, cache) -> (x, residual)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

import torch

CATEGORIES = ("mixer", "ffn", "norm", "position", "token_input", "block")


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]    # a negative entry -n: any size in the checkpoint, n when the tensor is drawn at random
    init: str = "normal"      # "normal": N(0, std) | "ones" | "ones_jitter": 1 + N(0, 0.01) | "zeros" | "uniform": U(lo, hi)
    optional: bool = False    # may be absent from the checkpoint (the part then gets None)
    lo: float = 0.0           # bounds of "uniform"
    hi: float = 1.0


@dataclass
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)   # local name -> checkpoint name
    parts: Dict[str, "PartSpec"] = field(default_factory=dict)  # nested parts (a mixer's position encoding)


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer keeps between steps.

    ``kind``: "full" (every key and value), "window" (only the last ``window`` positions), "chunk"
    (only the keys of the block of ``window`` positions, counted from position 0, that the next
    query lies in) or "none".  ``value_dim``: size of a value head where it differs from
    ``head_dim`` (0: the same).  ``state_shape``/``state_dtype``: per-request state of fixed size
    (None if none).  ``states``: further per-request states by name, float32, as (name, shape)
    pairs; a mixer made of several lists those of all its members.  ``keep_first`` (kind "window"):
    the keys of positions below it stay visible, and held, whatever the window has passed.
    ``shared_values``: a key's first ``value_dim`` entries are its value; no values are stored.
    ``pool_block`` = P > 0: beside its pages of keys and values the entry keeps, in pages of their own, one mean key
    and one mean value for every complete block of P positions of a request (never given back before the request ends)."""
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: Optional[Tuple[int, ...]] = None
    state_dtype: Optional[torch.dtype] = None
    value_dim: int = 0
    states: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()
    keep_first: int = 0
    shared_values: bool = False
    pool_block: int = 0

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim

    @property
    def stored_v_dim(self) -> int:
        """Entries a page holds per value (0 where values are read out of the keys)."""
        return 0 if self.shared_values else self.v_dim

    def group_key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window, self.state_shape, self.state_dtype,
                self.value_dim, self.states, self.keep_first, self.shared_values, self.pool_block)

    def merged(self, other: "CacheNeed") -> "CacheNeed":
        """The need of a cache entry that ``self`` and ``other`` both read: everything either of them
        still sees is kept.  Raises where they differ in more than the window and the kept positions."""
        from dataclasses import replace
        if self.kind not in ("full", "window") or other.kind not in ("full", "window"):
            if self.group_key() == other.group_key():
                return self
            raise ValueError("cache needs of this kind cannot be merged")
        if replace(self, kind="full", window=0, keep_first=0).group_key() != replace(other, kind="full", window=0, keep_first=0).group_key():
            raise ValueError("layers that share a cache entry differ in head counts, head sizes or states")
        if self.kind == "full" or other.kind == "full":
            return replace(self, kind="full", window=0, keep_first=0)
        return replace(self, window=max(self.window, other.window), keep_first=max(self.keep_first, other.keep_first))


@dataclass
class Runtime:
    """Where and how parts compute: device, compute element type and the operator set."""
    device: torch.device
    dtype: torch.dtype
    ops: Any
    shared: Dict[str, torch.Tensor] = field(default_factory=dict)   # tensors of the model that parts of every layer read


_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str):
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; known: {CATEGORIES}")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        return cls
    return deco


def part_kinds(category: str):
    return sorted(_REGISTRY[category])


def build_part(category: str, spec: PartSpec, runtime: Runtime):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise KeyError(f"no {category} part of kind {spec.kind!r}; registered: {part_kinds(category)}") from None
    return cls(spec, runtime)


class Part:
    """Base of all parts: keeps the spec and the runtime, has no tensors by default."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, Optional[torch.Tensor]]) -> None:
        pass

    def children(self) -> Dict[str, "Part"]:
        """Nested parts by the name they have in ``spec.parts``."""
        return {}

    # helpers for subclasses
    def _to_compute(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.rt.device, dtype=self.rt.dtype).contiguous()

    def _to_f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.rt.device, dtype=torch.float32).contiguous()

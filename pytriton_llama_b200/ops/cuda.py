"""Tensor-level wrappers of the hand-written sm_100a kernels.

``CudaOps`` is the only implementation of the operator set that the engine's parts call.  It
loads the library built from ``csrc/`` through ctypes and launches on torch's current CUDA stream;
torch itself is used for allocation and, in bfloat16, for the plain library matrix products
(cuBLAS) where lite_llama uses nn.Linear / F.linear too (lite_llama/models/llama.py:22-24,37-40).
There is no CPU path: a tensor that is not on a CUDA device, or a library that cannot be built
or loaded, raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import build
from .worklists import PAD_TOKEN_ROW, StepWork, WorkList

_c_int = ctypes.c_int
_c_ll = ctypes.c_longlong
_c_f = ctypes.c_float
_ptr = ctypes.c_void_p

_SIGNATURES = {
    "ptl_embed_gather": [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr],
    "ptl_add_rmsnorm": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr],
    "ptl_silu_mul": [_ptr, _ptr, _c_int, _c_int, _ptr],
    "ptl_rope_kv_write": [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _ptr],
    "ptl_add_bias_rmsnorm": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr],
    "ptl_embed_scaled": [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_f, _ptr, _ptr],
    "ptl_clamped_glu": [_ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _c_f, _c_f, _ptr],
    "ptl_token_side": [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr],
    "ptl_causal_conv": [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int,
                        _c_int, _c_int, _ptr],
    "ptl_selective_scan": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr,
                           _c_int, _ptr],
    "ptl_gated_delta_rule": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f,
                             _c_f, _ptr],
    "ptl_gated_head_norm": [_ptr, _c_int, _c_int, _ptr, _ptr, _c_f, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int,
                            _ptr],
    "ptl_kv_write_normed": [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_f, _ptr],
    "ptl_chunk_attention": [_ptr, _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_int, _c_f, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr],
    "ptl_stream_mix_norm": [_ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_f, _ptr],
    "ptl_gelu_tanh": [_ptr, _ptr, _c_ll, _ptr],
    "ptl_qk_norm_rotate_store": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _c_f, _ptr, _ptr, _c_int, _c_f, _ptr,
                                 _ptr, _c_int, _c_ll, _ptr],
    "ptl_window_attention": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                             _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _c_f, _c_int, _c_f, _c_int,
                             _c_int, _ptr, _ptr, _c_int, _c_int, _ptr],
    "ptl_head_norm_rotate_store": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _c_f, _ptr, _ptr, _c_int, _c_int,
                                   _ptr, _ptr, _c_int, _c_ll, _ptr],
    "ptl_pool_blocks": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _ptr],
    "ptl_post_norm_add": [_ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _c_f, _ptr, _ptr, _c_ll, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int,
                          _c_int, _ptr],
    "ptl_add_layernorm": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _c_int, _ptr],
    "ptl_xielu": [_ptr, _ptr, _c_ll, _c_f, _c_f, _ptr],
    "ptl_general_delta_scan": [_ptr, _ptr, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _c_f, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int,
                               _c_int, _c_f, _ptr],
    "ptl_latent_norm_store": [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr, _c_int, _c_f, _ptr, _ptr, _c_int, _ptr, _ptr,
                              _c_ll, _ptr],
    "ptl_rotate_head_part": [_ptr, _c_int, _c_int, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr],
    "ptl_head_gate": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr],
    "ptl_latent_gather": [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr],
    "ptl_causal_softmax_rows": [_ptr, _c_int, _ptr, _c_ll, _c_int, _ptr, _c_int, _c_f, _c_int, _ptr],
    "ptl_head_linear": [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr],
    "ptl_gla_scan": [_ptr, _ptr, _c_int, _ptr, _ptr, _c_f, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_f, _ptr, _c_f,
                     _ptr],
    "ptl_moe_gather": [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr],
    "ptl_moe_grouped": [_ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr],
    "ptl_moe_combine": [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr],
    "ptl_paged_attention_simt": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr],
}
_GEMM_SIG = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr]


class NormedActivation:
    """The input of an RMS norm whose normalisation is still to be done by the product that reads it:
    ``xs`` = bfloat16(residual * weight) [tokens, width] and, per token, ``slots`` partial sums of
    residual^2 in ``sumsq``.  The row scale rsqrt(sum / width + eps) is applied by the consumer."""
    __slots__ = ("xs", "sumsq", "slots", "eps", "weight", "ops")

    def __init__(self, xs, sumsq, slots, eps, weight, ops=None):
        self.xs, self.sumsq, self.slots, self.eps, self.weight, self.ops = xs, sumsq, slots, eps, weight, ops

    @property
    def shape(self):
        return self.xs.shape

    @property
    def dtype(self):
        return self.xs.dtype

    def materialise(self) -> torch.Tensor:
        """The normed activation as a plain tensor (for consumers that cannot apply the scale)."""
        return self.ops.finish_norm(self)


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_LIB = None


def load_library() -> ctypes.CDLL:
    """The kernel library, built on first use.  Raises if it cannot be built or loaded."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = build.library_path()
    lib = ctypes.CDLL(str(path))
    for base, sig in _SIGNATURES.items():
        for suffix in ("_f32", "_bf16"):
            fn = getattr(lib, base + suffix)
            fn.argtypes = sig
            fn.restype = _c_int
    for name in ("ptl_gemm_simt_f32", "ptl_gemm_simt_bf16", "ptl_gemm_simt_bf16_f32out"):
        fn = getattr(lib, name)
        fn.argtypes = _GEMM_SIG
        fn.restype = _c_int
    lib.ptl_decode_attention_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int,
                                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr, _ptr]
    lib.ptl_decode_attention_bf16.restype = _c_int
    lib.ptl_decode_attention_rope_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int,
                                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr,
                                                   _ptr, _ptr, _ptr]
    lib.ptl_decode_attention_rope_bf16.restype = _c_int
    lib.ptl_prefill_attention_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                               _c_int, _c_int, _c_f, _c_int, _c_int, _ptr]
    lib.ptl_prefill_attention_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]
    lib.ptl_gemm_tc_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16_norm.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int,
                                          _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_gemm_tc_bf16_norm.restype = _c_int
    lib.ptl_gemm_small_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr,
                                        _ptr, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_gemm_small_bf16.restype = _c_int
    lib.ptl_finish_norm_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_finish_norm_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16_qkv_rope.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int,
                                              _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_gemm_tc_bf16_qkv_rope.restype = _c_int
    lib.ptl_rope_table.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _ptr]
    lib.ptl_rope_table.restype = _c_int
    lib.ptl_gemm_tc_k_parts.argtypes = [_c_int, _c_int, _c_int]
    lib.ptl_gemm_tc_k_parts.restype = _c_int
    lib.ptl_add_partials.argtypes = [_ptr, _ptr, _c_int, _c_ll, _c_ll, _ptr]
    lib.ptl_add_partials.restype = _c_int
    lib.ptl_prefill_attention_tc_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                  _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _ptr, _ptr]
    lib.ptl_prefill_attention_tc_bf16.restype = _c_int
    lib.ptl_argmax.argtypes = [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_argmax.restype = _c_int
    lib.ptl_take_tokens.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _ptr]
    lib.ptl_take_tokens.restype = _c_int
    lib.ptl_token_logprob.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_token_logprob.restype = _c_int
    lib.ptl_sample.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_sample.restype = _c_int
    lib.ptl_sample_work_words.argtypes = []
    lib.ptl_sample_work_words.restype = _c_int
    lib.ptl_softcap.argtypes = [_ptr, _c_ll, _c_f, _ptr]
    lib.ptl_softcap.restype = _c_int
    lib.ptl_prefill_attention_opts_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                    _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_f, _c_int,
                                                    _c_int, _ptr, _ptr, _c_int, _c_int, _ptr]
    lib.ptl_prefill_attention_opts_bf16.restype = _c_int
    lib.ptl_moe_tile_rows.argtypes = []
    lib.ptl_moe_tile_rows.restype = _c_int
    lib.ptl_moe_route.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr]
    lib.ptl_moe_route.restype = _c_int
    lib.ptl_moe_plan.argtypes = [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]
    lib.ptl_moe_plan.restype = _c_int
    lib.ptl_moe_wide_rows.argtypes = []
    lib.ptl_moe_wide_rows.restype = _c_int
    lib.ptl_moe_grouped_wide_bf16.argtypes = [_ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr]
    lib.ptl_moe_grouped_wide_bf16.restype = _c_int
    lib.ptl_lowrank_tanh_linear.argtypes = [_ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]
    lib.ptl_lowrank_tanh_linear.restype = _c_int
    lib.ptl_head_linear_few_bf16.argtypes = _SIGNATURES["ptl_head_linear"]
    lib.ptl_head_linear_few_bf16.restype = _c_int
    lib.ptl_last_error.restype = ctypes.c_char_p
    lib.ptl_set_dependent_launch.argtypes = [_c_int]
    lib.ptl_get_dependent_launch.restype = _c_int
    if os.environ.get("PTL_DEPENDENT_LAUNCH", "1") == "0":
        lib.ptl_set_dependent_launch(0)
    _LIB = lib
    return lib


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "_f32"
    if dtype == torch.bfloat16:
        return "_bf16"
    raise KernelError(f"unsupported element type {dtype}")


class CudaOps:
    """The operator set of the engine on one CUDA device."""

    name = "cuda"

    def __init__(self, device: torch.device):
        device = torch.device(device)
        if device.type != "cuda":
            raise KernelError(f"the kernels run on CUDA devices only, got {device}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self.device = device
        self.lib = load_library()
        major, minor = torch.cuda.get_device_capability(device)
        if major != 10:
            raise KernelError(f"the kernels are compiled for sm_100a only; device reports sm_{major}{minor}")
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self._device_index = device.index if device.index is not None else torch.cuda.current_device()
        self._sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self.launches = 0      # kernels of this library launched so far (library matrix products not counted)

    # ------------------------------------------------------------------ work lists of a step
    QUERY_TILE = 128   # query rows per tile of the prompt attention kernels; a block takes a pair of consecutive tiles
    WORK_LISTS = {
        # token rows that are the only new token of their request: the split-key decode attention's items
        "decode_items": WorkList(width=1, group=1, pad=PAD_TOKEN_ROW),
        # tiles of longer portions: (request row, first token row, rows, first position); in pairs, the
        # second tile continues the first or has no rows; a padding tile has no rows
        "prefill_tiles": WorkList(width=4, group=2, pad=0),
    }

    def plan_step(self, q_lens, starts):
        """The attention kernels' work lists of a step whose request r brings ``q_lens[r]`` tokens
        after ``starts[r]`` cached ones (host integers; the engine packs them and hands them back on
        the device in ``StepContext.work``)."""
        tile = self.QUERY_TILE
        dec, tiles, t0 = [], [], 0
        for r, (n, s) in enumerate(zip(q_lens, starts)):
            if n == 1:
                dec.append(t0)
            else:
                for a in range(0, n, 2 * tile):       # the kernel fetches every key once for both tiles of a pair
                    b = a + tile
                    tiles += [r, t0 + a, min(tile, n - a), s + a,
                              r, t0 + b, max(0, min(tile, n - b)), s + b]
            t0 += n
        return {"decode_items": dec, "prefill_tiles": tiles}

    def hints_for(self, q_lens, ctx_lens):
        """What the attention operators read of a step context, for callers that launch them
        without an engine (kernel tests, micro-benchmarks): the work lists of a step whose request r
        brings ``q_lens[r]`` tokens and holds ``ctx_lens[r]`` afterwards, on the device."""
        from types import SimpleNamespace
        lists = self.plan_step(list(q_lens), [c - n for n, c in zip(q_lens, ctx_lens)])
        T = sum(q_lens)
        work = {}
        for name, values in lists.items():
            info = self.WORK_LISTS[name]
            t = torch.tensor(values if values else [0], dtype=torch.int32, device=self.device)[:len(values)]
            work[name] = StepWork(t, len(values) // info.width, info.width == 1 and values == list(range(T)))
        return SimpleNamespace(work=work, max_ctx_len=max(ctx_lens), q_lens=list(q_lens), ctx_lens=list(ctx_lens),
                               host_lengths_exact=True)

    @staticmethod
    def _work(hints, name):
        work = getattr(hints, "work", None)
        return work.get(name) if work else None

    # ------------------------------------------------------------------ timing by class of kernels (diagnostic)
    KERNEL_CLASSES = {
        "embed": "elementwise", "take_tokens": "elementwise", "silu_mul": "elementwise", "add_rmsnorm": "norm",
        "embed_scaled": "elementwise", "softcap": "elementwise", "clamped_glu": "elementwise", "token_side": "token_input",
        "causal_conv": "recurrent", "selective_scan": "recurrent", "gated_delta_rule": "recurrent", "gated_head_norm": "norm",
        "kv_write_normed": "attention", "chunk_attention": "attention",
        "linear": "product", "linear_add": "product", "gate_up_silu": "product", "gemm_tc": "product",
        "_qkv_rope_product": "product", "rope_kv_write": "rope", "_rope_table": "rope",
        "paged_attention": "attention", "_attention_tensor_cores": "attention",
        "sample": "sampling", "token_logprobs": "sampling",
        "stream_mix_norm": "norm", "gelu_tanh": "elementwise", "qk_norm_rotate_store": "rope", "window_attention": "attention",
        "gla_scan": "recurrent", "routed_experts": "experts",
        "add_layernorm": "norm", "xielu": "elementwise", "lowrank_tanh_linear": "recurrent", "general_delta_scan": "recurrent",
        "latent_norm_store": "rope", "rotate_head_part": "rope", "head_linear": "product",
        "latent_gather": "attention", "causal_softmax_rows": "attention",
        "head_norm_rotate_store": "rope", "pool_blocks": "attention", "post_norm_add": "norm", "mean_of_normed": "norm",
    }

    def enable_timing(self) -> None:
        """From now on every operator call is bracketed by two CUDA events on the launching stream
        and ``take_timings`` reports the device time by class of kernels.  Operators that only chain
        others (projection, rotation and attention of a mixer) are not timed themselves, their links
        are; of nested timed operators the outermost counts.  Not for captured steps: events recorded
        inside a capture measure nothing."""
        if getattr(self, "_timed", None) is not None:
            return
        self._timed, self._timing_depth = [], 0
        for name, cls in self.KERNEL_CLASSES.items():
            setattr(self, name, self._timed_operator(getattr(self, name), cls))

    def _timed_operator(self, fn, cls):
        def call(*args, **kwargs):
            if self._timing_depth:
                return fn(*args, **kwargs)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._timing_depth += 1
            try:
                start.record()
                out = fn(*args, **kwargs)
                end.record()
            finally:
                self._timing_depth -= 1
            self._timed.append((cls, start, end))
            return out
        return call

    def take_timings(self) -> dict:
        """Milliseconds by class of kernels since the last call (waits for the device); {} when timing is off."""
        if getattr(self, "_timed", None) is None:
            return {}
        torch.cuda.synchronize(self.device)
        out = {}
        for cls, start, end in self._timed:
            out[cls] = out.get(cls, 0.0) + start.elapsed_time(end)
        self._timed = []
        return out

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        """The current stream's handle.  Asked for before every launch (a graph capture changes it), so
        through torch's raw accessor where it has one: building a Stream object each time took 7 us."""
        raw = self._raw_stream
        if raw is not None:
            return raw(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, rc: int, kernels: int = 1) -> None:
        if rc != 0:
            raise KernelError(self.lib.ptl_last_error().decode())
        self.launches += kernels

    def _want(self, t: torch.Tensor, name: str, dtype=None) -> None:
        if t.device != self.device:
            raise KernelError(f"{name} lives on {t.device}, expected {self.device}")
        if not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{name} has element type {t.dtype}, expected {dtype}")

    def empty(self, shape, dtype) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ operators
    def embed(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._want(ids, "ids", torch.int32)
        self._want(table, "table")
        out = self.empty((ids.shape[0], table.shape[1]), table.dtype)
        fn = getattr(self.lib, "ptl_embed_gather" + _suffix(table.dtype))
        self._check(fn(_p(out), _p(table), _p(ids), ids.shape[0], table.shape[1], table.shape[0],
                       _p(self._status), self._stream()))
        return out

    def take_tokens(self, tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor) -> None:
        """tokens[i] = sampled[src[i]] where src[i] >= 0, in place."""
        for name, t in (("tokens", tokens), ("src", src), ("sampled", sampled)):
            self._want(t, name, torch.int32)
        self._check(self.lib.ptl_take_tokens(_p(tokens), _p(src), _p(sampled), tokens.shape[0], sampled.shape[0],
                                             self._stream()))

    def bad_token_seen(self) -> bool:
        """True if an embedding lookup met an id outside the vocabulary since the last call (syncs)."""
        bad = bool(self._status.item())
        if bad:
            self._status.zero_()
        return bad

    def add_rmsnorm(self, x: Optional[torch.Tensor], residual: Optional[torch.Tensor], weight: torch.Tensor,
                    eps: float, rows: Optional[torch.Tensor] = None,
                    dtype: Optional[torch.dtype] = None,
                    bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """y = rmsnorm(residual + x) * weight, the sum kept as the new float32 residual.  ``bias``
        (float32 [hidden]) is added into the sum as well.

        Without ``rows`` the residual tensor is updated in place (created from ``x`` when None).
        With ``rows`` (int32 indices) only those rows are normed and no residual is written."""
        src = x if x is not None else residual
        hidden = src.shape[-1]
        dtype = dtype or (x.dtype if x is not None else None)
        if dtype is None:
            raise KernelError("add_rmsnorm: give dtype when there is no x")
        self._want(weight, "norm weight", torch.float32)
        if x is not None:
            self._want(x, "x", dtype)
        if residual is not None:
            self._want(residual, "residual", torch.float32)
        if rows is not None:
            self._want(rows, "rows", torch.int32)
            n_out = rows.shape[0]
            res_out = None
        else:
            n_out = src.shape[0]
            res_out = residual if residual is not None else self.empty((n_out, hidden), torch.float32)
        y = self.empty((n_out, hidden), dtype)
        if bias is not None:
            self._want(bias, "bias", torch.float32)
            fn = getattr(self.lib, "ptl_add_bias_rmsnorm" + _suffix(dtype))
            self._check(fn(_p(y), _p(res_out), _p(residual), _p(x), _p(bias), _p(weight), _p(rows), n_out, hidden,
                           float(eps), self._stream()))
            return y, res_out
        fn = getattr(self.lib, "ptl_add_rmsnorm" + _suffix(dtype))
        self._check(fn(_p(y), _p(res_out), _p(residual), _p(x), _p(weight), _p(rows), n_out, hidden,
                       float(eps), self._stream()))
        return y, res_out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, fresh_weights: bool = False) -> torch.Tensor:
        """x[T, K] @ w[N, K]^T.  float32: the library's own FFMA kernel (true 32-bit);
        bfloat16: the tensor-core product of this library (a cuBLAS product for sizes it leaves out).
        ``x`` may be a ``NormedActivation``.  ``fresh_weights``: ``w`` was written by an earlier kernel of the same
        step (keys gathered for a product of queries against them).  The tensor-core kernel asks for its first weight
        tiles before it waits for the kernel ahead of it, which is right for a model's weights only; such a product
        is therefore launched as an ordinary successor of what runs before it."""
        if fresh_weights and self.lib.ptl_get_dependent_launch():
            self.lib.ptl_set_dependent_launch(0)
            try:
                return self.linear(x, w, out_dtype)
            finally:
                self.lib.ptl_set_dependent_launch(1)
        if isinstance(x, NormedActivation):
            out = self.gemm_tc(x, w, self.EPI_F32 if out_dtype == torch.float32 else self.EPI_BF16)
            if out is not None:
                return out
            x = x.materialise()
        self._want(x, "x")
        self._want(w, "w", x.dtype)
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: x is [{M},{K}] but w is {list(w.shape)}")
        if x.dtype == torch.float32:
            out = self.empty((M, N), torch.float32)
            self._check(self.lib.ptl_gemm_simt_f32(_p(out), _p(x), _p(w), M, N, K, K, K, N, 0, self._stream()))
            return out
        if not (out_dtype == torch.bfloat16 and self.library_product(M, N, K, self.EPI_BF16)):
            out = self.gemm_tc(x, w, self.EPI_F32 if out_dtype == torch.float32 else self.EPI_BF16)
            if out is not None:
                return out
        # sizes the tensor-core kernel does not take (K no multiple of 8, or below 64) or leaves to the library
        return self._library_mm(x, w, out_dtype)

    @staticmethod
    def _library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """x @ w^T by the library with float32 sums throughout.  torch lets cuBLAS add the parts of a
        split K range in bfloat16 by default; it does so for widths that are no multiple of 8, and
        an element that is small beside the partial sums it is made of then comes out wrong by as
        much as its own size (a [129, 512] x [50, 512]^T product: 0.4 % of the largest element
        everywhere, 43 % of a small one).  The engine's own shapes are not touched by the setting
        (same kernels, same time); it is put back after the call."""
        matmul = torch.backends.cuda.matmul
        before = matmul.allow_bf16_reduced_precision_reduction
        matmul.allow_bf16_reduced_precision_reduction = False
        try:
            if out_dtype == torch.float32:
                return torch.mm(x, w.t(), out_dtype=torch.float32)
            return torch.mm(x, w.t())
        finally:
            matmul.allow_bf16_reduced_precision_reduction = before

    library_products = os.environ.get("PTL_LIBRARY_PRODUCTS", "1") != "0"

    def library_product(self, M: int, N: int, K: int, epi: int) -> bool:
        """True where the plain library product (cuBLAS through torch.mm, which is what lite_llama's
        nn.Linear layers are: lite_llama/models/llama.py:22-24,37-40) is the one to take.  Measured
        on a B200 with cold caches (``python -m pytriton_llama_b200.ops.microbench product_shapes``):
        a product of more than 64 tokens whose 128 x 256 tiles do not fill the SMs twice is faster
        there, by 2 to 10 us, than this library's tcgen05 kernel even after the library's result has
        been rotated by ``rope_kv_write`` or read once more by the norm that adds it to the residual
        (q|k|v, output and down projection at 128 to 2,048 tokens: few tiles, each walking a long K
        range alone).  The products with the SiLU*up epilogue, of few tokens, with float32 results
        and of many tiles stay with the tcgen05 kernel.  ``PTL_LIBRARY_PRODUCTS=0`` keeps everything there."""
        if not self.library_products or M <= 64 or epi not in (self.EPI_BF16, self.EPI_ADD_F32):
            return False
        return -(-M // 128) * -(-N // 256) <= 2 * self._sm_count

    fuses_next_norm = os.environ.get("PTL_FUSED_NORM", "1") != "0"
    small_products = os.environ.get("PTL_SMALL_PRODUCTS", "1") != "0"      # steps of up to 8 tokens: gemm_small for weights of a few MB
    # Steps of up to this many tokens fold the norms into the products around them.  With more
    # tokens a step is no longer bound by the number of kernels, and the add epilogue of the
    # products with a short K range has no time to spare for the extra stores.
    FUSED_NORM_MAX_TOKENS = int(os.environ.get("PTL_FUSED_NORM_MAX", "64"))

    def linear_add(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, next_norm=None):
        """residual += x @ w^T in the product's epilogue (float32 residual, in place) and None; where
        that is not possible the plain product, for the caller to add.  With ``next_norm`` = (weight,
        eps) of the RMS norm that reads the residual next, the epilogue prepares that norm's input
        as well and a ``NormedActivation`` is returned instead of None (where the sizes allow it)."""
        if x.dtype == torch.bfloat16 and residual is not None and not self.library_product(x.shape[0], w.shape[0], x.shape[1], self.EPI_ADD_F32):
            if next_norm is not None and self.fuses_next_norm and x.shape[0] <= self.FUSED_NORM_MAX_TOKENS:
                normed = self.gemm_tc(x, w, self.EPI_ADD_F32, out=residual, emit_norm=next_norm)
                if normed is not None:
                    return normed
            if self.gemm_tc(x, w, self.EPI_ADD_F32, out=residual) is not None:
                return None
        return self.linear(x, w)

    def fused_ffn_layout(self, dtype: torch.dtype, hidden: int, inter: int) -> bool:
        """True if gate and up rows should alternate (gate_0, up_0, gate_1, ...) so that the
        gate/up product can apply SiLU(gate)*up in its epilogue."""
        return dtype == torch.bfloat16 and hidden % 8 == 0 and hidden >= 64

    def gate_up_silu(self, x, w_alternating: torch.Tensor) -> torch.Tensor:
        out = self.gemm_tc(x, w_alternating, self.EPI_SILU_MUL)
        if out is None and isinstance(x, NormedActivation):
            out = self.gemm_tc(x.materialise(), w_alternating, self.EPI_SILU_MUL)
        if out is None:
            raise KernelError("gate_up_silu: sizes not taken; load the weights in the plain layout instead")
        return out

    # epilogues of the tensor-core product
    EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3

    def _tc_status_word(self):
        if getattr(self, "_tc_status", None) is None:
            self._tc_status = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._tc_status

    def gemm_tc(self, x, w: torch.Tensor, epi: int = 0, out: Optional[torch.Tensor] = None,
                splits: int = 0, emit_norm=None):
        """x[M,K] @ w[N,K]^T in bfloat16 on the tcgen05 tensor cores with a fused epilogue.
        ``epi``: EPI_BF16 -> [M,N] bfloat16; EPI_F32 -> [M,N] float32; EPI_ADD_F32 adds into ``out``
        (float32 [M,N], in place); EPI_SILU_MUL -> [M,N/2] bfloat16 for weights whose rows alternate
        gate_j, up_j.  ``x`` may be a ``NormedActivation``: its row scale is applied before the
        epilogue.  ``emit_norm`` = (weight, eps) with EPI_ADD_F32 returns the ``NormedActivation`` of the
        norm that follows.  Returns None when the kernel does not take the sizes."""
        scale = None
        if isinstance(x, NormedActivation):
            scale, x = x, x.xs
        self._want(x, "x", torch.bfloat16)
        self._want(w, "w", torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"gemm_tc: x is [{M},{K}] but w is {list(w.shape)}")
        if K % 8 or K < 64:
            return None
        if epi == self.EPI_ADD_F32:
            if out is None:
                raise KernelError("gemm_tc: the add epilogue needs the float32 tensor to add into")
            self._want(out, "out", torch.float32)
            ld = N
        elif epi == self.EPI_SILU_MUL:
            out = self.empty((M, N // 2), torch.bfloat16)
            ld = N // 2
        elif epi == self.EPI_F32 and M > 64 and splits > 1:
            out = self.empty((splits, M, N), torch.float32)      # partial sums of the parts of the K range
            ld = N
        else:
            out = self.empty((M, N), torch.float32 if epi == self.EPI_F32 else torch.bfloat16)
            ld = N
        if epi == self.EPI_ADD_F32 and scale is None and emit_norm is None and M > 64 and N % 4 == 0 and splits == 0:
            # a few hundred tokens, or a narrow product: too few tiles for the SMs, so the K range is
            # cut into parts as well; their float32 partial sums are added into ``out`` in a fixed order
            parts = self.lib.ptl_gemm_tc_k_parts(M, N, K)
            if parts > 1:
                partial = self.empty((parts, M, N), torch.float32)
                self._check(self.lib.ptl_gemm_tc_bf16(_p(partial), _p(x), _p(w), M, N, K, N, self.EPI_F32,
                                                      _p(self._tc_status_word()), parts, self._stream()))
                self._check(self.lib.ptl_add_partials(_p(out), _p(partial), parts, M * N, M * N, self._stream()))
                return out
        normed = slots = None
        if emit_norm is not None:
            weight, eps = emit_norm
            self._want(weight, "norm weight", torch.float32)
            width = (N + 7) // 8           # a slot per 8 features at most (the product for a few tokens), per 16 otherwise
            normed = NormedActivation(self.empty((M, N), torch.bfloat16), self.empty((M, width), torch.float32), 0,
                                      float(eps), weight, ops=self)
            slots = ctypes.c_int(0)
        if M <= 8 and epi != self.EPI_SILU_MUL and splits == 0 and self.small_products:
            # a few tokens and a weight of a few megabytes (q|k|v and output projection of a decode step): the
            # product without tensor memory and clusters, whose latency is a third; -2 where it does not fit
            rc = self.lib.ptl_gemm_small_bf16(
                _p(out), _p(x), _p(w), M, N, K, ld, epi,
                _p(normed.xs) if normed else None, _p(normed.weight) if normed else None,
                _p(normed.sumsq) if normed else None, normed.sumsq.shape[1] if normed else 0,
                ctypes.byref(slots) if normed else None,
                _p(scale.sumsq) if scale else None, scale.slots if scale else 0, scale.sumsq.shape[1] if scale else 0,
                scale.eps if scale else 0.0, self._stream())
            if rc != -2:
                self._check(rc)
                if normed is not None:
                    normed.slots = slots.value
                    return normed
                return out
        if scale is None and emit_norm is None:
            rc = self.lib.ptl_gemm_tc_bf16(_p(out), _p(x), _p(w), M, N, K, ld, epi, _p(self._tc_status_word()), splits,
                                           self._stream())
            if rc == -2:
                return None
            self._check(rc)
            return out
        rc = self.lib.ptl_gemm_tc_bf16_norm(
            _p(out), _p(x), _p(w), M, N, K, ld, epi, _p(self._tc_status_word()), splits,
            _p(normed.xs) if normed else None, _p(normed.weight) if normed else None,
            _p(normed.sumsq) if normed else None, normed.sumsq.shape[1] if normed else 0,
            ctypes.byref(slots) if normed else None,
            _p(scale.sumsq) if scale else None, scale.slots if scale else 0, scale.sumsq.shape[1] if scale else 0,
            scale.eps if scale else 0.0, self._stream())
        if rc == -2:
            return None
        self._check(rc)
        if normed is not None:
            normed.slots = slots.value
            return normed
        return out

    def check_status(self) -> None:
        """Raises if a kernel flagged a problem since the last call: a token outside the vocabulary
        reached the embedding, or a wait inside a tensor-core kernel gave up (synchronises)."""
        if self.bad_token_seen():
            raise KernelError("a token id outside the vocabulary reached the embedding kernel")
        code = self.gemm_tc_status()
        if code:
            raise KernelError(f"a wait inside a tcgen05 kernel gave up (code {code}); results since the last check are invalid")

    def gemm_tc_status(self) -> int:
        """0, or the code of the wait that gave up inside a tensor-core product since the last call (syncs)."""
        if getattr(self, "_tc_status", None) is None:
            return 0
        code = int(self._tc_status.item())
        if code:
            self._tc_status.zero_()
        return code

    def linear_simt(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The CUDA-core product for any element type (checks of the tensor-core kernels)."""
        self._want(x, "x")
        self._want(w, "w", x.dtype)
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        out = self.empty((M, N), out_dtype)
        if x.dtype == torch.float32:
            fn = self.lib.ptl_gemm_simt_f32
        elif out_dtype == torch.float32:
            fn = self.lib.ptl_gemm_simt_bf16_f32out
        else:
            fn = self.lib.ptl_gemm_simt_bf16
        self._check(fn(_p(out), _p(x), _p(w), M, N, K, K, K, N, 0, self._stream()))
        return out

    def finish_norm(self, normed: NormedActivation) -> torch.Tensor:
        """The RMS norm that a product's epilogue prepared, finished as a plain bfloat16 tensor."""
        tokens, width = normed.xs.shape
        out = self.empty((tokens, width), torch.bfloat16)
        self._check(self.lib.ptl_finish_norm_bf16(_p(out), _p(normed.xs), _p(normed.sumsq), tokens, normed.slots, normed.sumsq.shape[1],
                                                  width, float(normed.eps), self._stream()))
        return out

    def silu_mul(self, gu: torch.Tensor) -> torch.Tensor:
        self._want(gu, "gate_up")
        tokens, two_i = gu.shape
        out = self.empty((tokens, two_i // 2), gu.dtype)
        fn = getattr(self.lib, "ptl_silu_mul" + _suffix(gu.dtype))
        self._check(fn(_p(out), _p(gu), tokens, two_i // 2, self._stream()))
        return out

    def rope_kv_write(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                      rot: int, slots: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                      nq: int, nkv: int, d: int, page_size: int) -> None:
        self._want(qkv, "qkv")
        self._want(positions, "positions", torch.int32)
        if inv_freq is not None:
            self._want(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() < rot // 2:
                raise KernelError("inv_freq shorter than half the rotary width")
        if cache is not None:
            self._want(cache, "cache", qkv.dtype)
            self._want(slots, "slots", torch.int32)
            num_slots = cache.shape[0] * page_size
        else:
            num_slots = 0
        if qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError(f"qkv rows have {qkv.shape[1]} elements, expected {(nq + 2 * nkv) * d}")
        fn = getattr(self.lib, "ptl_rope_kv_write" + _suffix(qkv.dtype))
        self._check(fn(_p(qkv), _p(positions), _p(inv_freq), _p(slots), _p(cache), qkv.shape[0], nq, nkv, d,
                       rot, page_size, num_slots, self._stream()))

    def paged_attention(self, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                        tok_req: torch.Tensor, positions: torch.Tensor, nq: int, nkv: int, d: int,
                        page_size: int, scale: float, window: int = 0, splits: int = 1,
                        hints=None) -> torch.Tensor:
        """q is [T, >= nq*d] (the q part of a qkv buffer is fine); returns [T, nq*d]."""
        self._want(q, "q")
        self._want(cache, "cache", q.dtype)
        self._want(block_table, "block_table", torch.int32)
        self._want(tok_req, "tok_req", torch.int32)
        self._want(positions, "positions", torch.int32)
        tokens = q.shape[0]
        out = self.empty((tokens, nq * d), q.dtype)
        if (q.dtype == torch.bfloat16 and d in (64, 128) and nq // nkv <= 16 and self._work(hints, "decode_items") is not None
                and self._work(hints, "prefill_tiles") is not None):
            self._attention_tensor_cores(out, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                         window, hints)
            return out
        part_acc = part_ml = None
        if splits > 1:
            part_acc = self.empty((tokens, nq, splits, d), torch.float32)
            part_ml = self.empty((tokens, nq, splits, 2), torch.float32)
        fn = getattr(self.lib, "ptl_paged_attention_simt" + _suffix(q.dtype))
        self._check(fn(_p(out), _p(q), _p(cache), _p(block_table), _p(tok_req), _p(positions), _p(part_acc),
                       _p(part_ml), tokens, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                       float(scale), int(window), int(splits), cache.shape[0], self._stream()),
                    kernels=2 if splits > 1 else 1)
        return out

    def rope_attention(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int,
                       slots: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                       tok_req: torch.Tensor, nq: int, nkv: int, d: int, page_size: int, scale: float,
                       window: int = 0, splits: int = 1, hints=None, write: bool = True) -> torch.Tensor:
        """``rope_kv_write`` followed by ``paged_attention``.  A bfloat16 step of single tokens only
        runs both in the decode attention kernel (rotation over the whole head, head sizes 64 and
        128); everything else takes the two kernels."""
        dec, tiles = self._work(hints, "decode_items"), self._work(hints, "prefill_tiles")
        fused = (os.environ.get("PTL_FUSED_ROPE", "1") != "0" and qkv.dtype == torch.bfloat16 and d in (64, 128)
                 and nq // nkv <= 16 and dec is not None and tiles is not None
                 and dec.items == qkv.shape[0] and not tiles.items
                 and (inv_freq is None or rot == d) and qkv.shape[1] >= (nq + 2 * nkv) * d)
        if not fused:
            self.rope_kv_write(qkv, positions, inv_freq, rot, slots if write else None, cache if write else None,
                               nq, nkv, d, page_size)
            return self.paged_attention(qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                        window=window, splits=splits, hints=hints)
        for name, t in (("qkv", qkv), ("cache", cache)):
            self._want(t, name, torch.bfloat16)
        for name, t in (("block_table", block_table), ("tok_req", tok_req), ("positions", positions)):
            self._want(t, name, torch.int32)
        if inv_freq is not None:
            self._want(inv_freq, "inv_freq", torch.float32)
        if write:
            self._want(slots, "slots", torch.int32)
        out = self.empty((qkv.shape[0], nq * d), qkv.dtype)
        self._attention_tensor_cores(out, qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                     window, hints, rope=(inv_freq, slots if write else None))
        return out

    def begin_forward(self) -> None:
        """Called by the model at the start of every forward pass: what was worked out for the last
        step's positions (the table of rotary angles) is forgotten."""
        self._rope_memo = None

    def _rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor, half: int) -> torch.Tensor:
        """(cos, sin) [tokens, half] of this step's angles, worked out once per forward pass and used by every layer."""
        key = (positions.data_ptr(), positions._version, inv_freq.data_ptr(), positions.shape[0], half)
        memo = getattr(self, "_rope_memo", None)
        if memo is not None and memo[0] == key:
            return memo[1]
        table = self.empty((positions.shape[0], half, 2), torch.float32)
        self._check(self.lib.ptl_rope_table(_p(table), _p(positions), _p(inv_freq), positions.shape[0], half, self._stream()))
        self._rope_memo = (key, table)
        return table

    def projected_rope_attention(self, x, w_qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                                 rot: int, slots: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                                 tok_req: torch.Tensor, nq: int, nkv: int, d: int, page_size: int, scale: float,
                                 window: int = 0, splits: int = 1, hints=None, write: bool = True) -> torch.Tensor:
        """The q|k|v projection, ``rope_kv_write`` and ``paged_attention`` of a mixer.  A bfloat16
        step of more than 64 tokens rotates q and k and writes k and v to the cache in the
        projection's epilogue (head sizes 64 and 128, the whole head rotated); everything else
        projects first and goes on with ``rope_attention``."""
        fused = (os.environ.get("PTL_FUSED_QKV_ROPE", "1") != "0" and isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16
                 and x.shape[0] > 64 and write and slots is not None and inv_freq is not None and rot == d and d in (64, 128)
                 and w_qkv.shape[0] == (nq + 2 * nkv) * d and cache.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                 and x.shape[1] >= 64 and not self.library_product(x.shape[0], w_qkv.shape[0], x.shape[1], self.EPI_BF16))
        if fused:
            self._want(x, "x", torch.bfloat16)
            self._want(w_qkv, "w_qkv", torch.bfloat16)
            self._want(cache, "cache", torch.bfloat16)
            self._want(slots, "slots", torch.int32)
            self._want(positions, "positions", torch.int32)
            self._want(inv_freq, "inv_freq", torch.float32)
            M, K = x.shape
            N = w_qkv.shape[0]
            table = self._rope_table(positions, inv_freq, d // 2)
            qkv = self.empty((M, N), torch.bfloat16)          # only the q columns are written (and read)
            if self._qkv_rope_product(qkv, x, w_qkv, table, slots, cache, nq, nkv, d, page_size):
                return self.paged_attention(qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                            window=window, splits=splits, hints=hints)
        qkv = self.linear(x, w_qkv)
        return self.rope_attention(qkv, positions, inv_freq, rot, slots, cache, block_table, tok_req, nq, nkv, d, page_size,
                                   scale, window=window, splits=splits, hints=hints, write=write)

    def _qkv_rope_product(self, qkv, x, w_qkv, table, slots, cache, nq, nkv, d, page_size) -> bool:
        """The q|k|v projection with rotary encoding and the cache write in its epilogue; False where the kernel does not take the sizes."""
        M, K = x.shape
        rc = self.lib.ptl_gemm_tc_bf16_qkv_rope(_p(qkv), _p(x), _p(w_qkv), M, w_qkv.shape[0], K, _p(self._tc_status_word()), _p(table),
                                                _p(slots), _p(cache), nq, nkv, d, page_size,
                                                cache.shape[0] * page_size, self._stream())
        if rc == -2:
            return False
        self._check(rc)
        return True

    DECODE_BLOCKS = int(os.environ.get("PTL_DECODE_BLOCKS", "592"))    # blocks the decode attention aims for: the four per SM that fit at once
    DECODE_KEYS_PER_WIDE_BLOCK = int(os.environ.get("PTL_DECODE_KEYS_PER_WIDE_BLOCK", "1024"))   # keys a block of the two-per-SM form walks at most

    _DECODE_COUNTERS = 1 << 16

    def _attention_tensor_cores(self, out, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                window, hints, rope=None) -> None:
        """bfloat16 attention on the tensor cores: single tokens through the split-key decode kernel,
        longer portions through the tiled prompt kernel; both write their rows of ``out``."""
        stream = self._stream()
        num_pages = cache.shape[0]
        dec, tiles = hints.work["decode_items"], hints.work["prefill_tiles"]
        n_decode, n_tiles = dec.items, tiles.items
        if n_decode:
            longest = min(hints.max_ctx_len, window) if window else hints.max_ctx_len
            pairs = n_decode * nkv
            # small batches: 128-key tiles at two blocks per SM (296 in flight); large ones: 64-key tiles, four per SM
            target = 296 if pairs <= 148 else self.DECODE_BLOCKS
            splits = max(1, min(target // pairs, -(-longest // 128)))
            if target == 296 and splits > 8:
                splits = 8      # what a cluster merges through shared memory; more splits would go through global memory (slower)
            if target == 296 and longest > self.DECODE_KEYS_PER_WIDE_BLOCK * splits:
                # Long contexts at small batches: a block of the cluster form has two 128-key tiles in
                # flight, and with more than eight to walk that no longer covers the memory's latency
                # (one request of 131,072 tokens: 196 us against 55 us).  Four blocks per SM with three
                # 64-key tiles each in flight do, merged by the last block of a token's splits.
                splits = max(splits, min(self.DECODE_BLOCKS // pairs, -(-longest // 128)))
            # The split count of this kernel is decided here, from the number of blocks the machine
            # holds (``attn_splits`` of the step context is the CUDA-core kernel's).  A caller may fix
            # it (``decode_splits``) and leave the counters out (``decode_counters`` False) to pin one
            # of the three ways of merging.
            splits = int(getattr(hints, "decode_splits", 0) or splits)
            part_acc = part_ml = counters = None
            if splits > 1:
                splits = min(splits, 512)
                part_acc = self.empty((q.shape[0], nq, splits, d), torch.float32)
                part_ml = self.empty((q.shape[0], nq, splits, 2), torch.float32)
                if q.shape[0] * nkv <= self._DECODE_COUNTERS and getattr(hints, "decode_counters", True):
                    if getattr(self, "_decode_counters", None) is None:
                        self._decode_counters = torch.zeros(self._DECODE_COUNTERS, dtype=torch.int32, device=self.device)
                    counters = self._decode_counters        # the last block of a token's splits merges them in the kernel
            items = None if dec.in_order else _p(dec.tensor)
            if rope is not None:
                rc = self.lib.ptl_decode_attention_rope_bf16(
                    _p(out), _p(part_acc), _p(part_ml), _p(q), _p(cache), _p(block_table), items, _p(tok_req),
                    _p(positions), n_decode, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                    float(scale), int(window), splits, num_pages, _p(counters), _p(rope[0]), _p(rope[1]), stream)
            else:
                rc = self.lib.ptl_decode_attention_bf16(
                    _p(out), _p(part_acc), _p(part_ml), _p(q), _p(cache), _p(block_table), items, _p(tok_req),
                    _p(positions), n_decode, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                    float(scale), int(window), splits, num_pages, _p(counters), stream)
            group = nq // nkv
            in_cluster = (n_decode * nkv * splits <= 296 and 2 <= splits <= 8
                          and splits * 4 * -(-group // splits) * (d + 2) * 4 <= 16 * 1024)     # as launch_decode decides
            self._check(rc, kernels=2 if splits > 1 and counters is None and not in_cluster else 1)
        if n_tiles:
            if os.environ.get("PTL_PREFILL_TC", "1") != "0":
                rc = self.lib.ptl_prefill_attention_tc_bf16(
                    _p(out), _p(q), _p(cache), _p(block_table), _p(tiles.tensor), n_tiles, q.shape[0],
                    q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size, float(scale), int(window), num_pages,
                    _p(self._tc_status_word()), stream)
                if rc != -2:          # -2: sizes the tcgen05 kernel leaves to the warp-level one
                    self._check(rc)
                    return
            self._check(self.lib.ptl_prefill_attention_bf16(
                _p(out), _p(q), _p(cache), _p(block_table), _p(tiles.tensor), n_tiles, q.shape[1],
                nq * d, block_table.shape[1], nq, nkv, d, page_size, float(scale), int(window), num_pages, stream))

    # ------------------------------------------------------------------ the float32 stream, recurrent and chunked mixers
    def embed_scaled(self, ids: torch.Tensor, table: torch.Tensor, scale: float, positions: torch.Tensor,
                     base: float) -> torch.Tensor:
        """float32 [T, width]: table[ids] * scale, plus (``base`` > 0) the sinusoidal position vector whose entries
        2i and 2i + 1 are sin and cos of position * base^(-2i / width)."""
        self._want(ids, "ids", torch.int32)
        self._want(positions, "positions", torch.int32)
        self._want(table, "table")
        width = table.shape[1]
        freq = None
        if base:
            memo = getattr(self, "_position_freq", None)
            if memo is None or memo[0] != (width, float(base)):
                i = torch.arange((width + 1) // 2, dtype=torch.float64)
                memo = self._position_freq = ((width, float(base)), (float(base) ** (-2.0 * i / width)).to(self.device))
            freq = memo[1]
        out = self.empty((ids.shape[0], width), torch.float32)
        fn = getattr(self.lib, "ptl_embed_scaled" + _suffix(table.dtype))
        self._check(fn(_p(out), _p(table), _p(ids), _p(positions), _p(freq), ids.shape[0], width, table.shape[0], float(scale),
                       _p(self._status), self._stream()))
        return out

    def softcap(self, logits: torch.Tensor, cap: float) -> None:
        """logits <- cap * tanh(logits / cap), in place."""
        self._want(logits, "logits", torch.float32)
        self._check(self.lib.ptl_softcap(_p(logits), logits.numel(), float(cap), self._stream()))

    def clamped_glu(self, gu: torch.Tensor, bias: Optional[torch.Tensor], limit: float, alpha: float, up_shift: float) -> torch.Tensor:
        """gu [T, 2*inter] (gate columns first) + bias -> min(g, limit) * sigmoid(alpha * g) * (clamp(u, +-limit) + up_shift)."""
        self._want(gu, "gate_up")
        if bias is not None:
            self._want(bias, "bias", torch.float32)
        tokens, two_i = gu.shape
        out = self.empty((tokens, two_i // 2), gu.dtype)
        fn = getattr(self.lib, "ptl_clamped_glu" + _suffix(gu.dtype))
        self._check(fn(_p(out), _p(gu), _p(bias), tokens, two_i // 2, float(limit), float(alpha), float(up_shift), self._stream()))
        return out

    def token_side(self, residual: torch.Tensor, x: Optional[torch.Tensor], bias: Optional[torch.Tensor], tokens: torch.Tensor,
                   table: torch.Tensor, column: int, dim: int, w_gate: torch.Tensor, w_proj: torch.Tensor, norm_w: torch.Tensor,
                   eps: float) -> None:
        """residual (float32, in place) <- s + rmsnorm(W_proj (gelu_tanh(W_gate s) * table[token, column:column+dim])) * norm_w
        with s = residual + x + bias."""
        self._want(residual, "residual", torch.float32)
        self._want(tokens, "tokens", torch.int32)
        self._want(table, "table")
        self._want(w_gate, "w_gate", table.dtype)
        self._want(w_proj, "w_proj", table.dtype)
        self._want(norm_w, "norm weight", torch.float32)
        if x is not None:
            self._want(x, "x", table.dtype)
        if bias is not None:
            self._want(bias, "bias", torch.float32)
        fn = getattr(self.lib, "ptl_token_side" + _suffix(table.dtype))
        self._check(fn(_p(residual), _p(x), _p(bias), _p(tokens), _p(table), table.shape[1], int(column), int(dim), table.shape[0],
                       _p(w_gate), _p(w_proj), _p(norm_w), residual.shape[0], residual.shape[1], float(eps), self._stream()))

    def causal_conv(self, x: torch.Tensor, column: int, channels: int, w: torch.Tensor, b: Optional[torch.Tensor],
                    state: torch.Tensor, ctx, silu: bool = True) -> torch.Tensor:
        """Causal convolution per channel over columns ``column``.. of x [T, ld] with the taps w [channels, taps] (the last
        is the current token's); ``state`` [slots, taps - 1, channels] holds each request's last inputs and is moved on."""
        self._want(x, "x")
        self._want(w, "conv weight", torch.float32)
        self._want(state, "conv state", torch.float32)
        if b is not None:
            self._want(b, "conv bias", torch.float32)
        taps = w.shape[1]
        if w.shape[0] != channels or state.shape[1] != max(taps - 1, 1) or state.shape[2] != channels:
            raise KernelError(f"causal_conv: weight {list(w.shape)} and state {list(state.shape)} do not fit {channels} channels")
        out = self.empty((x.shape[0], channels), x.dtype)
        # a step in which every request brings one token (a captured decode step has as many rows as requests, padding
        # included): the kernel that convolves also moves the state on
        single = int(getattr(ctx, "max_q_len", 0) == 1)
        fn = getattr(self.lib, "ptl_causal_conv" + _suffix(x.dtype))
        self._check(fn(_p(out), _p(x), x.shape[1], int(column), int(channels), _p(w), _p(b), taps, _p(state), _p(ctx.q_start),
                       _p(ctx.tok_req), _p(ctx.positions), _p(ctx.state_slot), x.shape[0], ctx.num_requests, int(bool(silu)),
                       single, self._stream()), kernels=2 if taps > 1 and not single else 1)
        return out

    def selective_scan(self, xc: torch.Tensor, dt: torch.Tensor, dt_b: torch.Tensor, A: torch.Tensor, bc: torch.Tensor,
                       D: torch.Tensor, xz: torch.Tensor, z_column: int, state: torch.Tensor, ctx) -> torch.Tensor:
        """The scan of ``parts/scan.py``: xc [T, inner], dt float32 [T, inner] before bias and softplus, A float32
        [inner, n], bc [T, 2n] (B | C), the gate z in columns ``z_column``.. of xz; state float32 [slots, inner, n]."""
        inner, n = A.shape
        self._want(xc, "xc")
        self._want(bc, "bc", xc.dtype)
        self._want(xz, "xz", xc.dtype)
        for name, t in (("dt", dt), ("dt bias", dt_b), ("A", A), ("D", D), ("scan state", state)):
            self._want(t, name, torch.float32)
        if xc.shape[1] != inner or dt.shape != xc.shape or bc.shape[1] != 2 * n or tuple(state.shape[1:]) != (inner, n):
            raise KernelError("selective_scan: shapes do not fit")
        out = self.empty(xc.shape, xc.dtype)
        fn = getattr(self.lib, "ptl_selective_scan" + _suffix(xc.dtype))
        self._check(fn(_p(out), _p(xc), _p(dt), _p(dt_b), _p(A), _p(bc), _p(D), _p(xz), xz.shape[1], int(z_column), inner, n,
                       _p(state), _p(ctx.q_start), _p(ctx.positions), _p(ctx.state_slot), ctx.num_requests, self._stream()))
        return out

    def gated_delta_rule(self, qkv: torch.Tensor, ba: torch.Tensor, rate: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
                         ctx, H: int, G: int, d: int, dv: int, unit_eps: float, q_scale: float) -> torch.Tensor:
        """The recurrence of ``parts/delta_rule.py``: qkv [T, q | k | v] after convolution, ba float32 [T, 2H]; returns the
        heads' read-outs, float32 [T, H*dv]; state float32 [slots, H, d, dv]."""
        self._want(qkv, "qkv")
        for name, t in (("ba", ba), ("rate", rate), ("dt_bias", dt_bias), ("state", state)):
            self._want(t, name, torch.float32)
        if qkv.shape[1] != 2 * G * d + H * dv or ba.shape[1] != 2 * H or tuple(state.shape[1:]) != (H, d, dv):
            raise KernelError("gated_delta_rule: shapes do not fit")
        out = self.empty((qkv.shape[0], H * dv), torch.float32)
        fn = getattr(self.lib, "ptl_gated_delta_rule" + _suffix(qkv.dtype))
        self._check(fn(_p(out), _p(qkv), _p(ba), _p(rate), _p(dt_bias), _p(state), _p(ctx.q_start), _p(ctx.positions),
                       _p(ctx.state_slot), ctx.num_requests, H, G, d, dv, float(unit_eps), float(q_scale), self._stream()))
        return out

    def gated_head_norm(self, o: torch.Tensor, weight: torch.Tensor, eps: float, gate: torch.Tensor, gate_column: int, H: int,
                        dv: int, out: torch.Tensor, column: int, scale: float, gate_kind: str = "silu",
                        weight_per_head: bool = False) -> None:
        """out[:, column + h*dv + e] = o[:, h, e] / rms_e(o[:, h]) * weight[e] * silu(gate[:, gate_column + h*dv + e]) * scale.
        ``gate_kind`` "sigmoid": the gate passes a sigmoid instead; ``weight_per_head``: the weight is [H*dv]."""
        if gate_kind not in ("silu", "sigmoid") or weight.numel() != (H * dv if weight_per_head else dv):
            raise KernelError("gated_head_norm: unknown gate or a weight of the wrong size")
        self._want(o, "o", torch.float32)
        self._want(weight, "norm weight", torch.float32)
        self._want(gate, "gate")
        self._want(out, "out", gate.dtype)
        fn = getattr(self.lib, "ptl_gated_head_norm" + _suffix(gate.dtype))
        self._check(fn(_p(out), out.shape[1], int(column), _p(o), _p(weight), float(eps), _p(gate), gate.shape[1], int(gate_column),
                       o.shape[0], H, dv, float(scale), int(gate_kind == "sigmoid"), int(weight_per_head), self._stream()))

    def kv_write_normed(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], slots: torch.Tensor, cache: torch.Tensor, H: int,
                        G: int, d: int, dv: int, page_size: int, eps: float) -> None:
        """Stores k (+ bias) and v (+ bias, divided by its root mean square per head when eps > 0) of qkv [T, q | k | v]
        in the tokens' slots of a cache whose pages hold keys, then values."""
        self._want(qkv, "qkv")
        self._want(cache, "cache", qkv.dtype)
        self._want(slots, "slots", torch.int32)
        if bias is not None:
            self._want(bias, "bias", torch.float32)
        if qkv.shape[1] != H * d + G * (d + dv) or cache[0].numel() != G * page_size * (d + dv):
            raise KernelError("kv_write_normed: shapes do not fit")
        fn = getattr(self.lib, "ptl_kv_write_normed" + _suffix(qkv.dtype))
        self._check(fn(_p(cache), _p(qkv), _p(bias), _p(slots), qkv.shape[0], H, G, d, dv, page_size, cache.shape[0] * page_size,
                       float(eps), self._stream()))

    def chunk_attention(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                        tok_req: torch.Tensor, positions: torch.Tensor, H: int, G: int, d: int, dv: int, page_size: int,
                        scale: float, chunk: int, r1: Optional[torch.Tensor], r2: Optional[torch.Tensor],
                        talk: Optional[torch.Tensor], out: torch.Tensor, column: int, out_scale: float, max_keys: int = 0) -> None:
        """The attention of ``parts/chunk_attention.py`` for every token of the step; the heads' outputs times
        ``out_scale`` go to columns ``column``.. of ``out``.  ``max_keys``: the most keys a query sees (default: the
        chunk, or every position the block table can name)."""
        self._want(qkv, "qkv")
        self._want(cache, "cache", qkv.dtype)
        self._want(out, "out", qkv.dtype)
        for name, t in (("block_table", block_table), ("tok_req", tok_req), ("positions", positions)):
            self._want(t, name, torch.int32)
        for name, t in (("bias", bias), ("r1", r1), ("r2", r2), ("talk", talk)):
            if t is not None:
                self._want(t, name, torch.float32)
        reach = block_table.shape[1] * page_size
        max_keys = int(max_keys) or (min(chunk, reach) if chunk else reach)
        fn = getattr(self.lib, "ptl_chunk_attention" + _suffix(qkv.dtype))
        self._check(fn(_p(out), out.shape[1], int(column), _p(qkv), qkv.shape[1], _p(bias), _p(cache), _p(block_table),
                       block_table.shape[1], _p(tok_req), _p(positions), qkv.shape[0], H, G, d, dv, page_size, float(scale),
                       int(chunk), _p(r1), _p(r2), _p(talk), max_keys, cache.shape[0], float(out_scale), self._stream()))

    # ------------------------------------------------------------------ copies of the stream, windowed attention, gated linear attention, experts
    def stream_mix_norm(self, streams: Optional[torch.Tensor], init: Optional[torch.Tensor], y: Optional[torch.Tensor],
                        mix: Optional[torch.Tensor], out: Optional[torch.Tensor], read: torch.Tensor, weight: torch.Tensor, eps: float,
                        n_streams: int, rows: Optional[torch.Tensor], dtype: torch.dtype):
        """The write of a sub-layer's output ``y`` to the copies of the stream (float32 [T, S, width], in place:
        new_t = sum_s mix[s, t] old_s + out[t] y) and the read of the next one, u = sum_t read[t] new_t, through an RMS
        norm: (normed [T, width] in ``dtype``, streams).  ``streams`` None: the copies start as ``init`` [T, width].
        With ``rows`` (int32) only those rows are worked and nothing is stored."""
        if streams is None:
            self._want(init, "init", dtype)
            streams = self.empty((init.shape[0], n_streams, init.shape[1]), torch.float32)
        else:
            self._want(streams, "streams", torch.float32)
            init = None
        T, S, width = streams.shape
        if S != n_streams:
            raise KernelError(f"stream_mix_norm: {S} copies of the stream, expected {n_streams}")
        y_f32 = 0
        if y is not None:
            y_f32 = int(y.dtype == torch.float32 and dtype != torch.float32)
            self._want(y, "y", torch.float32 if y_f32 else dtype)
            self._want(mix, "mix", torch.float32)
            self._want(out, "out", torch.float32)
            if tuple(y.shape) != (T, width) or tuple(mix.shape) != (S, S) or out.shape[0] != S:
                raise KernelError("stream_mix_norm: shapes do not fit")
        self._want(read, "read", torch.float32)
        self._want(weight, "norm weight", torch.float32)
        if rows is not None:
            self._want(rows, "rows", torch.int32)
        n_out = rows.shape[0] if rows is not None else T
        normed = self.empty((n_out, width), dtype)
        fn = getattr(self.lib, "ptl_stream_mix_norm" + _suffix(dtype))
        self._check(fn(_p(normed), _p(streams), _p(init), _p(y), y_f32, _p(mix) if y is not None else None,
                       _p(out) if y is not None else None, _p(read), _p(weight), _p(rows), n_out, S, width, float(eps), self._stream()))
        return normed, streams

    def gelu_tanh(self, x: torch.Tensor) -> torch.Tensor:
        """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), float32 inside."""
        self._want(x, "x")
        out = torch.empty_like(x)
        fn = getattr(self.lib, "ptl_gelu_tanh" + _suffix(x.dtype))
        self._check(fn(_p(out), _p(x), x.numel(), self._stream()))
        return out

    def qk_norm_rotate_store(self, proj: torch.Tensor, H: int, G: int, d: int, dv: int, q_norm: Optional[torch.Tensor],
                             k_norm: Optional[torch.Tensor], eps: float, positions: torch.Tensor, freq: Optional[torch.Tensor],
                             dims: int, amplitude: float, slots: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                             page_size: int) -> None:
        """On proj [T, q | k | v] (H heads of d, G of d, G of dv; G = 0: queries only), in place: RMS norm of the whole
        q and of the whole k part with their weights (eps > 0), rotation of the pairs (2i, 2i+1), i < dims/2, of every
        head by position * freq[i] with cos and sin times ``amplitude``; k and v go to the tokens' slots of a cache
        whose pages hold keys, then values."""
        self._want(proj, "proj")
        self._want(positions, "positions", torch.int32)
        for name, t in (("q norm", q_norm), ("k norm", k_norm), ("freq", freq)):
            if t is not None:
                self._want(t, name, torch.float32)
        num_slots = 0
        if G and cache is not None:
            self._want(cache, "cache", proj.dtype)
            self._want(slots, "slots", torch.int32)
            if cache[0].numel() != G * page_size * (d + dv):
                raise KernelError("qk_norm_rotate_store: the cache's pages do not fit the heads")
            num_slots = cache.shape[0] * page_size
        if freq is not None and freq.numel() < dims // 2:
            raise KernelError("qk_norm_rotate_store: fewer frequencies than pairs")
        fn = getattr(self.lib, "ptl_qk_norm_rotate_store" + _suffix(proj.dtype))
        self._check(fn(_p(proj), proj.shape[0], proj.shape[1], H, G, d, dv, _p(q_norm), _p(k_norm), float(eps), _p(positions),
                       _p(freq), int(dims) if freq is not None else 0, float(amplitude), _p(slots) if G else None,
                       _p(cache) if G else None, page_size, num_slots, self._stream()))

    def window_attention(self, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tok_req: torch.Tensor,
                         positions: torch.Tensor, H: int, G: int, d: int, dv: int, page_size: int, scale: float, window: int = 0,
                         keep_first: int = 0, splits: int = 1, hints=None, sink: bool = False, temp_coef: float = 0.0,
                         temp_every: int = 1, shared_values: bool = False, distance_bias: float = 0.0, gate_column: int = -1,
                         pool: int = 0, summary: Optional[torch.Tensor] = None,
                         summary_table: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Softmax attention of every token over the keys j <= p of its request with p - j < window or j < keep_first
        (window 0: all); q is [T, >= H*d], the result [T, H*dv].  ``sink``: one more term of score 0 in the
        denominator; ``temp_coef``: scores of the query at position p times 1 + temp_coef * ln(floor((p + 1) /
        temp_every) + 1); ``shared_values``: the cache's pages hold keys only and a key's first dv entries are its value.
        ``distance_bias`` = c: head h takes 2^(-c (h + 1) / H) * (p - j) off its scores; ``gate_column``: the heads are
        multiplied by the sigmoid of q's columns from there; ``pool`` = P with ``summary`` (pages of mean keys and
        values, laid out as the cache's) and its block table: every block of P positions that lies wholly behind the
        window is seen as its mean."""
        self._want(q, "q")
        self._want(cache, "cache", q.dtype)
        for name, t in (("block_table", block_table), ("tok_req", tok_req), ("positions", positions)):
            self._want(t, name, torch.int32)
        if cache[0].numel() != G * page_size * (d + (0 if shared_values else dv)):
            raise KernelError("window_attention: the cache's pages do not fit the heads")
        tokens = q.shape[0]
        out = self.empty((tokens, H * dv), q.dtype)
        if pool and window:
            self._want(summary, "summary", q.dtype)
            self._want(summary_table, "summary_table", torch.int32)
            if summary[0].numel() != cache[0].numel():
                raise KernelError("window_attention: the pages of block means do not fit the cache's")
            pooled = (int(pool), _p(summary), _p(summary_table), summary_table.shape[1], summary.shape[0])
        else:
            pooled = (0, None, None, 0, 0)
        options = (int(bool(shared_values)), int(bool(sink)), float(temp_coef), int(temp_every), float(distance_bias),
                   int(gate_column), *pooled)
        if (q.dtype == torch.bfloat16 and d == dv and d in (64, 128) and not shared_values and self._work(hints, "prefill_tiles") is not None
                and self._work(hints, "decode_items") is not None and os.environ.get("PTL_WINDOW_TC", "1") != "0"):
            if self._window_attention_tensor_cores(out, q, cache, block_table, tok_req, positions, H, G, d, page_size, scale,
                                                   window, keep_first, hints, options):
                return out
        longest = getattr(hints, "max_ctx_len", 0) or block_table.shape[1] * page_size
        if window:
            longest = min(longest, window + keep_first + (longest // pooled[0] + 32 if pooled[0] else 0))
        splits = self._window_splits(tokens, H, longest)
        self._window_attention_simt(out, q, cache, block_table, tok_req, positions, H, G, d, dv, page_size, scale, window,
                                    keep_first, splits, None, options)
        return out

    def _window_splits(self, tokens: int, H: int, longest: int) -> int:
        """Parts of a token's key list for the CUDA-core kernel: enough warps to fill the SMs, at least 64 keys each."""
        warps = max(1, tokens * H)
        return int(max(1, min(longest // 64, (self._sm_count * 16) // warps, 64)))

    def _window_attention_simt(self, out, q, cache, block_table, tok_req, positions, H, G, d, dv, page_size, scale, window,
                               keep_first, splits, rows, options=(0, 0, 0.0, 1)) -> None:
        """``rows``: None for every token row, else (int32 row indices or None for 0..n-1, n).  ``options``: (values
        inside the keys, sink term, temperature coefficient, temperature step[, distance bias exponent, gate column,
        block length of the means, their pages, their block table, its width, number of their pages])."""
        if len(options) == 4:
            options = (*options, 0.0, -1, 0, None, None, 0, 0)
        tokens = q.shape[0]
        items, n_rows = (None, tokens) if rows is None else rows
        part_acc = part_ml = None
        if splits > 1:
            part_acc = self.empty((tokens, H, splits, dv), torch.float32)
            part_ml = self.empty((tokens, H, splits, 2), torch.float32)
        fn = getattr(self.lib, "ptl_window_attention" + _suffix(q.dtype))
        self._check(fn(_p(out), _p(q), _p(cache), _p(block_table), _p(tok_req), _p(positions), _p(part_acc), _p(part_ml), n_rows,
                       q.shape[1], out.shape[1], block_table.shape[1], H, G, d, dv, page_size, float(scale), int(window),
                       int(keep_first), int(splits), cache.shape[0], _p(items), *options, self._stream()),
                    kernels=2 if splits > 1 else 1)

    def _window_attention_tensor_cores(self, out, q, cache, block_table, tok_req, positions, H, G, d, page_size, scale, window,
                                       keep_first, hints, options=(0, 0, 0.0, 1, 0.0, -1, 0, None, None, 0, 0)) -> bool:
        """bfloat16, key and value heads of 64 or 128: the portions of a step on the tensor cores (the warp-level prompt
        kernel, which walks the kept first keys as key tiles of their own before the window's), its single tokens on
        the CUDA-core kernel with their key lists split; both write their rows of ``out``."""
        dec, tiles = hints.work["decode_items"], hints.work["prefill_tiles"]
        if tiles.items:
            rc = self.lib.ptl_prefill_attention_opts_bf16(
                _p(out), _p(q), _p(cache), _p(block_table), _p(tiles.tensor), tiles.items, q.shape[1], H * d, block_table.shape[1],
                H, G, d, page_size, float(scale), int(window), int(keep_first), cache.shape[0], *options[1:], self._stream())
            if rc == -2:
                return False
            self._check(rc)
        if dec.items:
            longest = getattr(hints, "max_ctx_len", 0) or block_table.shape[1] * page_size
            if window:
                longest = min(longest, window + keep_first + (longest // options[6] + 32 if len(options) > 6 and options[6] else 0))
            self._window_attention_simt(out, q, cache, block_table, tok_req, positions, H, G, d, d, page_size, scale, window,
                                        keep_first, self._window_splits(dec.items, H, longest),
                                        (None if dec.in_order else dec.tensor, dec.items), options)
        return True

    def gla_scan(self, proj: torch.Tensor, z: Optional[torch.Tensor], bias: Optional[torch.Tensor], inv_tau: float,
                 state: torch.Tensor, ctx, H: int, d: int, dv: int, q_scale: float, head_decay: Optional[torch.Tensor] = None,
                 k_scale: float = 1.0) -> torch.Tensor:
        """The recurrence of ``parts/gla.py``: proj [T, q | k | v | ...], z float32 [T, H*d] (the decay's argument before
        its bias); state float32 [slots, H, d, dv]; returns the heads' read-outs, float32 [T, H*dv].  With ``head_decay``
        float32 [H] and no ``z`` every channel of a head decays by that fixed factor (``parts/retention.py``);
        ``k_scale`` multiplies the keys."""
        self._want(proj, "proj")
        self._want(state, "state", torch.float32)
        if z is None:
            self._want(head_decay, "head_decay", torch.float32)
            if head_decay.numel() != H:
                raise KernelError("gla_scan: one decay per head")
        else:
            for name, t in (("z", z), ("bias", bias)):
                self._want(t, name, torch.float32)
            if z.shape[1] != H * d or bias.shape[0] != H * d:
                raise KernelError("gla_scan: shapes do not fit")
        if tuple(state.shape[1:]) != (H, d, dv):
            raise KernelError("gla_scan: shapes do not fit")
        out = self.empty((proj.shape[0], H * dv), torch.float32)
        fn = getattr(self.lib, "ptl_gla_scan" + _suffix(proj.dtype))
        self._check(fn(_p(out), _p(proj), proj.shape[1], _p(z), _p(bias), float(inv_tau), _p(state), _p(ctx.q_start), _p(ctx.positions),
                       _p(ctx.state_slot), ctx.num_requests, H, d, dv, float(q_scale), _p(head_decay) if z is None else None,
                       float(k_scale), self._stream()))
        return out

    # ------------------------------------------------------------------ operators of the Podizen parts
    def head_norm_rotate_store(self, proj: torch.Tensor, H: int, G: int, d: int, dv: int, q_norm: Optional[torch.Tensor],
                               k_norm: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
                               inv_freq: Optional[torch.Tensor], rot: int, slots: Optional[torch.Tensor],
                               cache: Optional[torch.Tensor], page_size: int) -> None:
        """On proj [T, q | k | v | ...] (H heads of d, G of d, G of dv; G = 0: nothing is stored), in place: every q and k
        head divided by its own root mean square and multiplied by the weight [d] of its kind (eps > 0), entries i and
        i + rot/2 of every head turned by position * inv_freq[i] (``inv_freq`` float32 or float64; the angle is worked
        out in 64 bits either way); k and v go to the tokens' slots of a cache whose pages hold keys, then values."""
        self._want(proj, "proj")
        self._want(positions, "positions", torch.int32)
        for name, t in (("q norm", q_norm), ("k norm", k_norm)):
            if t is not None:
                self._want(t, name, torch.float32)
        if inv_freq is not None:
            self._want(inv_freq, "inv_freq")
            if inv_freq.dtype not in (torch.float32, torch.float64):
                raise KernelError("head_norm_rotate_store: frequencies are float32 or float64")
        if eps > 0 and (q_norm.numel() != d or (G and k_norm.numel() != d)):
            raise KernelError("head_norm_rotate_store: the norm weights have the size of a head")
        num_slots = 0
        if G and cache is not None:
            self._want(cache, "cache", proj.dtype)
            self._want(slots, "slots", torch.int32)
            if cache[0].numel() != G * page_size * (d + dv):
                raise KernelError("head_norm_rotate_store: the cache's pages do not fit the heads")
            num_slots = cache.shape[0] * page_size
        if inv_freq is not None and inv_freq.numel() < rot // 2:
            raise KernelError("head_norm_rotate_store: fewer frequencies than pairs")
        fn = getattr(self.lib, "ptl_head_norm_rotate_store" + _suffix(proj.dtype))
        self._check(fn(_p(proj), proj.shape[0], proj.shape[1], H, G, d, dv, _p(q_norm), _p(k_norm), float(eps), _p(positions),
                       _p(inv_freq), int(inv_freq is not None and inv_freq.dtype == torch.float64),
                       int(rot) if inv_freq is not None else 0, _p(slots) if G else None, _p(cache) if G else None,
                       page_size, num_slots, self._stream()))

    def pool_blocks(self, cache: torch.Tensor, block_table: torch.Tensor, tok_req: torch.Tensor, positions: torch.Tensor,
                    summary_slots: torch.Tensor, summary: torch.Tensor, G: int, d: int, dv: int, page_size: int, block: int) -> None:
        """For every token with a slot (>= 0) in ``summary``: the mean key and mean value of the ``block`` positions that
        end with the token's own, read from the cache's pages, written to that slot."""
        self._want(cache, "cache")
        self._want(summary, "summary", cache.dtype)
        for name, t in (("block_table", block_table), ("tok_req", tok_req), ("positions", positions), ("summary_slots", summary_slots)):
            self._want(t, name, torch.int32)
        if cache[0].numel() != G * page_size * (d + dv) or summary[0].numel() != cache[0].numel():
            raise KernelError("pool_blocks: the pages do not fit the heads")
        fn = getattr(self.lib, "ptl_pool_blocks" + _suffix(cache.dtype))
        self._check(fn(_p(summary), _p(cache), _p(block_table), _p(tok_req), _p(positions), _p(summary_slots), positions.shape[0],
                       block_table.shape[1], G, d, dv, page_size, int(block), cache.shape[0], summary.shape[0] * page_size,
                       self._stream()))

    def post_norm_add(self, outs, weights, post_weight: torch.Tensor, eps: float, residual: torch.Tensor, dtype=None,
                      results: Optional[torch.Tensor] = None, index: int = 0, coeffs: Optional[torch.Tensor] = None,
                      next_weight: Optional[torch.Tensor] = None):
        """u = outs[0], or with ``weights`` the mean over m of rmsnorm(outs[m]) * weights[m];  X = residual + rmsnorm(u) *
        post_weight.  With ``results`` float32 [n, T, W]: results[index] = X and the stream becomes
        sum_{j <= index} coeffs[j] * results[j], else the stream is X.  The stream is written over ``residual``.  Returns
        (rmsnorm(stream) * next_weight in ``dtype`` or None, residual).  One kernel."""
        a0 = outs[0]
        self._want(a0, "sub-layer output")
        self._want(residual, "residual", torch.float32)
        self._want(post_weight, "post weight", torch.float32)
        T, W = residual.shape
        dtype = dtype or a0.dtype
        members = 0 if weights is None else len(outs)
        if members > 2 or len(outs) > (members or 1):
            raise KernelError("post_norm_add: at most two members")
        for o in outs:
            if tuple(o.shape) != (T, W) or o.dtype != a0.dtype or not o.is_contiguous():
                raise KernelError("post_norm_add: the outputs do not fit the stream")
        if a0.dtype not in (dtype, torch.float32):
            raise KernelError("post_norm_add: outputs are of the compute type or float32")
        stride = 0
        if results is not None:
            self._want(results, "results", torch.float32)
            self._want(coeffs, "coeffs", torch.float32)
            if tuple(results.shape[1:]) != (T, W) or not 0 <= index < results.shape[0] or coeffs.numel() <= index:
                raise KernelError("post_norm_add: the buffer of results does not fit")
            stride = results.stride(0)
        y = self.empty((T, W), dtype) if next_weight is not None else None
        fn = getattr(self.lib, "ptl_post_norm_add" + _suffix(dtype))
        self._check(fn(_p(a0), _p(outs[1]) if members > 1 else None, _p(weights[0]) if members else None,
                       _p(weights[1]) if members > 1 else None, members, _p(post_weight), float(eps), _p(residual), _p(results),
                       stride, int(index), _p(coeffs), _p(next_weight), _p(y), T, W, int(a0.dtype == torch.float32 and dtype != torch.float32),
                       self._stream()))
        return y, residual

    def mean_of_normed(self, members, eps: float, dtype) -> torch.Tensor:
        """(1 / M) sum_m rmsnorm(x_m) * w_m over ``members`` = [(x_m [T, W], w_m float32 [W])], M <= 2."""
        outs, weights = [x for x, _ in members], [w for _, w in members]
        if not 1 <= len(outs) <= 2:
            raise KernelError("mean_of_normed: one or two members")
        T, W = outs[0].shape
        y = self.empty((T, W), dtype)
        fn = getattr(self.lib, "ptl_post_norm_add" + _suffix(dtype))
        self._check(fn(_p(outs[0]), _p(outs[1]) if len(outs) > 1 else None, _p(weights[0]), _p(weights[1]) if len(outs) > 1 else None,
                       len(outs), None, float(eps), None, None, 0, 0, None, None, _p(y), T, W,
                       int(outs[0].dtype == torch.float32 and dtype != torch.float32), self._stream()))
        return y

    # ------------------------------------------------------------------ operators of the Sogalix parts
    def add_layernorm(self, x: Optional[torch.Tensor], residual: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor,
                      eps: float, rows: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None,
                      add_bias: Optional[torch.Tensor] = None, keep_sum: bool = True):
        """y = layernorm(residual + x (+ add_bias)) * weight + bias, the sum kept as the new float32 residual
        (updated in place; created when ``residual`` is None, unless ``keep_sum`` is False).  With ``rows`` (int32
        indices) only those rows are normed and no residual is written.  ``dtype``: y's element type; float32
        from a bfloat16 ``x`` is allowed."""
        src = x if x is not None else residual
        hidden = src.shape[-1]
        dtype = dtype or (x.dtype if x is not None else None)
        if dtype is None:
            raise KernelError("add_layernorm: give dtype when there is no x")
        self._want(weight, "norm weight", torch.float32)
        self._want(bias, "norm bias", torch.float32)
        if x is not None:
            self._want(x, "x")
            if dtype not in (x.dtype, torch.float32):
                raise KernelError("add_layernorm: y is of x's element type or float32")
        if residual is not None:
            self._want(residual, "residual", torch.float32)
        if add_bias is not None:
            self._want(add_bias, "add_bias", torch.float32)
        if rows is not None:
            self._want(rows, "rows", torch.int32)
            n_out, res_out = rows.shape[0], None
        else:
            n_out = src.shape[0]
            res_out = residual if residual is not None else (self.empty((n_out, hidden), torch.float32) if keep_sum else None)
        y = self.empty((n_out, hidden), dtype)
        x_type = x.dtype if x is not None else dtype
        fn = getattr(self.lib, "ptl_add_layernorm" + _suffix(x_type))
        self._check(fn(_p(y), _p(res_out), _p(residual), _p(x), _p(add_bias), _p(weight), _p(bias), _p(rows), n_out, hidden,
                       float(eps), int(dtype == torch.float32 and x_type != torch.float32), self._stream()))
        return y, res_out

    def xielu(self, x: torch.Tensor, pos_factor: float, neg_factor: float) -> torch.Tensor:
        """z > 0: pos_factor z^2 + z/2;  z <= 0: neg_factor (exp(z) - 1 - z) + z/2; float32 inside."""
        self._want(x, "x")
        out = torch.empty_like(x)
        fn = getattr(self.lib, "ptl_xielu" + _suffix(x.dtype))
        self._check(fn(_p(out), _p(x), x.numel(), float(pos_factor), float(neg_factor), self._stream()))
        return out

    def lowrank_tanh_linear(self, x: torch.Tensor, column: int, w2: torch.Tensor) -> torch.Tensor:
        """tanh(x[:, column:column + rank]) @ w2[n, rank]^T, float32 [T, n]."""
        self._want(x, "x", torch.float32)
        self._want(w2, "w2", torch.float32)
        n, rank = w2.shape
        if column + rank != x.shape[1]:
            raise KernelError("lowrank_tanh_linear: the inner inputs are the last columns of x")
        z = self.empty((x.shape[0], n), torch.float32)
        self._check(self.lib.ptl_lowrank_tanh_linear(_p(z), _p(x), x.shape[0], x.shape[1], int(column), rank, _p(w2), n,
                                                     self._stream()))
        return z

    def general_delta_scan(self, proj: torch.Tensor, aw: torch.Tensor, a_bias: torch.Tensor, z: torch.Tensor, w_bias: torch.Tensor,
                           decay_limit: float, state: torch.Tensor, ctx, H: int, d: int, unit_eps: float) -> torch.Tensor:
        """The recurrence of ``parts/general_delta.py``: proj [T, r | k | v | ...]; aw float32 whose first H*d columns are
        the removal rate's argument before its bias; z float32 [T, H*d], the decay's argument before its bias; state
        float32 [slots, H, d, d]; returns the heads' read-outs, float32 [T, H*d]."""
        self._want(proj, "proj")
        for name, t in (("aw", aw), ("a_bias", a_bias), ("z", z), ("w_bias", w_bias), ("state", state)):
            self._want(t, name, torch.float32)
        n = H * d
        if proj.shape[1] < 3 * n or aw.shape[1] < n or z.shape[1] != n or a_bias.numel() != n or w_bias.numel() != n or \
                tuple(state.shape[1:]) != (H, d, d):
            raise KernelError("general_delta_scan: shapes do not fit")
        out = self.empty((proj.shape[0], n), torch.float32)
        fn = getattr(self.lib, "ptl_general_delta_scan" + _suffix(proj.dtype))
        self._check(fn(_p(out), _p(proj), proj.shape[1], _p(aw), aw.shape[1], _p(a_bias), _p(z), _p(w_bias), float(decay_limit),
                       _p(state), _p(ctx.q_start), _p(ctx.positions), _p(ctx.state_slot), ctx.num_requests, H, d, float(unit_eps),
                       self._stream()))
        return out

    def latent_norm_store(self, proj: torch.Tensor, Q: int, q_norm: torch.Tensor, R: int, kv_norm: Optional[torch.Tensor], n: int,
                          eps: float, positions: torch.Tensor, freq: Optional[torch.Tensor], dims: int,
                          slots: Optional[torch.Tensor], cache: Optional[torch.Tensor], page_size: int) -> torch.Tensor:
        """On proj [T, q latent (Q) | kv latent (R) | rotated key part (n) | ...]: returns the RMS-normed q latent
        [T, Q]; with R > 0 the normed kv latent and the key part, its pairs (2i, 2i+1), i < dims/2, turned by
        position * freq[i], go to the tokens' slots of a cache whose pages hold keys of R + n entries only."""
        self._want(proj, "proj")
        self._want(q_norm, "q norm", torch.float32)
        self._want(positions, "positions", torch.int32)
        num_slots = 0
        if R:
            self._want(kv_norm, "kv norm", torch.float32)
            self._want(cache, "cache", proj.dtype)
            self._want(slots, "slots", torch.int32)
            if freq is not None:
                self._want(freq, "freq", torch.float32)
            if cache[0].numel() != page_size * (R + n) or (dims and (freq is None or freq.numel() < dims // 2)):
                raise KernelError("latent_norm_store: the cache's pages or the frequencies do not fit")
            num_slots = cache.shape[0] * page_size
        out = self.empty((proj.shape[0], Q), proj.dtype)
        fn = getattr(self.lib, "ptl_latent_norm_store" + _suffix(proj.dtype))
        self._check(fn(_p(out), _p(proj), proj.shape[0], proj.shape[1], Q, _p(q_norm), R, _p(kv_norm) if R else None, n if R else 0,
                       float(eps), _p(positions), _p(freq) if R else None, int(dims) if R else 0, _p(slots) if R else None,
                       _p(cache) if R else None, num_slots, self._stream()))
        return out

    LATENT_QUERY_CHUNK = 512        # tokens whose scores against a request's keys are held at a time (all heads)

    def latent_attention(self, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, ctx, H: int, R: int, n: int,
                         page_size: int, scale: float) -> torch.Tensor:
        """Causal softmax attention of H query heads over one kept row [latent (R) | rotated key part (n)] per
        position, the latent being the value: q [T, H*(R+n)] -> [T, H*R].  Single tokens, float32 and steps whose
        host lengths are not the step's own (a captured shape) take the paged kernel; in bfloat16 every prompt
        portion of a step whose context says its host lengths are exact is worked as two tensor-core products
        around a float32 softmax, per request and per ``LATENT_QUERY_CHUNK`` tokens: all heads' queries of the
        chunk against the request's gathered rows, the weights (rounded once) against the gathered latents."""
        d = R + n
        portions = [(r, qn) for r, qn in enumerate(getattr(ctx, "q_lens", []) or []) if qn > 1]
        dec = self._work(ctx, "decode_items")
        composed = (q.dtype == torch.bfloat16 and portions and getattr(ctx, "host_lengths_exact", False) and dec is not None
                    and 32 * (d + 2) * 2 <= 48 * 1024 and os.environ.get("PTL_LATENT_PRODUCTS", "1") != "0")
        if not composed:
            return self.window_attention(q, cache, block_table, ctx.tok_req, ctx.positions, H, 1, d, R, page_size, scale,
                                         splits=getattr(ctx, "attn_splits", 1), hints=ctx, shared_values=True)
        self._want(q, "q")
        self._want(cache, "cache", q.dtype)
        if cache[0].numel() != page_size * d or q.shape[1] != H * d:
            raise KernelError("latent_attention: the cache's pages or the queries do not fit the sizes")
        T = q.shape[0]
        out = self.empty((T, H * R), q.dtype)
        if dec.items:       # the step's single tokens: the paged kernel on their rows
            longest = getattr(ctx, "max_ctx_len", 0) or block_table.shape[1] * page_size
            self._window_attention_simt(out, q, cache, block_table, ctx.tok_req, ctx.positions, H, 1, d, R, page_size, scale, 0, 0,
                                        self._window_splits(dec.items, H, longest),
                                        (None if dec.in_order else dec.tensor, dec.items), (1, 0, 0.0, 1))
        t0 = 0
        starts = {}
        for r, qn in enumerate(ctx.q_lens):
            starts[r] = t0
            t0 += qn
        for r, qn in portions:
            c = int(ctx.ctx_lens[r])
            c_pad = -(-c // 64) * 64
            keys = self.empty((c_pad, d), q.dtype)
            latents_t = self.empty((R, c_pad), q.dtype)
            self.latent_gather(keys, latents_t, cache, block_table, r, c, R, page_size)
            first = c - qn                                  # position of the portion's first token
            for a in range(0, qn, self.LATENT_QUERY_CHUNK):
                b = min(qn, a + self.LATENT_QUERY_CHUNK)
                rows = slice(starts[r] + a, starts[r] + b)
                n_keys = min(c_pad, -(-(first + b) // 64) * 64)      # no row of the chunk sees a later key
                scores = self.linear(q[rows].view((b - a) * H, d), keys[:n_keys], out_dtype=torch.float32, fresh_weights=True)
                weights = self.empty(((b - a) * H, c_pad), q.dtype)
                self.causal_softmax_rows(weights, scores, ctx.positions, rows.start, H, scale)
                out[rows] = self.linear(weights, latents_t, fresh_weights=True).view(b - a, H * R)
        return out

    def latent_gather(self, keys: torch.Tensor, latents_t: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, r: int,
                      ctx_len: int, R: int, page_size: int) -> None:
        """keys [c_pad, d] <- the first ctx_len kept rows of the request in row r of the block table (zeros after them);
        latents_t [R, c_pad] <- their first R entries, keys along the rows."""
        self._want(keys, "keys", cache.dtype)
        self._want(latents_t, "latents_t", cache.dtype)
        self._want(block_table, "block_table", torch.int32)
        c_pad, d = keys.shape
        if tuple(latents_t.shape) != (R, c_pad) or cache[0].numel() != page_size * d or not 0 <= r < block_table.shape[0]:
            raise KernelError("latent_gather: shapes do not fit")
        fn = getattr(self.lib, "ptl_latent_gather" + _suffix(cache.dtype))
        self._check(fn(_p(keys), _p(latents_t), _p(cache), block_table.data_ptr() + 4 * r * block_table.shape[1], int(ctx_len), c_pad,
                       d, R, page_size, cache.shape[0], self._stream()))

    def causal_softmax_rows(self, weights: torch.Tensor, scores: torch.Tensor, positions: torch.Tensor, first_token: int, H: int,
                            scale: float, sink: bool = False) -> None:
        """scores float32 [tokens*H, n_keys] (row = token * H + head, tokens from ``first_token`` of the step on) ->
        weights [tokens*H, >= n_keys]: softmax of scale * score over the keys up to the token's position, zeros beyond."""
        self._want(scores, "scores", torch.float32)
        self._want(weights, "weights")
        self._want(positions, "positions", torch.int32)
        rows, n_keys = scores.shape
        if weights.shape[0] != rows or weights.shape[1] < n_keys or rows % H or first_token + rows // H > positions.shape[0]:
            raise KernelError("causal_softmax_rows: shapes do not fit")
        fn = getattr(self.lib, "ptl_causal_softmax_rows" + _suffix(weights.dtype))
        self._check(fn(_p(weights), weights.shape[1], _p(scores), rows, n_keys, positions.data_ptr() + 4 * first_token, H,
                       float(scale), int(bool(sink)), self._stream()))

    HEAD_FEW_MAX_TOKENS = int(os.environ.get("PTL_HEAD_FEW_MAX", "16"))              # tokens up to which the heads' products take the row-per-warp kernel
    HEAD_PRODUCT_MIN_TOKENS = int(os.environ.get("PTL_HEAD_PRODUCT_MIN", "128"))     # tokens from which the heads' products go to the library

    def head_linear(self, x: torch.Tensor, x_ld: int, x_col: int, w: torch.Tensor, out: torch.Tensor, out_ld: int, out_col: int,
                    H: int, gate: Optional[torch.Tensor] = None, gate_column: int = 0) -> None:
        """For every head h: out[:, h*out_ld + out_col + o] = sum_i x[:, h*x_ld + x_col + i] * w[h, o, i], with ``gate``
        times sigmoid(gate[:, gate_column + h]).  x rows hold H heads of x_ld entries, out rows H heads of out_ld."""
        self._want(x, "x")
        self._want(w, "w", x.dtype)
        self._want(out, "out", x.dtype)
        n_out, n_in = w.shape[1], w.shape[2]
        if w.shape[0] != H or x.shape[1] != H * x_ld or out.shape[1] != H * out_ld or x_col + n_in > x_ld or out_col + n_out > out_ld:
            raise KernelError("head_linear: shapes do not fit")
        gate_ptr = None
        if gate is not None:
            self._want(gate, "gate", x.dtype)
            gate_ptr = gate.data_ptr() + gate_column * gate.element_size()
        T = x.shape[0]
        if x.dtype == torch.bfloat16 and T >= self.HEAD_PRODUCT_MIN_TOKENS and self.library_products:
            # many tokens: one batched product of the library on the tensor cores (float32 sums), the operands
            # and the result addressed in place by their strides; the heads' gates by a kernel of their own
            a = x.view(T, H, x_ld)[:, :, x_col:x_col + n_in].transpose(0, 1)            # [H, T, n_in]
            o = out.view(T, H, out_ld)[:, :, out_col:out_col + n_out].transpose(0, 1)    # [H, T, n_out]
            matmul = torch.backends.cuda.matmul
            before = matmul.allow_bf16_reduced_precision_reduction
            matmul.allow_bf16_reduced_precision_reduction = False
            try:
                torch.bmm(a, w.transpose(1, 2), out=o)
            finally:
                matmul.allow_bf16_reduced_precision_reduction = before
            if gate is not None:
                self._check(self.lib.ptl_head_gate_bf16(_p(out), out_ld, out_col, n_out, T, H, gate_ptr, gate.shape[1], self._stream()))
            return
        fn = getattr(self.lib, "ptl_head_linear" + _suffix(x.dtype))
        if (x.dtype == torch.bfloat16 and T <= self.HEAD_FEW_MAX_TOKENS and n_in % 8 == 0 and n_in <= 1536 and x_ld % 8 == 0
                and x_col % 8 == 0 and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            fn = self.lib.ptl_head_linear_few_bf16          # few tokens: a warp per output feature reads its weight row once
        self._check(fn(out.data_ptr() + out_col * out.element_size(), x.data_ptr() + x_col * x.element_size(), _p(w), x.shape[0],
                       n_out, n_in, x.shape[1], out.shape[1], H, x_ld, out_ld, gate_ptr, gate.shape[1] if gate is not None else 0,
                       self._stream()))

    def rotate_head_part(self, x: torch.Tensor, x_ld: int, x_col: int, out: torch.Tensor, out_ld: int, out_col: int, H: int, n: int,
                         positions: torch.Tensor, freq: Optional[torch.Tensor], dims: int) -> None:
        """The n entries at x_col of every head of x go to out_col of the same head of out, their pairs (2i, 2i+1),
        i < dims/2, turned by position * freq[i]."""
        self._want(x, "x")
        self._want(out, "out", x.dtype)
        self._want(positions, "positions", torch.int32)
        if freq is not None:
            self._want(freq, "freq", torch.float32)
        if x.shape[1] != H * x_ld or out.shape[1] != H * out_ld:
            raise KernelError("rotate_head_part: shapes do not fit")
        fn = getattr(self.lib, "ptl_rotate_head_part" + _suffix(x.dtype))
        self._check(fn(_p(out), out_ld, out_col, _p(x), x_ld, x_col, x.shape[0], H, n, _p(positions), _p(freq),
                       int(dims) if freq is not None else 0, self._stream()))

    moe_tensor_cores = os.environ.get("PTL_MOE_TC", "1") != "0"
    MOE_WIDE_MIN_ROWS = int(os.environ.get("PTL_MOE_WIDE_MIN", "512"))   # (token, choice) pairs from which tiles of 128 rows pay

    def routed_experts(self, x: torch.Tensor, logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, top: int,
                       scale_input: bool, shared: Optional[torch.Tensor], score: str = "sigmoid", groups: int = 1,
                       keep_groups: int = 1, renormalise: bool = False) -> torch.Tensor:
        """x [T, width], router logits float32 [T, E], expert weights [E, 2*inter, width] (gate rows, then up rows) and
        [E, width, inter]: every token's ``top`` experts by sigmoid(logit), weighted by that score on the expert's input
        (``scale_input``) or output, summed, plus ``shared`` [T, width]; float32 [T, width].  ``score`` "softmax": the
        scores are the softmax over all experts; ``groups`` > 1: only experts of the ``keep_groups`` groups of neighbours
        with the largest best score can be chosen; ``renormalise``: chosen scores divided by their sum.  Six kernels and no word
        back to the host: route, plan (sort by expert), gather, two grouped products, combine.  The products walk tiles
        of 32 rows of one expert; in bfloat16 steps with many tokens walk tiles of 128 rows."""
        self._want(x, "x")
        self._want(logits, "logits", torch.float32)
        self._want(w_gate_up, "expert gate/up weights", x.dtype)
        self._want(w_down, "expert down weights", x.dtype)
        if shared is not None:
            self._want(shared, "shared", x.dtype)
        T, width = x.shape
        E, two_inter, _ = w_gate_up.shape
        inter = two_inter // 2
        if logits.shape[1] != E or tuple(w_down.shape) != (E, width, inter) or w_gate_up.shape[2] != width:
            raise KernelError("routed_experts: shapes do not fit")
        n = T * top
        tile = self.lib.ptl_moe_tile_rows()
        max_tiles = -(-n // tile) + min(E, n)
        use_wide = (x.dtype == torch.bfloat16 and self.moe_tensor_cores and n >= self.MOE_WIDE_MIN_ROWS and width % 8 == 0
                    and inter % 8 == 0)
        max_wide = -(-n // self.lib.ptl_moe_wide_rows()) + min(E, n) if use_wide else 0
        stream = self._stream()
        ints = self.empty((2 * n + 3 * max_tiles + 3 * max_wide + 4,), torch.int32)
        ids, pos, tiles = ints[:n], ints[n:2 * n], ints[2 * n:2 * n + 3 * max_tiles]
        wide = ints[2 * n + 3 * max_tiles:2 * n + 3 * max_tiles + 3 * max_wide] if use_wide else None
        meta = ints[2 * n + 3 * max_tiles + 3 * max_wide:]
        weights = self.empty((n,), torch.float32)
        if score not in ("sigmoid", "softmax"):
            raise KernelError(f"routed_experts: score {score!r}")
        self._check(self.lib.ptl_moe_route(_p(ids), _p(weights), _p(logits), T, E, top, int(score == "softmax"), int(groups),
                                           int(keep_groups) if groups > 1 else 1, int(bool(renormalise)), stream))
        self._check(self.lib.ptl_moe_plan(_p(pos), _p(tiles), _p(meta), _p(ids), n, E, max_tiles, _p(wide), max_wide, stream))
        rows = max_tiles * tile
        sorted_x = self.empty((rows, width), x.dtype)
        sfx = _suffix(x.dtype)
        self._check(getattr(self.lib, "ptl_moe_gather" + sfx)(_p(sorted_x), _p(x), _p(pos), _p(weights), n, top, width,
                                                              int(bool(scale_input)), stream))
        hidden = self.empty((rows, inter), x.dtype)
        tc = int(self.moe_tensor_cores)
        grouped = getattr(self.lib, "ptl_moe_grouped" + sfx)
        y = self.empty((rows, width), torch.float32)
        if use_wide:
            self._check(self.lib.ptl_moe_grouped_wide_bf16(_p(hidden), inter, _p(sorted_x), _p(w_gate_up), _p(wide), _p(meta), max_wide,
                                                           two_inter, width, 1, stream))
            self._check(self.lib.ptl_moe_grouped_wide_bf16(_p(y), width, _p(hidden), _p(w_down), _p(wide), _p(meta), max_wide, width,
                                                           inter, 0, stream))
        else:
            self._check(grouped(_p(hidden), inter, _p(sorted_x), _p(w_gate_up), _p(tiles), _p(meta), max_tiles, two_inter, width, 1, tc, stream))
            self._check(grouped(_p(y), width, _p(hidden), _p(w_down), _p(tiles), _p(meta), max_tiles, width, inter, 0, tc, stream))
        out = self.empty((T, width), torch.float32)
        self._check(getattr(self.lib, "ptl_moe_combine" + sfx)(_p(out), _p(y), _p(shared), _p(pos), _p(weights), T, top, width,
                                                               int(bool(scale_input)), stream))
        return out

    def token_logprobs(self, logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        """log softmax(logits[row])[tokens[row]] as float32 [rows]."""
        self._want(logits, "logits", torch.float32)
        self._want(tokens, "tokens", torch.int32)
        rows, vocab = logits.shape
        out = self.empty((rows,), torch.float32)
        scratch = self.empty((2, rows, 32), torch.float32)   # per row the maxima of 32 slices and their sums of exponentials
        self._check(self.lib.ptl_token_logprob(_p(out), _p(logits), _p(tokens), _p(scratch[0]), _p(scratch[1]), rows, vocab, vocab,
                                               self._stream()), kernels=2)
        return out

    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
               u: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 token per row (written to ``out`` if given); rows with temperature <= 0 (or
        temperature None) take the argmax."""
        self._want(logits, "logits", torch.float32)
        rows, vocab = logits.shape
        if out is None:
            out = self.empty((rows,), torch.int32)
        else:
            self._want(out, "out", torch.int32)
            if out.shape[0] != rows:
                raise KernelError(f"sample: out has {out.shape[0]} rows, the logits {rows}")
        if temperature is None and rows <= 65535:
            scratch = self.empty((2, rows, 32), torch.float32)   # per row 32 best values, and (as int32) their indices
            self._check(self.lib.ptl_argmax(_p(out), _p(logits), _p(scratch[0]), _p(scratch[1]), rows, vocab, vocab,
                                            self._stream()), kernels=2)
            return out
        probs = work = None
        kernels = 2
        if temperature is not None:
            for name, t in (("temperature", temperature), ("top_p", top_p), ("u", u)):
                self._want(t, name, torch.float32)
            probs = self.empty((rows, vocab), torch.float32)
            work = self._sample_work(rows)
            kernels = 6
        scratch = self.empty((2, rows, 32), torch.float32)   # per row the maxima of 32 slices, and (as int32) their indices
        self._check(self.lib.ptl_sample(_p(out), _p(logits), _p(probs), _p(temperature), _p(top_p), _p(u), _p(scratch[0]),
                                        _p(scratch[1]), _p(work), rows, vocab, vocab, self._stream()), kernels=kernels)
        return out

    def _sample_work(self, rows: int) -> torch.Tensor:
        """The histograms of the sampling kernels: zero before the first call, and every call leaves
        them zero, so one buffer serves all calls on this device's stream."""
        have = getattr(self, "_sample_work_buf", None)
        words = self.lib.ptl_sample_work_words()
        if have is None or have.numel() < rows * words:
            cap = max(64, 1 << (rows - 1).bit_length())
            self._sample_work_buf = have = torch.zeros(cap * words, dtype=torch.int64, device=self.device)
        return have

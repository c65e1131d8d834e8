"""Loads the compiled kernel libraries and declares their C signatures.

The kernels are the only implementation of their operations: there is no CPU or
framework fallback.  If the library cannot be built or loaded, or no CUDA device
is present, the first use raises ``KernelsUnavailable``.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict

from ..csrc import build as _build


class KernelsUnavailable(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


P, I, F, LL = c_void_p, c_int, c_float, c_longlong

_CORE_SIGNATURES = {
    "slb_embedding_f32": [P, P, P, I, I, I, F, P],
    "slb_embedding_bf16": [P, P, P, I, I, I, F, P],
    "slb_logit_transform": [P, I, I, I, F, F, P],
    "slb_add_rmsnorm_f32": [P, P, P, P, P, I, I, F, P],
    "slb_add_rmsnorm_bf16": [P, P, P, P, P, I, I, F, P],
    "slb_swiglu_f32": [P, P, I, I, I, I, I, P],
    "slb_swiglu_bf16": [P, P, I, I, I, I, I, P],
    "slb_qkv_rope_cache_f32": [P, I, P, P, P, P, I, I, I, P, I, P, I, P, P, I, I, I, I, P],
    "slb_qkv_rope_cache_bf16": [P, I, P, P, P, P, I, I, I, P, I, P, I, P, P, I, I, I, I, P],
    "slb_cache_write_status": [I],
    "slb_paged_attention_generic_f32": [P, I, P, P, P, I, P, I, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "slb_paged_attention_generic_bf16": [P, I, P, P, P, I, P, I, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "slb_paged_attention_generic_status": [I],
    "slb_paged_attention_generic_tile_rows": [],
    "slb_gemm_simt_f32": [P, I, P, I, P, I, P, I, I, I, P],
    "slb_gemm_simt_bf16": [P, I, P, I, P, I, P, I, I, I, P],
    "slb_gemm_simt_bf16_f32out": [P, I, P, I, P, I, P, I, I, I, P],
    "slb_sample_rows": [P, I, I, I, P, P, P, P, P, P, P, P],
    "slb_gemm_tc_decode_bf16": [P, I, P, I, P, I, P, P, I, I, I, I, I, I, I, I, P, I, F, I, P],
    "slb_split_sum": [P, P, I, P, I, I, I, I, P],
    "slb_gemm_tc_cluster_bf16": [P, I, P, I, P, I, P, I, I, I, I, I, P, I, F, I, P],
    "slb_gemm_tc_qkv_rope_bf16": [P, I, P, I, P, P, P, P, I, I, I, P, I, P, I, P, P, I, I, I, I, I, I, I,
                                  P, I, F, I, P],
    "slb_gemm_tc_resid_norm_bf16": [P, I, P, I, P, P, I, P, P, I, P, I, I, I, I, I, I, P],
    "slb_add_rmsnorm_parts_bf16": [P, P, I, LL, P, P, P, P, I, I, F, P],
    "slb_qkv_rope_cache_parts_bf16": [P, I, LL, I, P, P, P, P, I, I, I, P, I, P, I, P, P, I, I, I, I, P],
    "slb_gemm_tc_status": [I],
}

# optional entry points: declared when the library exports them
_OPTIONAL_SIGNATURES = {}

_libs: Dict[str, ctypes.CDLL] = {}
_pdl = True
_pdl_early = False
trace_buffer = None        # device address of a timeline buffer (``ops.timeline``) or None


def loaded_libraries():
    return list(_libs.values())


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of this package: a kernel may
    be scheduled while its predecessor in the stream drains (each kernel waits on
    the device for its predecessor before it touches activations).  Applies to the
    libraries loaded so far and to those loaded later."""
    global _pdl
    _pdl = bool(on)
    for lib in _libs.values():
        lib.slb_set_pdl(1 if _pdl else 0)


def pdl_enabled() -> bool:
    return _pdl


_FLAG_PDL_EARLY, _FLAG_EVICT_FIRST = 1, 2
_evict_first = True


def _kernel_flags() -> int:
    return (_FLAG_PDL_EARLY if _pdl_early else 0) | (_FLAG_EVICT_FIRST if _evict_first else 0)


def set_pdl_early(on: bool) -> None:
    """The long kernels (matrix products, decode attention) let their successor be scheduled
    at their start instead of after their main loop: its blocks become resident beside theirs
    wherever an SM has room and fetch their first weight tiles meanwhile."""
    global _pdl_early
    _pdl_early = bool(on)
    for lib in _libs.values():
        lib.slb_set_kernel_flags(_kernel_flags())


def set_evict_first(on: bool) -> None:
    """What a step streams once (weights, the cache) is fetched with the L2 policy "evict first",
    so that the activations between the kernels stay in the L2 cache (on by default)."""
    global _evict_first
    _evict_first = bool(on)
    for lib in _libs.values():
        lib.slb_set_kernel_flags(_kernel_flags())


def _apply_switches(lib: ctypes.CDLL) -> None:
    lib.slb_set_pdl.argtypes = [I]
    lib.slb_set_pdl(1 if _pdl else 0)
    lib.slb_set_kernel_flags.argtypes = [I]
    lib.slb_set_kernel_flags(_kernel_flags())
    lib.slb_set_trace.argtypes = [P, I]
    lib.slb_set_trace(trace_buffer, len(_libs))


def _declare(lib: ctypes.CDLL, sigs: dict, required: bool) -> None:
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if required:
                raise KernelsUnavailable(f"kernel library lacks symbol {name}") from None
            continue
        fn.argtypes = args
        fn.restype = c_int


def core() -> ctypes.CDLL:
    lib = _libs.get("core")
    if lib is None:
        try:
            path = _build.ensure_library()
            lib = ctypes.CDLL(path)
        except (OSError, _build.BuildError) as e:
            raise KernelsUnavailable(f"the servelab_b200 CUDA kernels are not available: {e}") from e
        _declare(lib, _CORE_SIGNATURES, True)
        _declare(lib, _OPTIONAL_SIGNATURES, False)
        _apply_switches(lib)
        _libs["core"] = lib
    return lib


_ATTN_SIGNATURES = {
    "slb_prefill_attention_bf16": [P, I, P, P, P, I, P, I, P, P, P, P, I, I, I, I, I, F, I, P],
    "slb_decode_attention_bf16": [P, I, P, P, P, I, P, I, P, P, I, I, I, I, I, F, I, I, P],
    "slb_prefill_attention_tile_rows": [],
    "slb_decode_attention_max_splits": [],
    "slb_attention_head_dim": [],
    "slb_attention_status": [I],
    "slb_prefill_attention_tc_supported": [I, I],
    "slb_prefill_attention_tc_tile_rows": [I],
    "slb_prefill_attention_tc_status": [I],
    "slb_prefill_attention_tc_where": [P],
    "slb_decode_attention_ws_bf16": [P, I, P, P, P, I, P, I, P, P, P, I, I, I, I, I, F, I, I, I, F, I, I, P],
    "slb_decode_attention_ws_max_cluster_splits": [],
    "slb_decode_attention_ws_supported": [I],
    "slb_decode_attention_ws_status": [I],
    "slb_decode_attention_ws_splits_used": [I],
    "slb_decode_attention_ws_max_splits": [],
    "slb_decode_attention_ws_tile_keys": [],
}


def attention(head_dim: int) -> ctypes.CDLL:
    key = f"attn{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        try:
            lib = ctypes.CDLL(_build.attention_library(head_dim))
        except (OSError, _build.BuildError) as e:
            raise KernelsUnavailable(
                f"the attention kernels for head size {head_dim} are not available: {e}") from e
        _declare(lib, _ATTN_SIGNATURES, True)
        if hasattr(lib, "slb_prefill_attention_tc_bf16"):
            lib.slb_prefill_attention_tc_bf16.argtypes = [P, I, P, P, P, I, P, I, P, P, P, P, I, I, I, I, I,
                                                          F, I, P]
            lib.slb_prefill_attention_tc_bf16.restype = I
        lib.slb_decode_attention_scratch_bytes.argtypes = [I, I, I]
        lib.slb_decode_attention_scratch_bytes.restype = ctypes.c_longlong
        lib.slb_decode_attention_ws_scratch_bytes.argtypes = [I, I, I]
        lib.slb_decode_attention_ws_scratch_bytes.restype = ctypes.c_longlong
        lib.slb_decode_attention_ws_counters.argtypes = [I, I, I]
        lib.slb_decode_attention_ws_counters.restype = ctypes.c_longlong
        if lib.slb_attention_head_dim() != head_dim:
            raise KernelsUnavailable(f"attention library built for head size "
                                     f"{lib.slb_attention_head_dim()}, wanted {head_dim}")
        _apply_switches(lib)
        _libs[key] = lib
    return lib


# measurements: called with the kernel's name after every launch of this package's kernels
# (``ops.profile.StepProfile`` records a CUDA event there); None costs one comparison a launch
after_launch = None


def check(code: int, what: str) -> None:
    if code == 0:
        if after_launch is not None:
            after_launch(what)
        return
    if code == -1:
        raise KernelError(f"{what}: arguments refused (a size or pointer the kernel does not take)")
    if code == -2:
        raise KernelError(f"{what}: a size is beyond the kernel's stated maximum")
    raise KernelError(f"{what}: CUDA error {code} at launch")

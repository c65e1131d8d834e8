"""Matrix products y = x W^T (+ b) for weights stored [out, in].

float32: always this package's CUDA-core kernel (true 32-bit, fixed summation
order per output).  bfloat16: the vendor library's tensor-core GEMM through
torch (the reference's engine also calls a library for its products,
servelab/parallel/tp_model.py:48-53), except for shapes whose rows are not
16-byte aligned, which go to the CUDA-core kernel, and for small token counts
(decode steps), which go to this package's tcgen05 weight-streaming kernel
(TMA-fed, accumulating in tensor memory).  An mma.sync weight-streaming kernel
also exists and is off by default.
"""

from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import kernels as K
from . import library as L

skinny_max_tokens = 0      # up to this many tokens the weight-streaming kernel runs (0: the
                           # library GEMM measured faster inside a captured step)
use_skinny = True          # switch for measurements


def _skinny_ok(x, w, M):
    return (use_skinny and M <= skinny_max_tokens and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


tc_max_tokens = 16         # up to this many tokens the tcgen05 weight-streaming kernel runs
tc_wide_max_tokens = 64    # ... and up to this many for products wide enough to need no K split
                           # (gate|up: 45.5 us against the library's 47.7 at 64 tokens; the narrow
                           # products lose to it above 16 tokens: their partial sums grow with M)
# Hand the K-split partial sums of a decode-step product to the kernel that consumes the
# result instead of reducing them in a kernel of their own, per kind of consumer.  "rope":
# the q/k/v kernel takes them with one block per (head, token).  "norm": the norm takes
# them with a cluster of blocks per row.  Each replaces the reduction kernel and the
# one-block-per-token form of itself (measured at batch 8 / 1 on the 7B shape: 3.31 / 3.13
# ms a step without, 3.28 / 3.10 with "rope", 3.22 / 3.04 with both).
defer_split_sums = {"rope": True, "norm": True}
fuse_swiglu = True         # the gate|up product of a decode step applies the activation itself


# Which weights follow which in a forward pass, by address: a hint with which the tcgen05
# product warms the L2 cache for its successor.  Set by the model after loading; a
# matrix used twice keeps its last successor (the hint may be wrong, never harmful).
# Weak references: the table keeps no model's weights alive.
_successor = {}


def set_weight_order(matrices) -> None:
    """``matrices``: the weight matrices in the order a forward pass multiplies by them;
    the last is followed by the first (the next step)."""
    _successor.clear()
    ms = [m for m in matrices if m is not None]
    for a, b in zip(ms, ms[1:] + ms[:1]):
        if a.data_ptr() != b.data_ptr():
            _successor[a.data_ptr()] = weakref.ref(b)


def _next_weight(w):
    ref = _successor.get(w.data_ptr())
    return ref() if ref is not None else None


def _tc_ok(x, w, M):
    limit = tc_max_tokens
    if M > limit and K.tc_decode_splits(w.shape[0], w.shape[1]) == 1:
        limit = max(limit, tc_wide_max_tokens)
    return (0 < M <= min(limit, K.TC_MAX_TOKENS) and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``w_gate_up`` [2I, h]: gate rows then up rows
    (``block`` 0), or alternating in runs of ``block`` rows.  Decode steps in bfloat16
    apply the activation in the product's epilogue; everything else runs the product and
    then the activation kernel."""
    M = x.shape[0]
    inter = w_gate_up.shape[0] // 2
    if (fuse_swiglu and x.dtype == torch.bfloat16 and block == K.SWIGLU_BLOCK and _tc_ok(x, w_gate_up, M)
            and K.tc_decode_splits(w_gate_up.shape[0], w_gate_up.shape[1]) == 1):
        return K.gemm_tc_decode(x, w_gate_up, None, swiglu=True, next_weight=_next_weight(w_gate_up))
    gu = linear(x, w_gate_up)
    act = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    K.swiglu(gu, act, block)
    return act


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, consumer: Optional[str] = None):
    """``consumer`` ("rope" or "norm"): the caller hands the result to a kernel of that
    kind, which accepts a ``SplitSum`` (partial sums of a K-split product); it may then
    get one instead of a tensor."""
    M, Kd = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        K.gemm_simt(x, w, out, bias)
        return out
    # bfloat16 activations
    if M == 0:
        return torch.empty((0, N), dtype=out_dtype, device=x.device)
    if _tc_ok(x, w, M):
        return K.gemm_tc_decode(x, w, None, bias, defer_sum=defer_split_sums.get(consumer, False),
                                out_dtype=out_dtype, next_weight=_next_weight(w))
    if _skinny_ok(x, w, M):
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_skinny(x, w, out, bias)
        return out
    if Kd % 8 or N % 8:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        K.gemm_simt(x, w, out, bias)
        return out
    if out_dtype == torch.float32:
        out = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            out += bias
        return out
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, w.t())
    return torch.mm(x, w.t())

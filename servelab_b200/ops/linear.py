"""Matrix products y = x W^T (+ b) for weights stored [out, in].

float32: always this package's CUDA-core kernel (true 32-bit, fixed summation
order per output).  bfloat16: the vendor library's tensor-core GEMM through
torch (the reference's engine also calls a library for its products,
servelab/parallel/tp_model.py:48-53), except for shapes whose rows are not
16-byte aligned, which go to the CUDA-core kernel, and for small token counts
(decode steps), which go to this package's tcgen05 weight-streaming kernels
(TMA-fed, accumulating in tensor memory).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K
from .profile import mark as _mark

tc_max_tokens = 16         # up to this many tokens the tcgen05 weight-streaming kernels run whatever the
                           # product's shape (above: see ``cluster_max_tokens_per_block``)
tc_wide_max_tokens = 64    # ... and up to this many for products wide enough to need no K split
                           # (gate|up: 45.5 us against the library's 47.7 at 64 tokens)
# (The plain twin of the cluster products, taken when ``cluster_sums`` is off.)  Hand the
# K-split partial sums of a decode-step product to the kernel that consumes the
# result instead of reducing them in a kernel of their own, per kind of consumer.  "rope":
# the q/k/v kernel takes them with one block per (head, token).  "norm": the norm takes
# them with a cluster of blocks per row.  Each replaces the reduction kernel and the
# one-block-per-token form of itself (measured at batch 8 / 1 on the 7B shape: 3.31 / 3.13
# ms a step without, 3.28 / 3.10 with "rope", 3.22 / 3.04 with both).
defer_split_sums = {"rope": True, "norm": True}
fuse_swiglu = True         # the gate|up product of a decode step applies the activation itself
# The product that closes a residual branch (o, down) of a decode step also does the add and
# the RMS norm that follow it: its epilogue updates the float32 stream and writes the normed
# rows without their factor 1 / rms, which the next product (q|k|v, gate|up) applies in its own
# epilogue.  The two norm kernels of a layer are not launched.
fuse_resid_norm = True


def _w_ok(w) -> bool:
    return w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0


def _tc_ok(x, w, M):
    limit = tc_max_tokens
    if M > limit and K.tc_decode_splits(w.shape[0], w.shape[1], K.tc_token_groups(M, w)) == 1:
        limit = max(limit, tc_wide_max_tokens)
    return (0 < M <= min(limit, K.TC_MAX_TOKENS) and _w_ok(w)
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


# The K splits of a decode-step product's row tile run as one thread-block cluster and add
# their results through shared memory, so the product needs neither partial sums in global
# memory nor a kernel that adds them.  Measured on the 7B shape at 8 tokens, product and the
# kernel after it, in a graph: o 10.4 -> 9.6 us; the q|k|v product with bias, rotation and
# cache write in its epilogue 11.7 -> 9.7 us.  Products with long K ranges (down: 37 k-blocks a
# block with the 8 splits a cluster allows, against 30 with 10) gained from it once the blocks
# fetched one another's sums together instead of one after the other: the batch-8 step went
# from 2.97 to 2.91 ms with down in the cluster form and a plain norm after it, instead of
# float32 partial sums that a cluster of norm blocks adds.
cluster_sums = True
cluster_max_kblocks = 64   # k-blocks (of 64) per block up to which the cluster form is used
cluster_max_tokens_per_block = 8  # tokens a block of the cluster may finish in its epilogue for a
                                  # product of more than 16 tokens (a warp a token, two tokens in
                                  # flight per warp).  Measured against the library's GEMMs for the
                                  # narrow products, ms a decode step on the 7B shape (8 K splits) at
                                  # 17 / 24 / 32 / 48 / 64 requests: 3.04 / 3.47 / 3.43 / 3.95 / 4.43
                                  # against 3.51 / 3.70 / 3.61 / 4.00 / 4.42 -- this package's kernels
                                  # chain through programmatic dependent launch and carry rotation,
                                  # cache write, residual add and norm in their epilogues.  With few
                                  # row tiles (the 0.5B shape: 3 K splits, 22 tokens a block at 64
                                  # requests) the library stays faster: 1.39 against 1.67 ms a step.
cluster_long_k_kblocks = 16      # products whose blocks stream more k-blocks than this ("long K") ...
cluster_long_k_max_tokens = 64   # ... use the cluster form also from 17 tokens up to here
fuse_qkv_rope = True       # the q|k|v product of a decode step rotates and writes the cache itself


def _cluster_ok(x, w, M) -> bool:
    if not (cluster_sums and x.dtype == torch.bfloat16 and 0 < M <= K.TC_MAX_TOKENS and _w_ok(w)
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
        return False
    N, Kd = w.shape
    groups = K.tc_token_groups(M, w)
    want = K.tc_decode_splits(N, Kd, groups)
    if want <= 1:
        return False
    if groups > 1:
        M = K.tc_token_group                   # (what a block sees)
    per_block = -(-(-(-Kd // 64)) // min(want, K.TC_MAX_CLUSTER))      # k-blocks of 64 a block streams
    if per_block > cluster_max_kblocks:
        return False
    if M <= tc_max_tokens:
        return True
    # Above that a block of the cluster finishes its share of the tokens one after the other in
    # its epilogue (tokens rank, rank + splits, ...): the cluster form is taken while that
    # share stays small, or for long K ranges (down), where streaming the weights is most of
    # the time either way (30.8 against 34.1 us with the norm at 64 tokens, 7B shape).
    splits = min(want, K.TC_MAX_CLUSTER)
    if -(-M // splits) <= cluster_max_tokens_per_block:
        return True
    return per_block > cluster_long_k_kblocks and M <= cluster_long_k_max_tokens


def qkv_projection(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor], positions,
                   seq_of_token, block_table, page_size: int, inv_freq, rotary_dim: int,
                   q_out: torch.Tensor, k_cache, v_cache, num_heads: int, num_kv_heads: int,
                   head_dim: int) -> None:
    """q|k|v = x W^T + bias, q and k rotated, q into ``q_out``, k and v into the paged cache
    (``k_cache`` None: no cache write).  One kernel for decode steps in bfloat16 with a head
    size the product's epilogue takes; otherwise the product, then the q/k/v kernel."""
    M = x.shape[0]
    xt = x.z if isinstance(x, K.ScaledRows) else x
    if (fuse_qkv_rope and xt.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
            and head_dim in K.TC_ROPE_HEAD_DIMS and _cluster_ok(xt, w_qkv, M)):
        K.gemm_tc_qkv_rope(x, w_qkv, bias, positions, seq_of_token, block_table, page_size, inv_freq,
                           rotary_dim, q_out, k_cache, v_cache, num_heads, num_kv_heads, head_dim)
        return
    qkv = linear(x, w_qkv, consumer="rope")                # the next kernel may add K-split parts
    K.qkv_rope_cache(qkv, bias, positions, seq_of_token, block_table, page_size, inv_freq,
                     rotary_dim, q_out, k_cache, v_cache, num_heads, num_kv_heads, head_dim)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``w_gate_up`` [2I, h]: gate rows then up rows
    (``block`` 0), or alternating in runs of ``block`` rows.  Decode steps in bfloat16
    apply the activation in the product's epilogue; everything else runs the product and
    then the activation kernel."""
    M = x.shape[0]
    inter = w_gate_up.shape[0] // 2
    xt = x.z if isinstance(x, K.ScaledRows) else x
    if (fuse_swiglu and xt.dtype == torch.bfloat16 and block == K.SWIGLU_BLOCK
            and K.tc_decode_splits(w_gate_up.shape[0], w_gate_up.shape[1],
                                   K.tc_token_groups(M, w_gate_up)) == 1
            and _tc_ok(xt, w_gate_up, M)):
        return K.gemm_tc_decode(x, w_gate_up, None, swiglu=True)
    gu = linear(x, w_gate_up)
    act = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    K.swiglu(gu, act, block)
    return act


def which_kernel(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> str:
    """The kernel ``linear`` runs for these operands: "simt" (CUDA cores), "tc_cluster" /
    "tc" (this package's tcgen05 kernels, K splits as a cluster / as partial sums or
    unsplit), "vendor" (library GEMM) or "empty"."""
    M, Kd = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        return "simt"
    if M == 0:
        return "empty"
    if out_dtype == torch.bfloat16 and _cluster_ok(x, w, M):
        return "tc_cluster"
    if _tc_ok(x, w, M):
        return "tc"
    if Kd % 8 or N % 8:
        return "simt"
    return "vendor"


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, consumer: Optional[str] = None):
    """``consumer`` ("rope" or "norm"): the caller hands the result to a kernel of that
    kind, which accepts an unfinished form: a ``SplitSum`` (partial sums of a K-split
    product) or, for "norm", a ``DeferredLinear`` (the product not launched yet: the norm
    launches it with itself in the epilogue).  The caller may then get one instead of a
    tensor and passes it on through ``plain_unless``."""
    M, N = x.shape[0], w.shape[0]
    out_dtype = out_dtype or x.dtype
    kernel = which_kernel(x.z if isinstance(x, K.ScaledRows) else x, w, out_dtype)
    if kernel not in ("tc_cluster", "tc"):
        x = K.plain_unless(None, x)            # (only this package's tcgen05 kernels take ScaledRows)
    if kernel == "empty":
        return torch.empty((0, N), dtype=out_dtype, device=x.device)
    if kernel == "tc_cluster":
        if consumer == "norm" and fuse_resid_norm:
            return K.DeferredLinear(x, w, bias)
        return K.gemm_tc_cluster(x, w, None, bias)
    if kernel == "tc":
        return K.gemm_tc_decode(x, w, None, bias, defer_sum=defer_split_sums.get(consumer, False),
                                out_dtype=out_dtype)
    if kernel == "simt":
        out = torch.empty((M, N), dtype=torch.float32 if x.dtype == torch.float32 else out_dtype,
                          device=x.device)
        K.gemm_simt(x, w, out, bias)
        return out
    if out_dtype == torch.float32:
        out = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            out += bias
    elif bias is not None:
        out = torch.addmm(bias.to(x.dtype), x, w.t())
    else:
        out = torch.mm(x, w.t())
    _mark("library gemm")
    return out

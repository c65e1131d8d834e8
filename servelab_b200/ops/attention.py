"""Chooses and launches the attention kernel for a step.

  float32                      plain kernel (CUDA cores, float32 throughout)
  bfloat16, all q_len == 1     split-KV decode kernel (tensor cores)
  bfloat16, otherwise          tensor-core prefill kernel
  bfloat16, head size not a    plain kernel
  multiple of 16

``force_generic`` switches every call to the plain kernel (tests and
measurements compare the fast kernels with it).
"""

from __future__ import annotations

import torch

from . import kernels as K
from . import library as L

force_generic = False
use_decode_kernel = True
use_prefill_kernel = True
MAX_HEAD_DIM = 256


def check_supported(head_dim: int, dtype: torch.dtype) -> None:
    if head_dim < 1 or head_dim > MAX_HEAD_DIM:
        raise L.KernelError(f"attention kernels take head sizes 1..{MAX_HEAD_DIM}, got {head_dim}")


def _generic(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale, window):
    g = H // Hkv
    tile_seq, tile_row0, n = ctx.attention_tiles(g, K.generic_attention_tile_rows())
    K.paged_attention_generic(q, k_cache, v_cache, out, table, ctx.cu_q, ctx.ctx_len, tile_seq,
                              tile_row0, n, H, Hkv, D, page_size, scale, window)


def paged_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale,
                    window) -> None:
    if q.dtype == torch.bfloat16 and not force_generic and K.has_fast_attention(D):
        if ctx.decode_only and use_decode_kernel:
            K.decode_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale,
                               window)
            return
        if use_prefill_kernel:
            K.prefill_attention(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size,
                                scale, window)
            return
    _generic(ctx, q, k_cache, v_cache, out, table, H, Hkv, D, page_size, scale, window)

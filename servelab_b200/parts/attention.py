"""Grouped-query softmax attention over the paged cache.

Per step: one fused q|k|v product (weights concatenated at load), then one
kernel that adds the q/k/v bias, rotates q and k by the token positions and
writes k (rotated) and v into the request's pages, then attention of every query
of the step over its request's cached keys (the step's own included), then the
output projection.  In bfloat16 decode steps the product's own epilogue does the second of
these (``ops.linear.qkv_projection``).  Order and formulas:
servelab/parallel/tp_model.py:48-53 (projections with bias), :128-129 (rotation before the cache write), :136-157
(scores * D^-1/2, causal mask, float32 softmax, P.V), :131 (bias-free output
projection).  ``window`` limits the visible keys to the last w positions.

Which attention kernel runs: float32 always takes the plain kernel; bfloat16
takes the tensor-core kernels when they exist for the head size (decode kernel
for steps of single tokens, prefill kernel otherwise) and the plain kernel else.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import linear, qkv_projection
from ..weights.source import BIAS, MATRIX, TensorDecl
from .base import Mixer
from .registry import POSITIONS, build_part, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    graph_safe = True
    accepts_scaled_rows = True        # ``x`` may be ScaledRows: the q|k|v product applies 1 / rms

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.position = build_part(POSITIONS, spec.position, f"{prefix}.{spec.position_name}", env)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        A.check_supported(spec.head_dim, env.dtype)
        if env.dtype == torch.bfloat16 and K.has_fast_attention(spec.head_dim) \
                and torch.cuda.is_available():
            from ..ops import library
            library.attention(spec.head_dim)      # built now, not in the middle of a step

    @classmethod
    def declare(cls, spec, prefix):
        h, q, kv = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        qn, kn, vn, on = (f"{prefix}.{n}" for n in (spec.q_name, spec.k_name, spec.v_name, spec.o_name))
        out = [TensorDecl(qn + ".weight", (q, h), MATRIX), TensorDecl(kn + ".weight", (kv, h), MATRIX),
               TensorDecl(vn + ".weight", (kv, h), MATRIX), TensorDecl(on + ".weight", (h, q), MATRIX)]
        if spec.qkv_bias:
            out += [TensorDecl(qn + ".bias", (q,), BIAS), TensorDecl(kn + ".bias", (kv,), BIAS),
                    TensorDecl(vn + ".bias", (kv,), BIAS)]
        if spec.out_bias:
            out.append(TensorDecl(on + ".bias", (h,), BIAS))
        return out

    @classmethod
    def cache_request(cls, spec):
        return PagedKVRequest(spec.num_kv_heads, spec.head_dim, spec.window)

    def load(self, store):
        s = self.spec
        qn, kn, vn, on = (f"{self.prefix}.{n}" for n in (s.q_name, s.k_name, s.v_name, s.o_name))
        self.w_qkv = store.cat([qn + ".weight", kn + ".weight", vn + ".weight"])
        self.b_qkv = store.cat([qn + ".bias", kn + ".bias", vn + ".bias"]) if s.qkv_bias else None
        self.w_o = store.get(on + ".weight")
        self.b_o = store.get(on + ".bias") if s.out_bias else None

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]                        # (x may be ScaledRows: the q|k|v product applies 1 / rms)
        table = ctx.block_tables[cache.group]
        rot = self.position.rotary_table()
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        device = x.device
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=device)
        k_cache, v_cache = (cache.k, cache.v) if owns_cache else (None, None)
        if self.position.transforms_qk:
            x = K.plain_unless(None, x)
            # an encoding of its own on the projected q and k: product with bias, the
            # encoding in place, then the q/k/v kernel without rotation (copy + cache write)
            qkv = linear(x, self.w_qkv, self.b_qkv)
            self.position.apply_to_qk(
                ctx, qkv[:, :self.q_size].view(T, s.num_heads, s.head_dim),
                qkv[:, self.q_size:self.q_size + self.kv_size].view(T, s.num_kv_heads, s.head_dim))
            K.qkv_rope_cache(qkv, None, ctx.positions, ctx.seq_of_token, table, cache.page_size,
                             None, 0, q, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim)
        else:
            qkv_projection(x, self.w_qkv, self.b_qkv, ctx.positions, ctx.seq_of_token, table,
                           cache.page_size, inv_freq, rotary_dim, q, k_cache, v_cache, s.num_heads,
                           s.num_kv_heads, s.head_dim)
        out = torch.empty_like(q)
        A.paged_attention(ctx, q, cache.k, cache.v, out, table, s.num_heads, s.num_kv_heads,
                          s.head_dim, cache.page_size, self.scale, s.window or 0)
        return linear(out, self.w_o, self.b_o, consumer="norm")

"""RMSNorm fused with the residual add that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (tests/test_triton_kernels.py:57-59,
servelab/attention/triton/paged_attention.py:76-91 in the reference); the weight
is held in float32.
"""

from __future__ import annotations

import torch

from ..ops import kernels as K
from ..weights.source import NORM, TensorDecl
from .base import Norm
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    accepts_split_sum = True      # ``delta`` may be a SplitSum (parts of a K-split product)
    accepts_deferred_linear = True    # ... or a product not launched yet, which then runs with the
                                      # add and this norm in its epilogue; the result is ScaledRows

    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + ".weight", (spec.dim,), NORM)]

    def load(self, store):
        self.weight = store.get(self.prefix + ".weight")

    def forward(self, ctx, resid, delta, out_rows=None):
        if isinstance(delta, K.DeferredLinear):
            if out_rows is None and self.env.dtype == torch.bfloat16:
                return K.gemm_tc_resid_norm(delta.x, delta.w, delta.bias, resid, self.weight,
                                            self.spec.eps)
            delta = delta.materialize()
        rows = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((rows, self.spec.dim), dtype=self.env.dtype, device=resid.device)
        K.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out, out_rows)
        return out

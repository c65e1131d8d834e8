"""Checked access to a model's tensors with the engine's precision policy.

Policy, by role of the tensor:
  * matrices (GEMM operands, the embedding table) go to the compute dtype:
    bfloat16 for serving, float32 for the 32-bit path (float16 checkpoints are
    converted; no tensor is kept in float16);
  * norm weights and biases are kept in float32 whatever their stored dtype
    (exact for bfloat16 sources; a tensor stored in 32-bit stays so), because
    the kernels that use them compute in float32;
  * integer tables become int32.
"""

from __future__ import annotations

from typing import Dict, Iterable, List

import torch

from .source import BIAS, MATRIX, NORM, TABLE, TensorDecl, WeightSource, check_source


class WeightStore:
    def __init__(self, source: WeightSource, decls: Iterable[TensorDecl],
                 compute_dtype: torch.dtype, device: str,
                 ignored_suffixes=(), optional=()):
        self.decls: Dict[str, TensorDecl] = {d.name: d for d in decls}
        check_source(source, self.decls.values(), ignored_suffixes, optional)
        self.source = source
        self.compute_dtype = compute_dtype
        self.device = device

    def device_dtype(self, name: str) -> torch.dtype:
        role = self.decls[name].role
        if role == TABLE:
            return torch.int32
        if role in (NORM, BIAS):
            return torch.float32
        return self.compute_dtype

    def get(self, name: str) -> torch.Tensor:
        """The named tensor on the device, contiguous, in its policy dtype."""
        t = self.source.read(name)
        return t.to(device=self.device, dtype=self.device_dtype(name)).contiguous()

    def cat(self, names: List[str], dim: int = 0) -> torch.Tensor:
        """Several checkpoint tensors fused along ``dim`` into one device tensor."""
        return torch.cat([self.get(n) for n in names], dim=dim).contiguous()

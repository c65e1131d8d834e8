"""Interfaces of the parts a layer is put together from.

A part is built from its spec (sizes and constants as parameters), declares the
checkpoint tensors it needs under a name prefix, loads them from a checked
``WeightStore`` and runs on the tokens of one step.  No part knows which model it
is in: everything it needs arrives through its spec, its prefix, the
``BuildEnv`` and, per step, the ``StepContext`` (``engine/batch.py``).

Kinds of part and what each must provide (beyond ``declare`` and ``load``):

  PositionEncoding   one of three seams.  ``rotary_table()`` -> (inv_freq float32
                     [rotary_dim/2], rotary_dim) or None: rotate-half, fused into the
                     mixer's q/k kernel.  ``apply_to_qk(ctx, q, k)`` with
                     ``transforms_qk = True``: any other encoding that acts on the
                     projected queries [T, H, D] and keys [T, Hkv, D] (bias already
                     added) in place, before the keys reach the cache.
                     ``apply_to_embedding(ctx, resid)``: encodings added to the
                     embedded tokens (default: nothing).
  Norm               ``forward(ctx, resid, delta, out_rows=None)``: adds ``delta``
                     (compute dtype, may be None) into the float32 stream ``resid``
                     in place and returns the normed rows in the compute dtype;
                     with ``out_rows`` (int32 row indices) only those rows are
                     produced and ``resid`` is left as it is.
  Mixer              ``cache_request(spec)`` (class method) -> PagedKVRequest,
                     FixedStateRequest or None; ``forward(ctx, x, cache,
                     owns_cache)`` -> [T, hidden] in the compute dtype.  ``cache``
                     is the ``LayerCache`` of the layer whose cache this run uses;
                     with ``owns_cache`` False the mixer must not write it.
  FeedForward        ``forward(ctx, x)`` -> [T, hidden] in the compute dtype.
  Block              ``forward(ctx, resid, delta, cache, owns_cache)`` ->
                     (resid, delta): the float32 stream and a not-yet-added
                     update, so that the add fuses with the next norm.

Optional, for parts that want to take part in kernel fusion across part boundaries: an
update handed from one part to the next may be unfinished (``ops.kernels.SplitSum``: the
float32 partial sums of a K-split product, which the consuming kernel adds itself).  A part
says that it takes the form with the class attribute ``accepts_split_sum``; a part that does
not set it always gets plain tensors.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..weights.source import TensorDecl
from ..weights.store import WeightStore


@dataclass
class BuildEnv:
    """What every part may know about the engine it is built into."""
    device: str
    dtype: torch.dtype            # compute dtype: torch.bfloat16 or torch.float32
    page_size: int = 16


@dataclass
class LayerCache:
    """Device memory of one layer's cache, handed to its mixer each step.

    Paged: ``k`` and ``v`` are [num_pages, kv_heads, page_size, head_dim] and
    ``group`` indexes ``ctx.block_tables``.  Fixed state: ``state`` is
    [num_slots, *shape] float32, indexed by ``ctx.state_slots``.
    """
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    page_size: int = 0


class Part:
    # True iff forward() only launches kernels on device buffers of the step
    # context (no host-side reads of the batch), so a step can be graph-captured
    graph_safe = False

    def __init__(self, spec, prefix: str, env: BuildEnv):
        self.spec, self.prefix, self.env = spec, prefix, env

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return []

    def load(self, store: WeightStore) -> None:
        pass


class PositionEncoding(Part):
    transforms_qk = False         # True: the mixer calls apply_to_qk() instead of rotating

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return None

    def apply_to_qk(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        """Change q [T, H, D] and k [T, Hkv, D] (views of the step's projection, bias
        added) in place by the tokens' positions (``ctx.positions``)."""
        raise NotImplementedError

    def apply_to_embedding(self, ctx, resid: torch.Tensor) -> None:
        pass


class Norm(Part):
    def forward(self, ctx, resid, delta, out_rows=None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_request(cls, spec):
        return None

    def forward(self, ctx, x, cache: LayerCache, owns_cache: bool) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    def forward(self, ctx, resid, delta, cache: LayerCache, owns_cache: bool):
        raise NotImplementedError

    @classmethod
    def cache_request(cls, spec):
        raise NotImplementedError

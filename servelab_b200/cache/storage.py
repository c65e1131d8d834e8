"""Device memory of the cache: pages per layer group, state records per layer.

``plan_groups`` sorts the cache requests of the run order's entries into groups:
paged requests with equal (kv heads, head size, window) share a group (one page
pool, one block table per request); runs that read an earlier run's cache own
nothing.  "layer" below means an entry of the run order.  Page
layout of one layer: k and v each [num_pages, kv_heads, page_size, head_dim], so
the page_size x head_dim tile of one (page, kv head) is contiguous.  The
reference keeps [layers, rows, kv_heads, head_dim] (servelab/kv_cache/pool.py:54-57).

Sizing follows the reference's rule (servelab/engine/engine.py:273-288): free
device bytes x utilisation / bytes per page across all layers.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import LayerCache
from .manager import FixedStateRequest, PagedKVRequest


@dataclass
class GroupPlan:
    request: PagedKVRequest
    layers: List[int]


def plan_groups(requests: Sequence[Optional[object]]) -> Tuple[List[GroupPlan], Dict[int, int]]:
    """(groups, layer -> group index) for the paged layers, in first-seen order."""
    groups: List[GroupPlan] = []
    of_layer: Dict[int, int] = {}
    for layer, req in enumerate(requests):
        if not isinstance(req, PagedKVRequest):
            continue
        for gi, g in enumerate(groups):
            if g.request == req:
                g.layers.append(layer)
                of_layer[layer] = gi
                break
        else:
            groups.append(GroupPlan(req, [layer]))
            of_layer[layer] = len(groups) - 1
    return groups, of_layer


def bytes_per_page(groups: Sequence[GroupPlan], page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page costs when every group gets the same number of pages."""
    el = torch.empty((), dtype=dtype).element_size()
    return sum(2 * len(g.layers) * g.request.num_kv_heads * g.request.head_dim * page_size * el
               for g in groups)


def pages_from_memory(groups, page_size, dtype, free_bytes: int, utilization: float) -> int:
    per = bytes_per_page(groups, page_size, dtype)
    if per == 0:
        return 16
    return max(16, int(free_bytes * utilization / per))


# What unwritten slots hold in the debugging mode: finite (the fast kernels multiply masked
# keys' values by a probability of zero, which NaN or infinity would not survive), and so
# large that a key that is read although it was never written takes the whole softmax and
# shows in the logits.
POISON = 1e30


class CacheStorage:
    def __init__(self, requests: Sequence[Optional[object]], num_pages: int, page_size: int,
                 num_state_slots: int, dtype: torch.dtype, device: str, poison: bool = False):
        """``poison``: a debugging mode in which every slot that no request has written holds
        ``POISON`` instead of zeros: fresh pages at the start, and pages again when they are
        given back (``poison_pages``).  A kernel that reads a slot it should not see (beyond
        the context, a page of another request's past) then changes the logits visibly."""
        self.groups, self.group_of_layer = plan_groups(requests)
        self.page_size = page_size
        self.num_pages = num_pages
        self.poison = poison
        self.layer_caches: Dict[int, LayerCache] = {}
        self._buffers = []
        for gi, g in enumerate(self.groups):
            r = g.request
            buf = torch.full((len(g.layers), 2, num_pages, r.num_kv_heads, page_size, r.head_dim),
                             POISON if poison else 0.0, dtype=dtype, device=device)
            self._buffers.append(buf)
            for li, layer in enumerate(g.layers):
                self.layer_caches[layer] = LayerCache(group=gi, k=buf[li, 0], v=buf[li, 1],
                                                      page_size=page_size)
        self.state_layers: List[int] = []
        for layer, req in enumerate(requests):
            if isinstance(req, FixedStateRequest):
                st = torch.zeros((num_state_slots,) + tuple(req.shape), dtype=torch.float32,
                                 device=device)
                self.layer_caches[layer] = LayerCache(state=st, page_size=page_size)
                self.state_layers.append(layer)
            elif req is None:
                self.layer_caches[layer] = LayerCache(page_size=page_size)

    @property
    def group_windows(self) -> List[Optional[int]]:
        return [g.request.window for g in self.groups]

    def clear_state_slots(self, slots: Sequence[int]) -> None:
        """Zero the state records of freshly taken slots (before their first step)."""
        if not slots or not self.state_layers:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.layer_caches[self.state_layers[0]].state.device)
        for layer in self.state_layers:
            self.layer_caches[layer].state.index_fill_(0, idx, 0.0)

    def snapshot_state(self, slots: Sequence[int]) -> List[torch.Tensor]:
        """Copies of the state records of ``slots``, one tensor per state layer."""
        if not self.state_layers or not slots:
            return []
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.layer_caches[self.state_layers[0]].state.device)
        return [self.layer_caches[layer].state.index_select(0, idx) for layer in self.state_layers]

    def restore_state(self, slots: Sequence[int], saved: List[torch.Tensor]) -> None:
        if not saved:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=saved[0].device)
        for layer, copy in zip(self.state_layers, saved):
            self.layer_caches[layer].state.index_copy_(0, idx, copy)

    def poison_pages(self, group: int, pages: Sequence[int]) -> None:
        """Debugging mode: pages that went back to the free list hold ``POISON`` again."""
        if not self.poison or not pages:
            return
        buf = self._buffers[group]
        idx = torch.tensor(list(pages), dtype=torch.long, device=buf.device)
        buf.index_fill_(2, idx, POISON)

    def nbytes(self) -> int:
        n = sum(b.numel() * b.element_size() for b in self._buffers)
        return n + sum(self.layer_caches[l].state.numel() * 4 for l in self.state_layers)

"""The step function: runs a batch of (request, its next tokens) from the cache.

``ModelRunner`` owns the model, the device cache and the cache manager.  Its
``step(entries)`` takes any mix of prompt portions and single decoded tokens, cut
anywhere, runs exactly those tokens as one batch against what earlier steps left
in the cache, and returns float32 logits at the wanted places.  Generation
(``LLMEngine``), trace replay (``bin/trace_run``) and the benchmark all drive this
one function.  Reference analogue: the packing and forward part of
``LLMEngine.step`` (servelab/engine/engine.py:183-218).
"""

from __future__ import annotations

import gc
import weakref
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, pages_from_memory, plan_groups
from ..config.engine import CacheConfig
from ..config.registry import load_config
from ..models.causal_lm import CausalLM
from ..ops import kernels as K
from ..parts import BuildEnv
from ..weights.source import FolderSource, WeightSource
from .batch import BatchEntry, StepContext

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class ModelRunner:
    def __init__(self, config, weights: WeightSource, dtype: str = "bfloat16",
                 cache_config: Optional[CacheConfig] = None, max_num_seqs: int = 64,
                 device: str = "cuda:0", cuda_graphs: bool = False,
                 max_model_len: Optional[int] = None):
        K.require_cuda()
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        self.config = config
        self.device = device
        self.dtype = _DTYPES[dtype]
        cache_config = cache_config or CacheConfig()
        self.page_size = cache_config.block_size
        self.spec = config.to_model_spec()
        torch.cuda.set_device(device)
        env = BuildEnv(device=device, dtype=self.dtype, page_size=self.page_size)
        self.model = CausalLM(self.spec, env)
        with torch.no_grad():
            self.model.load(weights)
        requests = self.model.cache_requests()
        groups, _ = plan_groups(requests)
        num_pages = cache_config.num_blocks
        if num_pages is None:
            torch.cuda.synchronize()
            free_bytes = torch.cuda.mem_get_info()[0]
            num_pages = pages_from_memory(groups, self.page_size, self.dtype, free_bytes,
                                          cache_config.gpu_memory_utilization)
        self.num_pages = num_pages
        self.storage = CacheStorage(requests, num_pages, self.page_size, max_num_seqs, self.dtype,
                                    device, poison=cache_config.poison_cache)
        self.cache = CacheManager(self.storage.group_windows, num_pages, self.page_size,
                                  max_num_seqs, reserve_pages=cache_config.reserve_blocks)
        if cache_config.poison_cache:
            storage = self.storage             # (the pools must not keep the runner alive)
            for g, pool in enumerate(self.cache.pools):
                pool.on_free = (lambda pages, g=g, storage=storage: storage.poison_pages(g, pages))
        self.num_groups = len(self.storage.groups)
        self.max_model_len = min(max_model_len or self.spec.max_position_embeddings,
                                 self.spec.max_position_embeddings, num_pages * self.page_size)
        # decode-only steps replay a CUDA graph per batch size (fixed addresses,
        # block tables padded to the longest request the engine admits)
        self.cuda_graphs = cuda_graphs
        self.max_graph_batch = max_num_seqs
        self._graphs = {}
        self._graph_pool = None
        # every part says itself whether its forward only launches kernels on the step's
        # device buffers (``graph_safe``); a mixer with state of its own does so too, by
        # indexing its state with ``ctx.state_slots`` on the device
        self._graph_safe = all(
            getattr(b, "graph_safe", False)
            for b in list(self.model.blocks) + [self.model.embedding_position, self.model.final_norm])
        self.graph_replays = 0
        # Steps with prompt portions replay graphs too, captured for padded sizes (tokens,
        # requests, wanted rows rounded up; ``StepContext.pack(pad=...)``): a layer costs the
        # host 0.2 ms of launches when run eagerly, which binds the steps of a small model.
        # A shape is captured when it comes up the second time; at most
        # ``max_portion_graphs`` are kept (least recently used first out).
        self.portion_graphs = True        # (only with ``cuda_graphs``)
        self.max_portion_graph_tokens = 2048
        self.max_portion_graphs = 24
        self.portion_graph_after = 2      # times a shape is asked for before it is captured
        self._portion_graphs = {}         # padded sizes -> (graph, context, logits)
        self._portion_seen = {}           # padded sizes -> times asked for
        self.portion_graph_replays = 0
        self._table_rows = {}             # (request, group) -> (stamp, block table as int32 array)
        # through a weak reference: the cache manager must not keep the runner alive in a
        # cycle, or a dropped engine (its graphs, its memory pool) would be destroyed only when
        # the garbage collector runs, which may be in the middle of another engine's capture
        me = weakref.ref(self)
        self.cache.release_listeners.append(lambda rid: me() is not None and me()._forget_table_rows(rid))
        self.graph_kernel_launches = {}   # batch size -> this package's kernels per replay

    @classmethod
    def from_folder(cls, folder: str, **kw) -> "ModelRunner":
        return cls(load_config(folder), FolderSource(folder), **kw)

    # ---------------------------------------------------------------- step
    def entry(self, request_id: str, tokens: Sequence[int], start: int,
              want: Sequence[int] = ()) -> BatchEntry:
        """A batch entry with the request's current block tables and state slot."""
        stamps = [self.cache.table_stamp(request_id, g) for g in range(self.num_groups)]
        return BatchEntry(tokens=tokens, start=start, want=want,
                          block_tables=[self._table_row(request_id, g, stamps[g])
                                        for g in range(self.num_groups)],
                          state_slot=self.cache.state_slot(request_id), table_stamps=stamps)

    def _table_row(self, request_id: str, group: int, stamp: int) -> np.ndarray:
        """The request's block table as an int32 array, converted anew only when the table
        has changed (its stamp): packing a step then copies arrays, not Python lists."""
        key = (request_id, group)
        hit = self._table_rows.get(key)
        if hit is None or hit[0] != stamp:
            hit = (stamp, np.asarray(self.cache.block_table(request_id, group), dtype=np.int32))
            self._table_rows[key] = hit
        return hit[1]

    def _forget_table_rows(self, request_id: str) -> None:
        for g in range(self.num_groups):
            self._table_rows.pop((request_id, g), None)

    def check_tokens(self, tokens: Sequence[int]) -> None:
        v = self.spec.vocab_size
        for t in tokens:
            if not 0 <= t < v:
                raise ValueError(f"token id {t} outside the vocabulary [0, {v})")

    def replays_graph(self, num_entries: int) -> bool:
        """Whether a step of ``num_entries`` single tokens, all wanting logits, replays a
        captured graph."""
        return self.cuda_graphs and self._graph_safe and 0 < num_entries <= self.max_graph_batch

    @torch.no_grad()
    def step(self, entries: List[BatchEntry],
             token_ids_from: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits [wanted, vocab] float32 (on the device) of this batch.
        ``token_ids_from`` (only for steps that replay a graph): int32 token ids on the
        device, one per entry, that replace the entries' own tokens; they may still be
        being computed by kernels queued earlier on the stream."""
        self.storage.clear_state_slots(self.cache.slots.drain_to_clear())
        if (self.replays_graph(len(entries))
                and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)):
            return self._step_graph(entries, token_ids_from)
        if token_ids_from is not None:
            raise ValueError("token ids from the device need a step that replays a graph")
        if self.cuda_graphs and self.portion_graphs and self._graph_safe and not self.storage.state_layers:
            pad = self._portion_pad(entries)
            if pad is not None:
                hit = self._portion_graphs.get(pad)
                seen = self._portion_seen[pad] = self._portion_seen.get(pad, 0) + 1
                if hit is not None or seen >= self.portion_graph_after:
                    return self._step_portion_graph(entries, pad)
        ctx = StepContext.pack(entries, self.num_groups, self.device)
        if ctx.num_tokens == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.forward(ctx, self.storage.layer_caches)

    @staticmethod
    def _round_up(n: int, steps) -> int:
        for limit, unit in steps:
            if n <= limit:
                return -(-n // unit) * unit
        return n

    def _portion_pad(self, entries: List[BatchEntry]):
        """(tokens, requests, wanted rows) a step is padded to, or None if it runs eagerly."""
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        if T == 0 or T > self.max_portion_graph_tokens:
            return None
        Tp = self._round_up(T, ((64, 16), (512, 64), (self.max_portion_graph_tokens, 256)))
        Sp = 1 << len(entries).bit_length()                 # a power of two above the requests
        Rp = 1 << (R - 1).bit_length() if R else 0
        return Tp, Sp, Rp

    def _step_portion_graph(self, entries: List[BatchEntry], pad) -> torch.Tensor:
        """A step of any composition through the graph captured for its padded sizes.  The
        returned logits live in the graph's memory until its next replay."""
        width = -(-self.max_model_len // self.page_size)
        R = sum(len(e.want) for e in entries)
        hit = self._portion_graphs.pop(pad, None)
        if hit is None:
            ctx = StepContext.pack(entries, self.num_groups, self.device, min_table_width=width, pad=pad)
            self.model.forward(ctx, self.storage.layer_caches)        # builds libraries, warms caches
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    logits = self.model.forward(ctx, self.storage.layer_caches)
            finally:
                if gc_was_on:
                    gc.enable()
            hit = (graph, ctx, logits)
            while len(self._portion_graphs) >= self.max_portion_graphs:
                self._portion_graphs.pop(next(iter(self._portion_graphs)))
        graph, ctx, logits = hit
        self._portion_graphs[pad] = hit                     # (most recently used last)
        StepContext.pack(entries, self.num_groups, self.device, min_table_width=width, into=ctx, pad=pad)
        graph.replay()
        self.portion_graph_replays += 1
        return logits[:R]

    def _step_graph(self, entries: List[BatchEntry],
                    token_ids_from: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A step of single decoded tokens, all wanting logits: replay the graph
        captured for this batch size.  The returned logits live in the graph's
        memory and are overwritten by the next replay of the same size."""
        B = len(entries)
        width = -(-self.max_model_len // self.page_size)
        hit = self._graphs.get(B)
        if hit is None:
            ctx = StepContext.pack(entries, self.num_groups, self.device, min_table_width=width)
            ctx.split_hint_len = self.max_model_len     # launch shapes must not depend on the step
            # the warm-up outside capture runs the step once and the first replay runs it again:
            # keys and values land in the same slots both times, but a mixer's own state would
            # advance twice, so the state of the step's slots is put back after the warm-up
            saved = self.storage.snapshot_state(ctx.state_slot_ids)
            self.model.forward(ctx, self.storage.layer_caches)
            self.storage.restore_state(ctx.state_slot_ids, saved)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = K.launch_count
            # objects that own device memory or graphs must not be destroyed while the stream is
            # capturing (their CUDA calls would invalidate the capture): collect what is garbage
            # now, and keep the collector off until the capture has ended
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    logits = self.model.forward(ctx, self.storage.layer_caches)
            finally:
                if gc_was_on:
                    gc.enable()
            self.graph_kernel_launches[B] = K.launch_count - before
            hit = self._graphs[B] = (graph, ctx, logits)
        graph, ctx, logits = hit
        StepContext.pack(entries, self.num_groups, self.device, min_table_width=width, into=ctx)
        if token_ids_from is not None:
            ctx.token_ids.copy_(token_ids_from)
        graph.replay()
        self.graph_replays += 1
        return logits

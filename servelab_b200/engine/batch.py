"""The batch of one step: what runs, described once on the host and copied to the
device in a single transfer.

A step is a list of entries, one per request taking part: its next tokens (a
portion of its prompt or a single decoded token), the position of the first of
them, which of them want logits, its block table in every cache group and its
state slot.  ``StepContext.pack`` flattens the entries along one token axis and
lays all integer arrays out in one pinned host buffer:

  token_ids[T] positions[T] seq_of_token[T] cu_q[S+1] ctx_len[S] state_slots[S]
  logit_rows[R] block_tables[group][S, max_pages] ...

Parts read these through the context (see ``parts/base.py``).  Reference
analogue: the per-step Python lists and ``SeqMeta(offset, q_len, ctx_len,
block_table)`` built by the engine (servelab/engine/engine.py:176-215); the flat
``slots`` array is replaced by a block-table lookup on the device.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class BatchEntry:
    """One request's share of a step."""
    tokens: Sequence[int]
    start: int                                   # position of tokens[0]
    want: Sequence[int] = ()                     # indices into ``tokens`` whose logits are wanted
    block_tables: Sequence[Sequence[int]] = ()   # one table per cache group (lists or int32 arrays)
    state_slot: int = 0
    table_stamps: Sequence[int] = ()             # per group: changes iff the table changed
                                                 # (empty: unknown, always copy)


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepContext:
    """Device-side view of a step plus a few host-side facts about it."""

    def __init__(self, device: str):
        self.device = device
        self.num_tokens = 0
        self.num_seqs = 0
        self.num_logit_rows = 0
        self.q_lens: List[int] = []
        self.state_slot_ids: List[int] = []
        self.ctx_lens: List[int] = []
        self.decode_only = False
        self.max_ctx_len = 0
        self.split_hint_len = 0       # context length the decode kernel sizes its splits for
        self.token_ids = self.positions = self.seq_of_token = None
        self.cu_q = self.ctx_len = self.state_slots = self.logit_rows = None
        self.block_tables: List[torch.Tensor] = []
        self._host2 = None            # two pinned buffers of a context that is overwritten in place
        self._flip = 0
        self._stamps = None
        self._tiles: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor, int]] = {}
        self.scratch: Dict[str, torch.Tensor] = {}   # per-step scratch parts may share

    # ------------------------------------------------------------ packing
    @classmethod
    def pack(cls, entries: Sequence[BatchEntry], num_groups: int, device: str,
             min_table_width: int = 1, into: Optional["StepContext"] = None,
             pad: Optional[Tuple[int, int, int]] = None, _host_only: bool = False) -> "StepContext":
        """``into``: a context packed earlier for the same number of requests,
        tokens, wanted rows and table widths; its device buffer is overwritten in
        place (a captured CUDA graph keeps reading the same addresses).
        ``pad`` = (tokens, requests, wanted rows): the step is laid out for these sizes,
        which must exceed what the entries hold in requests and not fall short in the
        others.  Padding tokens belong to the last, empty request (no pages: nothing is
        written to the cache, no attention tile covers them); padding rows repeat row 0."""
        if pad is not None:
            return cls._pack_padded(entries, num_groups, device, min_table_width, into, pad)
        ctx = cls(device)
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        want_rows: List[int] = []
        off = 0
        for e, n in zip(entries, q_lens):
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted index {w} outside the entry's {n} tokens")
                want_rows.append(off + w)
            off += n
        R = len(want_rows)
        widths = []
        for g in range(num_groups):
            widths.append(max([min_table_width] + [len(e.block_tables[g]) for e in entries]))

        sizes = [T, T, T, S + 1, S, S, R] + [S * w for w in widths]
        offsets, total = [], 0
        for n in sizes:
            offsets.append(total)
            total += _align4(max(n, 1))
        reuse = into is not None and into._dev.numel() == total and \
            into._layout == (T, S, R, tuple(widths)) and into._host2 is not None
        if reuse:
            # the context of a captured graph keeps two pinned buffers and alternates, so a
            # buffer is rewritten only after the copy issued two steps earlier; table rows
            # whose stamp is unchanged since that buffer's last use are left as they are
            into._flip ^= 1
            host = into._host2[into._flip]
            stamps = into._stamps[into._flip]
            hv = host.numpy()
        else:
            host = torch.empty(total, dtype=torch.int32,
                               pin_memory=torch.cuda.is_available() and not _host_only)
            stamps = None
            hv = host.numpy()
            hv[:] = 0
        o_tok, o_pos, o_seq, o_cu, o_ctx, o_slot, o_rows = offsets[:7]
        # every array in one assignment (a step of 64 requests would otherwise pay for several
        # hundred small ones)
        q = np.asarray(q_lens, dtype=np.int32)
        starts = np.asarray([e.start for e in entries], dtype=np.int32)
        cu = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q, out=cu[1:])
        if T == S and all(n == 1 for n in q_lens):
            hv[o_tok:o_tok + T] = [e.tokens[0] for e in entries]
            hv[o_pos:o_pos + T] = starts
            hv[o_seq:o_seq + T] = np.arange(S, dtype=np.int32)
        else:
            flat: List[int] = []
            for e in entries:
                flat.extend(e.tokens)
            hv[o_tok:o_tok + T] = flat
            hv[o_seq:o_seq + T] = np.repeat(np.arange(S, dtype=np.int32), q)
            # position of token j of request s: start_s + (j - cu_s)
            hv[o_pos:o_pos + T] = np.arange(T, dtype=np.int32) - np.repeat(cu[:-1] - starts, q)
        hv[o_cu:o_cu + S + 1] = cu
        hv[o_ctx:o_ctx + S] = starts + q
        hv[o_slot:o_slot + S] = [e.state_slot for e in entries]
        hv[o_rows:o_rows + R] = want_rows
        for g, w in enumerate(widths):
            base = offsets[7 + g]
            tab = hv[base:base + S * w].reshape(S, w) if S else None
            if tab is None:
                continue
            if stamps is None:
                tab[:] = -1
            for s, e in enumerate(entries):
                row = e.block_tables[g]
                if stamps is not None:
                    stamp = e.table_stamps[g] if e.table_stamps else None
                    if stamp is not None and stamps[g][s] == stamp:
                        continue
                    stamps[g][s] = stamp
                    tab[s, len(row):] = -1
                tab[s, :len(row)] = row
        if into is not None:
            if into._dev.numel() != total or into._layout != (T, S, R, tuple(widths)):
                raise ValueError("batch does not have the shape of the context to overwrite")
            if into._host2 is None:
                # first overwrite: set up the two alternating pinned buffers
                other = torch.empty(total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
                other.numpy()[:] = hv
                into._host2 = [host, other]
                into._flip = 0
                fresh = [[e.table_stamps[g] if e.table_stamps else None for e in entries]
                         for g in range(num_groups)]
                into._stamps = [fresh, [list(x) for x in fresh]]
            into._dev.copy_(host, non_blocking=True)
            into._host = host
            into.q_lens, into.state_slot_ids = q_lens, [e.state_slot for e in entries]
            into.ctx_lens = [e.start + n for e, n in zip(entries, q_lens)]
            into.max_ctx_len = max(into.ctx_lens) if into.ctx_lens else 0
            return into
        if _host_only:                                # (the padded form lays the arrays out anew)
            ctx._host = host
            ctx._widths = widths
            ctx.q_lens = q_lens
            ctx.state_slot_ids = [e.state_slot for e in entries]
            ctx.ctx_lens = [e.start + n for e, n in zip(entries, q_lens)]
            ctx.max_ctx_len = max(ctx.ctx_lens) if ctx.ctx_lens else 0
            return ctx
        dev = host.to(device, non_blocking=True)
        ctx._host = host                              # keep the pinned buffer alive
        ctx._dev = dev
        ctx._layout = (T, S, R, tuple(widths))

        def view(o, n):
            return dev[o:o + n]
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view(o_tok, T), view(o_pos, T), view(o_seq, T)
        ctx.cu_q, ctx.ctx_len = view(o_cu, S + 1), view(o_ctx, S)
        ctx.state_slots, ctx.logit_rows = view(o_slot, S), view(o_rows, R)
        ctx.block_tables = [dev[offsets[7 + g]:offsets[7 + g] + S * w].view(S, w)
                            for g, w in enumerate(widths)]
        ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows = T, S, R
        ctx.q_lens = q_lens
        ctx.state_slot_ids = [e.state_slot for e in entries]
        ctx.ctx_lens = [e.start + n for e, n in zip(entries, q_lens)]
        ctx.max_ctx_len = max(ctx.ctx_lens) if ctx.ctx_lens else 0
        ctx.split_hint_len = ctx.max_ctx_len
        ctx.decode_only = S > 0 and all(n == 1 for n in q_lens)
        return ctx

    @classmethod
    def _pack_padded(cls, entries, num_groups, device, min_table_width, into, pad):
        """The padded form of ``pack``: empty entries fill the requests, the last of them
        takes the padding tokens in the flat arrays only (its q_len stays 0, so no kernel
        that walks requests or tiles sees them)."""
        Tp, Sp, Rp = pad
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        if Sp <= S or Tp < T or Rp < R:
            raise ValueError("padding sizes must exceed the requests and hold the tokens and rows")
        empty_tables = [np.empty(0, dtype=np.int32)] * num_groups
        filler = [BatchEntry(tokens=(), start=0, want=(), block_tables=empty_tables, state_slot=0,
                             table_stamps=[-1] * num_groups) for _ in range(Sp - S)]
        inner = cls.pack(list(entries) + filler, num_groups, device, min_table_width, _host_only=True)
        # the inner layout has T tokens and R rows; rebuild it with the padded sizes
        widths = inner._widths
        sizes = [Tp, Tp, Tp, Sp + 1, Sp, Sp, Rp] + [Sp * w for w in widths]
        offsets, total = [], 0
        for n in sizes:
            offsets.append(total)
            total += _align4(max(n, 1))
        src = inner._host.numpy()
        in_sizes = [T, T, T, Sp + 1, Sp, Sp, R] + [Sp * w for w in widths]
        in_off, acc = [], 0
        for n in in_sizes:
            in_off.append(acc)
            acc += _align4(max(n, 1))
        reuse = into is not None
        if reuse:
            if into._layout != ("padded", Tp, Sp, Rp, tuple(widths)):
                raise ValueError("batch does not have the shape of the context to overwrite")
            into._flip ^= 1
            host = into._host2[into._flip]
        else:
            host = torch.empty(total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        hv = host.numpy()
        hv[:] = 0
        for i, (o, n) in enumerate(zip(in_off, in_sizes)):
            hv[offsets[i]:offsets[i] + n] = src[o:o + n]
        hv[offsets[2] + T:offsets[2] + Tp] = Sp - 1           # padding tokens: the last, empty request
        ctx = into if reuse else cls(device)
        if reuse:
            ctx._dev.copy_(host, non_blocking=True)
        else:
            other = torch.empty(total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
            ctx._host2, ctx._flip = [host, other], 0
            ctx._dev = host.to(device, non_blocking=True)
            ctx._layout = ("padded", Tp, Sp, Rp, tuple(widths))
            dev = ctx._dev

            def view(k, n):
                return dev[offsets[k]:offsets[k] + n]
            ctx.token_ids, ctx.positions, ctx.seq_of_token = view(0, Tp), view(1, Tp), view(2, Tp)
            ctx.cu_q, ctx.ctx_len = view(3, Sp + 1), view(4, Sp)
            ctx.state_slots, ctx.logit_rows = view(5, Sp), view(6, Rp)
            ctx.block_tables = [view(7 + g, Sp * w).view(Sp, w) for g, w in enumerate(widths)]
            ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows = Tp, Sp, Rp
            ctx._padded_tiles = {}
        ctx._host = host
        ctx.q_lens, ctx.state_slot_ids = inner.q_lens, inner.state_slot_ids
        ctx.ctx_lens, ctx.max_ctx_len = inner.ctx_lens, inner.max_ctx_len
        ctx.split_hint_len = inner.max_ctx_len
        ctx.decode_only = False
        ctx.real_sizes = (T, S, R)
        for key in ctx._padded_tiles:                       # the work lists of the kernels that asked
            ctx._refresh_tiles(key)
        return ctx

    def _tile_bound(self, group_size: int, rows_per_tile: int) -> int:
        return -(-self.num_tokens * group_size // rows_per_tile) + self.num_seqs

    def _refresh_tiles(self, key):
        group_size, rows_per_tile = key
        dev, hosts, flip = self._padded_tiles[key]
        bound = dev.numel() // 2
        rows = np.asarray(self.q_lens, dtype=np.int64) * group_size
        per_seq = -(-rows // rows_per_tile)
        first = np.cumsum(per_seq) - per_seq
        seqs = np.repeat(np.arange(len(self.q_lens)), per_seq)
        n = len(seqs)
        host = hosts[flip]
        hv = host.numpy()
        hv[:bound] = self.num_seqs - 1                      # tiles beyond the step's: the empty request
        hv[bound:] = 0
        hv[:n] = seqs
        hv[bound:bound + n] = (np.arange(n) - np.repeat(first, per_seq)) * rows_per_tile
        dev.copy_(host, non_blocking=True)
        self._padded_tiles[key] = (dev, hosts, flip ^ 1)

    # ------------------------------------------------- attention work list
    def attention_tiles(self, group_size: int, rows_per_tile: int):
        """Tiles of ``rows_per_tile`` query rows over each request's q_len *
        group_size flattened rows: (tile_seq, tile_row0, count) on the device."""
        key = (group_size, rows_per_tile)
        padded = getattr(self, "_padded_tiles", None)
        if padded is not None:
            # a padded context (it may be replayed in a graph): lists of a fixed length at fixed
            # addresses, rewritten whenever the context is packed anew
            if key not in padded:
                bound = self._tile_bound(group_size, rows_per_tile)
                pin = torch.cuda.is_available()
                hosts = [torch.empty(2 * bound, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
                padded[key] = (torch.empty(2 * bound, dtype=torch.int32, device=self.device), hosts, 0)
                self._refresh_tiles(key)
            dev = padded[key][0]
            bound = dev.numel() // 2
            return dev[:bound], dev[bound:], bound
        hit = self._tiles.get(key)
        if hit is None:
            rows = np.asarray(self.q_lens, dtype=np.int64) * group_size
            per_seq = -(-rows // rows_per_tile)                          # tiles of each request
            first = np.cumsum(per_seq) - per_seq                         # index of its first tile
            seqs = np.repeat(np.arange(len(self.q_lens)), per_seq)
            row0s = (np.arange(int(per_seq.sum())) - np.repeat(first, per_seq)) * rows_per_tile
            n_tiles = len(seqs)
            host = torch.from_numpy(np.concatenate([seqs, row0s]).astype(np.int32))
            if torch.cuda.is_available():
                host = host.pin_memory()
            dev = host.to(self.device, non_blocking=True)
            hit = (dev[:n_tiles], dev[n_tiles:], n_tiles)
            self._tiles[key] = hit
            self.scratch[f"_tiles_host_{key}"] = host
        return hit

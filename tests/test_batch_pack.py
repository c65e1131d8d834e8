"""``StepContext.pack`` on the CPU: the flat arrays of a step against a straightforward
construction, for fresh contexts and for contexts overwritten in place (the path a replayed
CUDA graph takes), with random mixes of prompt portions and single tokens, several cache
groups, windows (-1 entries) and tables that change or stay between steps."""

import random

import pytest
import torch

from servelab_b200.engine.batch import BatchEntry, StepContext


def expected(entries, num_groups, min_width):
    tok, pos, seq, cu, ctx_len, slots, rows = [], [], [], [0], [], [], []
    for s, e in enumerate(entries):
        n = len(e.tokens)
        rows += [len(tok) + w for w in e.want]
        tok += list(e.tokens)
        pos += list(range(e.start, e.start + n))
        seq += [s] * n
        cu.append(len(tok))
        ctx_len.append(e.start + n)
        slots.append(e.state_slot)
    tables = []
    for g in range(num_groups):
        w = max([min_width] + [len(e.block_tables[g]) for e in entries])
        tables.append([list(e.block_tables[g]) + [-1] * (w - len(e.block_tables[g])) for e in entries])
    return tok, pos, seq, cu, ctx_len, slots, rows, tables


def check(ctx, entries, num_groups, min_width):
    tok, pos, seq, cu, ctx_len, slots, rows, tables = expected(entries, num_groups, min_width)
    assert ctx.token_ids.tolist() == tok
    assert ctx.positions.tolist() == pos
    assert ctx.seq_of_token.tolist() == seq
    assert ctx.cu_q.tolist() == cu
    assert ctx.ctx_len.tolist() == ctx_len
    assert ctx.state_slots.tolist() == slots
    assert ctx.logit_rows.tolist() == rows
    assert [t.tolist() for t in ctx.block_tables] == tables
    assert ctx.num_tokens == len(tok) and ctx.num_seqs == len(entries) and ctx.num_logit_rows == len(rows)
    assert ctx.q_lens == [len(e.tokens) for e in entries]
    assert ctx.ctx_lens == ctx_len and ctx.max_ctx_len == max(ctx_len)
    assert ctx.state_slot_ids == slots
    assert ctx.decode_only == all(len(e.tokens) == 1 for e in entries)


def random_entries(rng, num_groups, page, decode_only=False, count=None):
    entries = []
    for s in range(count or rng.randint(1, 9)):
        n = 1 if decode_only or rng.random() < 0.4 else rng.randint(2, 70)
        start = rng.randint(0, 300)
        pages = -(-(start + n) // page)
        tables = []
        for g in range(num_groups):
            t = [rng.randint(0, 999) for _ in range(pages)]
            if g == 1:                                     # a windowed group: pages given back
                for i in range(max(0, pages - 3)):
                    t[i] = -1
            tables.append(t)
        want = sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))
        entries.append(BatchEntry(tokens=[rng.randint(0, 5000) for _ in range(n)], start=start, want=want,
                                  block_tables=tables, state_slot=rng.randint(0, 63),
                                  table_stamps=[rng.randint(0, 1 << 30) for _ in range(num_groups)]))
    return entries


@pytest.mark.parametrize("seed", range(8))
def test_fresh_contexts(seed):
    rng = random.Random(seed)
    groups = 1 + seed % 2
    entries = random_entries(rng, groups, page=8)
    width = rng.choice([1, 5, 64])
    check(StepContext.pack(entries, groups, "cpu", min_table_width=width), entries, groups, width)


@pytest.mark.parametrize("seed", range(6))
def test_padded_contexts_fresh_and_overwritten(seed):
    """The padded form that graphs of steps with prompt portions replay: the step's own arrays first,
    then padding tokens that belong to the last, empty request (no page in its table, q_len 0),
    empty requests, rows that repeat row 0; work lists of attention tiles of a fixed length whose
    surplus entries name the empty request.  Overwritten in place three times with other steps."""
    rng = random.Random(100 + seed)
    groups = 1 + seed % 2
    width = 64
    ctx = None
    for _ in range(4):
        entries = random_entries(rng, groups, page=8, count=rng.randint(1, 6))
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        pad = (512, 8, 32)
        ctx = StepContext.pack(entries, groups, "cpu", min_table_width=width, pad=pad, into=ctx)
        tok, pos, seq, cu, ctx_len, slots, rows, tables = expected(entries, groups, width)
        S = len(entries)
        assert (ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows) == pad and ctx.real_sizes == (T, S, R)
        assert ctx.token_ids.tolist() == tok + [0] * (512 - T)
        assert ctx.positions.tolist() == pos + [0] * (512 - T)
        assert ctx.seq_of_token.tolist() == seq + [7] * (512 - T)
        assert ctx.cu_q.tolist() == cu + [T] * (8 - S)
        assert ctx.ctx_len.tolist() == ctx_len + [0] * (8 - S)
        assert ctx.logit_rows.tolist() == rows + [0] * (32 - R)
        for g in range(groups):
            got = ctx.block_tables[g].tolist()
            assert got[:S] == tables[g] and all(v == -1 for row in got[S:] for v in row)
        assert not ctx.decode_only and ctx.q_lens == [len(e.tokens) for e in entries] + [0] * (8 - S)
        for group_size, rows_per_tile in ((2, 16), (7, 128)):
            tile_seq, tile_row0, n = ctx.attention_tiles(group_size, rows_per_tile)
            assert n == -(-512 * group_size // rows_per_tile) + 8 and len(tile_seq) == n
            want = [(s, r0) for s, e in enumerate(entries)
                    for r0 in range(0, len(e.tokens) * group_size, rows_per_tile)]
            got = list(zip(tile_seq.tolist(), tile_row0.tolist()))
            assert got[:len(want)] == want and all(t == (7, 0) for t in got[len(want):])
    with pytest.raises(ValueError):
        StepContext.pack(entries, groups, "cpu", min_table_width=width, pad=(512, len(entries), 32))


def test_entries_without_stamps_and_empty_want():
    e = [BatchEntry(tokens=[4, 5, 6], start=2, want=(), block_tables=[[7]], state_slot=3),
         BatchEntry(tokens=[9], start=40, want=(0,), block_tables=[[1, 2, 3, 4, 5, 6]], state_slot=0)]
    check(StepContext.pack(e, 1, "cpu"), e, 1, 1)
    with pytest.raises(ValueError):
        StepContext.pack([BatchEntry(tokens=[1], start=0, want=(1,), block_tables=[[0]])], 1, "cpu")


@pytest.mark.parametrize("seed", range(4))
def test_contexts_overwritten_in_place(seed):
    """Steps of single tokens into the same context, as the replayed graph does: tables grow
    by a page now and then (new stamp), most rows keep their stamp; a request is replaced by
    another one with a shorter table (the tail of its row must turn to -1)."""
    rng = random.Random(100 + seed)
    groups, page, width, B = 2, 4, 40, 6
    state = []
    for s in range(B):
        start = rng.randint(0, 60)
        state.append({"start": start, "slot": s, "stamp": [s * 1000, s * 1000 + 500],
                      "tables": [[rng.randint(0, 999) for _ in range(start // page + 1)] for _ in range(groups)]})

    def entries():
        return [BatchEntry(tokens=[rng.randint(0, 5000)], start=r["start"], want=(0,),
                           block_tables=[list(t) for t in r["tables"]], state_slot=r["slot"],
                           table_stamps=list(r["stamp"])) for r in state]
    ctx = StepContext.pack(entries(), groups, "cpu", min_table_width=width)
    for step in range(40):
        for r in state:
            r["start"] += 1
            if r["start"] // page + 1 > len(r["tables"][0]):
                for g in range(groups):
                    r["tables"][g].append(rng.randint(0, 999))
                    r["stamp"][g] += 1
        if step == 17:                                     # another request takes row 2
            state[2] = {"start": 3, "slot": 9, "stamp": [77777, 88888],
                        "tables": [[5], [6]]}
        e = entries()
        out = StepContext.pack(e, groups, "cpu", min_table_width=width, into=ctx)
        assert out is ctx
        check(ctx, e, groups, width)
    with pytest.raises(ValueError):
        StepContext.pack(entries()[:-1], groups, "cpu", min_table_width=width, into=ctx)


@pytest.mark.parametrize("q_lens,group,rows", [([1, 1, 1], 7, 64), ([37, 1, 300, 2], 7, 64), ([5], 1, 16),
                                               ([64, 65, 128], 2, 128), ([1], 20, 8)])
def test_attention_tiles(q_lens, group, rows):
    ctx = StepContext("cpu")
    ctx.q_lens = q_lens
    tile_seq, tile_row0, n = ctx.attention_tiles(group, rows)
    want = [(s, r0) for s, q in enumerate(q_lens) for r0 in range(0, q * group, rows)]
    assert n == len(want)
    assert list(zip(tile_seq.tolist(), tile_row0.tolist())) == want
    assert tile_seq.dtype == torch.int32 and tile_row0.dtype == torch.int32
    assert ctx.attention_tiles(group, rows)[0] is tile_seq            # computed once per step


def test_entries_follow_the_cache_manager_through_growth_windows_and_reuse_of_ids():
    """``ModelRunner.entry`` hands out block tables as arrays that it converts only when a
    table's stamp changes: after every change of the manager (growth, a window passing pages,
    release and a new request under the old id) they must equal the manager's own tables."""
    from servelab_b200.cache import CacheManager
    from servelab_b200.engine.runner import ModelRunner
    runner = ModelRunner.__new__(ModelRunner)                 # the host side only: no model, no device
    runner.cache = CacheManager([None, 12], 64, 4, 8)         # a full group and a windowed one
    runner.num_groups = 2
    runner._table_rows = {}
    runner.cache.release_listeners.append(runner._forget_table_rows)
    rng = random.Random(5)
    live = {}

    def check_all():
        for rid, n in live.items():
            e = runner.entry(rid, [1], n - 1, (0,))
            for g in range(2):
                assert list(e.block_tables[g]) == runner.cache.block_table(rid, g), (rid, g)
                assert e.block_tables[g].dtype.name == "int32"
            assert e.table_stamps == [runner.cache.table_stamp(rid, g) for g in range(2)]
            assert e.state_slot == runner.cache.state_slot(rid)
    for step in range(300):
        rid = f"r{rng.randint(0, 4)}"
        if rid not in live:
            if runner.cache.open(rid):
                if runner.cache.ensure(rid, 1):
                    live[rid] = 1
                else:
                    runner.cache.release(rid)
        elif rng.random() < 0.1:
            runner.cache.release(rid)
            del live[rid]
        else:
            n = live[rid] + rng.randint(1, 9)
            if runner.cache.ensure(rid, n):
                live[rid] = n
                runner.cache.trim(rid, n)
        check_all()
        # rows of requests that gave everything back are dropped at once
        assert {rid for rid, _ in runner._table_rows} <= set(live)
    runner.cache.check_invariants()

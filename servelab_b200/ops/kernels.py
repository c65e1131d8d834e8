"""Python entry points of the CUDA kernels (thin: pointer passing, no math).

Every function launches on torch's current CUDA stream and returns without
synchronising.  Tensors must be CUDA tensors, contiguous in their last dimension.
The dtype of the activations selects the float32 or the bfloat16 instance.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from . import library as L

_F32, _BF16 = torch.float32, torch.bfloat16


launch_count = 0       # launches of this package's kernels (library GEMMs not included)


class SplitSum:
    """A [M, N] result that exists as float32 partial sums ``parts`` [splits, M, N]
    of a matrix product split along K (plus an optional float32 ``bias`` [N] still
    to be added).  Kernels that consume it add the parts in order, so no separate
    reduction is launched; ``materialize()`` produces the plain tensor."""

    accept_flag = "accepts_split_sum"

    def __init__(self, parts: torch.Tensor, bias: Optional[torch.Tensor], dtype: torch.dtype):
        self.parts, self.bias, self.dtype = parts, bias, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]

    def materialize(self) -> torch.Tensor:
        S, M, N = self.parts.shape
        out = torch.empty((M, N), dtype=self.dtype, device=self.parts.device)
        L.check(L.core().slb_split_sum(self.parts.data_ptr(), out.data_ptr(), out.stride(0),
                                       _p(self.bias), 1 if self.dtype == _F32 else 0, M, N, S,
                                       _stream()), "split_sum")
        return out


class DeferredLinear:
    """A [M, N] result x . w^T (+ bias) whose product has not been launched: the consumer
    (a norm that takes it) launches the product with its own work in the product's epilogue
    (``gemm_tc_resid_norm``).  ``materialize()`` runs the plain product."""

    accept_flag = "accepts_deferred_linear"

    def __init__(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]):
        self.x, self.w, self.bias = x, w, bias

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    def materialize(self) -> torch.Tensor:
        return gemm_tc_cluster(self.x, self.w, None, self.bias)


class ScaledRows:
    """Normed rows [M, h] without their factor 1 / rms: ``z`` = bfloat16(resid * weight) and
    ``sumsq`` [M, tiles], the sums of squares of resid per 128-column tile, as
    ``gemm_tc_resid_norm`` leaves them.  A matrix product that takes this form multiplies
    its result by 1 / sqrt(sum(sumsq) / h + eps) per token in its epilogue, which equals the
    product of the normed rows because the factor is one number a row.  ``materialize()``
    runs the norm kernel on the (already updated) residual stream."""

    accept_flag = "accepts_scaled_rows"

    def __init__(self, z, sumsq, eps: float, resid, weight):
        self.z, self.sumsq, self.eps, self.resid, self.weight = z, sumsq, eps, resid, weight

    @property
    def shape(self):
        return self.z.shape

    @property
    def dtype(self):
        return self.z.dtype

    @property
    def device(self):
        return self.z.device

    def materialize(self) -> torch.Tensor:
        out = torch.empty_like(self.z)
        add_rmsnorm(self.resid, None, self.weight, self.eps, out)
        return out


def plain_unless(part, value):
    """``value`` as a tensor unless it is an unfinished form (``SplitSum``, ``DeferredLinear``,
    ``ScaledRows``) and ``part`` says (by the form's flag) that it takes it."""
    flag = getattr(type(value), "accept_flag", None)
    if flag is not None and not getattr(part, flag, False):
        return value.materialize()
    return value


# the current stream's handle without building a torch.cuda.Stream object for it (a few
# microseconds a launch, which a step of a small model notices)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    global launch_count
    launch_count += 1
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _suffix(dt: torch.dtype) -> str:
    if dt == _F32:
        return "f32"
    if dt == _BF16:
        return "bf16"
    raise L.KernelError(f"kernels take float32 or bfloat16, not {dt}")


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise L.KernelsUnavailable(
            "servelab_b200 needs a CUDA device (sm_100a): there is no CPU path")
    L.core()


# ------------------------------------------------------------- elementwise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32; ids int32 [T], out float32 [T, h]."""
    fn = getattr(L.core(), "slb_embedding_" + _suffix(table.dtype))
    L.check(fn(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1],
               table.shape[0], float(scale), _stream()), "embedding")


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """In place on float32 logits [R, V]: times ``scale``, then with ``softcap`` > 0 bounded to
    softcap * tanh(x / softcap)."""
    if logits.dtype != _F32:
        raise L.KernelError("logit_transform: float32 logits only")
    L.check(L.core().slb_logit_transform(logits.data_ptr(), logits.stride(0), logits.shape[0],
                                         logits.shape[1], float(scale), float(softcap), _stream()),
            "logit_transform")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, row_map: Optional[torch.Tensor] = None) -> None:
    """resid += delta (in place, float32; skipped when ``row_map`` selects rows);
    out[r] = rmsnorm(resid[src(r)] (+ delta)) * weight."""
    rows = out.shape[0]
    if isinstance(delta, SplitSum):
        if out.dtype != _BF16:
            delta = delta.materialize()
        else:
            S, M, N = delta.parts.shape
            L.check(L.core().slb_add_rmsnorm_parts_bf16(
                resid.data_ptr(), delta.parts.data_ptr(), S, M * N, _p(delta.bias),
                weight.data_ptr(), out.data_ptr(), _p(row_map), rows, out.shape[1], float(eps),
                _stream()), "add_rmsnorm")
            return
    fn = getattr(L.core(), "slb_add_rmsnorm_" + _suffix(out.dtype))
    L.check(fn(resid.data_ptr(), _p(delta), weight.data_ptr(), out.data_ptr(), _p(row_map),
               rows, out.shape[1], float(eps), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t, i] = silu(gate_i) * up_i of row t of ``gate_up`` ([T, 2 I], I = out.shape[1]).
    ``block`` == 0: a row holds all gates, then all ups; ``block`` > 0: gates and ups
    alternate in runs of ``block`` elements."""
    fn = getattr(L.core(), "slb_swiglu_" + _suffix(out.dtype))
    L.check(fn(gate_up.data_ptr(), out.data_ptr(), out.shape[0], out.shape[1],
               gate_up.stride(0), out.stride(0), int(block), _stream()), "swiglu")


# ----------------------------------------------------- rotary + cache write
def _num_pages(cache: Optional[torch.Tensor]) -> int:
    """Pages in a layer's cache [pages, kv heads, page size, head size]: the kernels skip a
    block-table entry beyond it (and set a status word) instead of touching memory outside."""
    return 0 if cache is None else cache.shape[0]


def cache_write_status(reset: bool = False) -> int:
    """0 unless the q/k/v kernel met a block-table entry outside the cache (synchronises)."""
    return L.core().slb_cache_write_status(1 if reset else 0)


def generic_attention_status(reset: bool = False) -> int:
    """0 unless the plain attention kernel met a block-table entry outside the cache."""
    return L.core().slb_paged_attention_generic_status(1 if reset else 0)


def qkv_rope_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                   seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                   inv_freq: Optional[torch.Tensor], rotary_dim: int, q_out: torch.Tensor,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    if isinstance(qkv, SplitSum):
        if bias is not None and qkv.bias is not None:
            raise L.KernelError("qkv_rope_cache: two biases")
        if q_out.dtype != _BF16:
            qkv = qkv.materialize()
        else:
            S, M, N = qkv.parts.shape
            L.check(L.core().slb_qkv_rope_cache_parts_bf16(
                qkv.parts.data_ptr(), S, M * N, N, _p(bias if bias is not None else qkv.bias),
                positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                block_table.shape[1], page_size, _num_pages(k_cache), _p(inv_freq), rotary_dim,
                q_out.data_ptr(), q_out.stride(0), _p(k_cache), _p(v_cache), M, num_heads,
                num_kv_heads, head_dim, _stream()), "qkv_rope_cache")
            return
    fn = getattr(L.core(), "slb_qkv_rope_cache_" + _suffix(qkv.dtype))
    L.check(fn(qkv.data_ptr(), qkv.stride(0), _p(bias), positions.data_ptr(),
               seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
               _num_pages(k_cache), _p(inv_freq), rotary_dim, q_out.data_ptr(), q_out.stride(0), _p(k_cache),
               _p(v_cache), qkv.shape[0], num_heads, num_kv_heads, head_dim, _stream()),
            "qkv_rope_cache")


# ---------------------------------------------------------------- attention
def generic_attention_tile_rows() -> int:
    return L.core().slb_paged_attention_generic_tile_rows()


def paged_attention_generic(q, k_cache, v_cache, out, block_table, cu_q, ctx_len, tile_seq,
                            tile_row0, num_tiles: int, num_heads: int, num_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int) -> None:
    fn = getattr(L.core(), "slb_paged_attention_generic_" + _suffix(q.dtype))
    L.check(fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
               out.stride(0), block_table.data_ptr(), block_table.shape[1], cu_q.data_ptr(),
               ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), num_tiles,
               num_heads, num_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale),
               int(window), _stream()), "paged_attention_generic")


# ---------------------------------------------------------- matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T (+ bias) on CUDA cores, float32 accumulation."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype == _F32 and out.dtype == _F32:
        fn = L.core().slb_gemm_simt_f32
    elif a.dtype == _BF16 and out.dtype == _BF16:
        fn = L.core().slb_gemm_simt_bf16
    elif a.dtype == _BF16 and out.dtype == _F32:
        fn = L.core().slb_gemm_simt_bf16_f32out
    else:
        raise L.KernelError(f"gemm_simt: unsupported dtypes {a.dtype} -> {out.dtype}")
    L.check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
               out.stride(0), _p(bias), M, N, K, _stream()), "gemm_simt")


# ----------------------------------------------------------------- sampling
def sample_rows(logits: torch.Tensor, out: torch.Tensor, temperature=None, top_k=None,
                top_p=None, seed=None, stream=None, position=None) -> None:
    """out[r] = sampled token of row r; all per-row parameter arrays live on the
    device (float32 / int32 / int64); ``temperature=None`` means greedy rows."""
    R, V = logits.shape
    L.check(L.core().slb_sample_rows(
        logits.data_ptr(), logits.stride(0), R, V, _p(temperature), _p(top_k), _p(top_p),
        _p(seed), _p(stream), _p(position), out.data_ptr(), _stream()), "sample_rows")


# ------------------------------------- tensor-core attention (bfloat16 only)
_sm_count = None
decode_ctas_per_sm = 2      # blocks per SM the split heuristic aims for


def _num_sms() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def attention_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the tensor-core attention kernels for this head
    size gave up (synchronises with the device)."""
    return L.attention(head_dim).slb_attention_status(1 if reset else 0)


def prefill_attention_tc_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the tcgen05 prefill attention gave up."""
    return L.attention(head_dim).slb_prefill_attention_tc_status(1 if reset else 0)


def prefill_attention_tc_where(head_dim: int) -> dict:
    """Where the roles of the tcgen05 prefill attention gave up a bounded wait last:
    per role (code, block, key tile, key tiles of the block); zeros if never."""
    import ctypes
    buf = (ctypes.c_int * 12)()
    L.attention(head_dim).slb_prefill_attention_tc_where(ctypes.cast(buf, ctypes.c_void_p))
    out = {}
    for i, role in enumerate(("loader", "mma", "softmax")):
        code, block, tile, ntiles = buf[4 * i:4 * i + 4]
        out[role] = {"code": hex(code), "block": block, "tile": tile, "tiles": ntiles}
    return out


def has_fast_attention(head_dim: int) -> bool:
    """The tensor-core kernels exist for head sizes that are multiples of 16 up to
    256; the library for a head size is built when it is first asked for."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


use_tc_prefill = True       # tcgen05 prefill attention where it applies (head size 64/128)


def prefill_attention(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                      head_dim, page_size, scale, window) -> None:
    lib = L.attention(head_dim)
    group = num_heads // num_kv_heads
    if (use_tc_prefill and hasattr(lib, "slb_prefill_attention_tc_bf16")
            and lib.slb_prefill_attention_tc_supported(page_size, group)):
        tile_seq, tile_row0, n = ctx.attention_tiles(group, lib.slb_prefill_attention_tc_tile_rows(group))
        L.check(lib.slb_prefill_attention_tc_bf16(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
            out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
            ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads,
            num_kv_heads, page_size, k_cache.shape[0], float(scale), int(window), _stream()),
            "prefill_attention_tc")
        return
    tile_seq, tile_row0, n = ctx.attention_tiles(num_heads // num_kv_heads,
                                                 lib.slb_prefill_attention_tile_rows())
    L.check(lib.slb_prefill_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.cu_q.data_ptr(),
        ctx.ctx_len.data_ptr(), tile_seq.data_ptr(), tile_row0.data_ptr(), n, num_heads,
        num_kv_heads, page_size, k_cache.shape[0], float(scale), int(window), _stream()),
        "prefill_attention")


def decode_splits(num_seqs: int, num_kv_heads: int, group: int, longest_context: int,
                  max_splits: int) -> int:
    """How many ways the keys of each request are split: enough blocks for
    ``decode_ctas_per_sm`` per SM, at most one split per 64 keys of the longest
    context."""
    ctas = num_seqs * num_kv_heads * ((group + 15) // 16)
    want = max(1, (decode_ctas_per_sm * _num_sms()) // max(ctas, 1))
    return max(1, min(want, max_splits, -(-longest_context // 64)))


def decode_attention_split(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                           head_dim, page_size, scale, window) -> None:
    """Attention for a step of single tokens, earlier form: four warps share every
    64-key tile behind a block-wide barrier and a second kernel combines the splits.
    Kept as the twin of ``decode_attention``."""
    lib = L.attention(head_dim)
    S = ctx.num_seqs
    splits = decode_splits(S, num_kv_heads, num_heads // num_kv_heads, ctx.split_hint_len,
                           lib.slb_decode_attention_max_splits())
    scratch = None
    if splits > 1:
        nbytes = lib.slb_decode_attention_scratch_bytes(S, num_heads, splits)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    L.check(lib.slb_decode_attention_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.ctx_len.data_ptr(),
        _p(scratch), S, num_heads, num_kv_heads, page_size, k_cache.shape[0], float(scale),
        int(window), splits, _stream()), "decode_attention")
    global launch_count
    launch_count += 1 if splits > 1 else 0          # the combine kernel


decode_ws_stages = 3           # depth of the kernel's shared-memory ring (2..4)
decode_ws_force_splits = 0     # measurements: launch this many splits instead of the choice below
# The kernel picks each request's number of splits itself, from the request's own length: one
# while it has at most `decode_ws_unsplit_tiles` 64-key tiles, and never more splits than were
# launched.  In the cluster form (the default) a split has two tiles at least, and a request
# takes more splits than one cluster holds only when that saves a block four tiles or more
# (a tile costs a block about 0.8 us while the GPU is not full, a second level of combining
# about 3 us).  In the arrival-counter form (the twin) a split has about
# `decode_ws_split_coef` * sqrt(tiles) tiles: there one block combines every split.
decode_ws_split_coef = 0.8
decode_ws_unsplit_tiles = 6    # (us at 256 / 512 keys, batch 8: 5.4 / 8.4 with 12, 5.4 / 6.0 with 6, 5.9 / 6.0 with 3)

_DECODE_COUNTERS = 1 << 16     # arrival counters held per device (256 KiB)
_decode_counters: Dict[int, torch.Tensor] = {}


def _decode_counter_buffer(device: torch.device) -> torch.Tensor:
    """Zeroed once; every launch of the decode kernel leaves the counters zero.  One
    fixed buffer per device, so addresses captured in CUDA graphs stay valid."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    buf = _decode_counters.get(index)
    if buf is None:
        buf = _decode_counters[index] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32,
                                                    device=device)
    return buf


def decode_ws_splits(num_seqs: int, num_kv_heads: int, group: int, longest_context: int,
                     max_splits: int, tile_keys: int, cluster: bool = False) -> int:
    """The most splits a request may use (the launch's grid): as many as keep all
    blocks of the step resident at once (two per SM), 1 for short contexts.  ``cluster``:
    the kernel's rule for the cluster form (two tiles a split at least) instead of the one
    for the arrival counter (about ``decode_ws_split_coef`` * sqrt(tiles) tiles a split)."""
    head_rows = 8 if group <= 8 else 16
    pairs = num_seqs * num_kv_heads * (-(-group // head_rows))
    tiles = max(1, -(-longest_context // tile_keys))
    if tiles <= decode_ws_unsplit_tiles:
        return 1
    slots = 2 * _num_sms()                      # two blocks of three stages fit on an SM
    per = 2 if cluster else max(1, math.ceil(decode_ws_split_coef * math.sqrt(tiles)))
    longest_uses = -(-tiles // per)             # the kernel's own rule for the longest context
    return max(1, min(max_splits, slots // max(pairs, 1), longest_uses))


def decode_attention_takes(head_dim: int, page_size: int) -> bool:
    """Whether the one-launch decode kernel takes this head size and page size."""
    return has_fast_attention(head_dim) and \
        bool(L.attention(head_dim).slb_decode_attention_ws_supported(page_size))


# The splits of a request combine through the shared memory of a thread-block cluster when
# there are at most eight of them (no scratch, no arrival counter, no round trip through the
# L2 cache: 7 us -> 2 us after the last key at batch 8 on the 7B shape).  A step that would
# like more splits but already has enough blocks to fill the GPU with eight takes eight; one
# with few requests and long contexts takes several clusters a request (up to 64 splits), whose
# partial results meet in global memory: every block of the cluster that finishes a slice of
# the outputs last combines that slice (at batch 1 the arrival-counter form, where one block
# combined everything, spent 16 us there whatever the number of splits).
decode_ws_cluster = True


def _decode_launch_shape(ctx, lib, q_device, num_heads, num_kv_heads):
    """(splits, scratch, counters, cluster) of a launch of the one-launch decode kernel."""
    S = ctx.num_seqs
    group = num_heads // num_kv_heads
    splits = decode_ws_force_splits or decode_ws_splits(
        S, num_kv_heads, group, ctx.split_hint_len, lib.slb_decode_attention_ws_max_splits(),
        lib.slb_decode_attention_ws_tile_keys(), decode_ws_cluster)
    scratch = counters = None
    cluster = False
    most = lib.slb_decode_attention_ws_max_cluster_splits()
    if splits > 1 and decode_ws_cluster:
        pairs = S * num_kv_heads * (-(-group // (8 if group <= 8 else 16)))
        if splits > most and pairs * most >= _num_sms():
            splits = most
        if splits > most:
            splits = splits // most * most          # whole clusters: their results meet in global memory
        cluster = True
    if splits > 1 and (not cluster or splits > most):
        if lib.slb_decode_attention_ws_counters(S, num_heads, num_kv_heads) > _DECODE_COUNTERS:
            splits = 1
        else:
            nbytes = lib.slb_decode_attention_ws_scratch_bytes(S, num_heads, splits)
            scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q_device)
            counters = _decode_counter_buffer(q_device)
    return splits, scratch, counters, cluster


def decode_attention(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                     head_dim, page_size, scale, window) -> None:
    """Attention for a step of single tokens (every q_len == 1): one launch; the
    splits of a request are combined by the block that finishes last.  Head sizes
    that are no multiple of 64 and page sizes that are no power of two from 8 go to
    ``decode_attention_split``."""
    lib = L.attention(head_dim)
    if not lib.slb_decode_attention_ws_supported(page_size):
        decode_attention_split(ctx, q, k_cache, v_cache, out, block_table, num_heads, num_kv_heads,
                               head_dim, page_size, scale, window)
        return
    S = ctx.num_seqs
    splits, scratch, counters, cluster = _decode_launch_shape(ctx, lib, q.device, num_heads, num_kv_heads)
    L.check(lib.slb_decode_attention_ws_bf16(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        out.stride(0), block_table.data_ptr(), block_table.shape[1], ctx.ctx_len.data_ptr(),
        _p(scratch), _p(counters), S, num_heads, num_kv_heads, page_size, k_cache.shape[0],
        float(scale), int(window), splits, int(decode_ws_stages), float(decode_ws_split_coef),
        int(decode_ws_unsplit_tiles), 1 if cluster else 0, _stream()), "decode_attention")


def decode_attention_status(head_dim: int, reset: bool = False) -> int:
    """0 unless a bounded wait inside the decode attention kernel gave up (or a block-table
    entry pointed outside the cache: 0x40)."""
    return L.attention(head_dim).slb_decode_attention_ws_status(1 if reset else 0)


def decode_attention_splits_used(head_dim: int, reset: bool = False) -> int:
    """The most splits any request has used in a launch of the one-launch decode kernel
    since the last reset; 0 if every request ran unsplit (synchronises)."""
    return L.attention(head_dim).slb_decode_attention_ws_splits_used(1 if reset else 0)


# ------------------------------------ tcgen05 weight-streaming product (decode)
TC_MAX_TOKENS = 64
tc_max_stages = 4          # cap on the kernel's shared-memory ring: with four stages two blocks fit
                           # on an SM, and the blocks of the next product become resident (and
                           # request their first weight tiles) beside those of a draining one


tc_blocks_per_sm = 2       # blocks of a product the K split aims at per SM.  Measured on the 7B
                           # shape (ms per decode step at batch 8 / batch 1): 1 block and 6 stages
                           # 3.48 / 3.31, 2 and 4: 3.39 / 3.20, 2 and 5: 3.66 / 3.45, 3 and 3:
                           # 3.45 / 3.22, 4 and 2: 3.48 / 3.26


tc_token_group = 16            # tokens a block takes when a step's tokens are cut into groups
tc_token_group_bytes = 20 << 20    # ... which happens for matrices up to this size from 17 tokens on: every
                                   # group reads the matrix again, from the L2 cache


def tc_token_groups(m: int, w) -> int:
    """Into how many groups of ``tc_token_group`` tokens the tcgen05 products cut a step of
    ``m`` tokens for the matrix ``w`` (1: not at all).  Small matrices only: with few row
    tiles a product has few blocks, and each would finish many tokens one after the other;
    cut into groups it has as many blocks again per group, at the price of reading the
    matrix once per group."""
    if m <= tc_token_group or w.numel() * w.element_size() > tc_token_group_bytes:
        return 1
    return -(-m // tc_token_group)


def tc_decode_splits(n_out: int, k: int, groups: int = 1) -> int:
    """K splits so that (row tiles x token groups x splits) is about ``tc_blocks_per_sm``
    blocks per SM."""
    tiles = -(-n_out // 128) * groups
    kblocks = -(-k // 64)
    slots = tc_blocks_per_sm * _num_sms()
    want = max(1, slots // tiles) if tiles < slots else 1      # all blocks resident at once
    return max(1, min(want, kblocks // 4 if kblocks >= 8 else 1))


# rows of gates, then as many of ups, and so on: the layout for which the tcgen05 product
# applies the activation in its epilogue (half of its 128-row tile)
SWIGLU_BLOCK = 64


def _row_scale(x):
    """(x as the tensor a product reads, sumsq pointer, tiles, eps)"""
    if isinstance(x, ScaledRows):
        return x.z, x.sumsq.data_ptr(), x.sumsq.shape[1], float(x.eps)
    return x, None, 0, 0.0


def gemm_tc_decode(x, w: torch.Tensor, out: Optional[torch.Tensor],
                   bias: Optional[torch.Tensor] = None, splits: int = 0,
                   defer_sum: bool = False, out_dtype: Optional[torch.dtype] = None,
                   swiglu: bool = False):
    """out[M,N] = x[M,K] . w[N,K]^T (+ bias) for up to 64 tokens on tcgen05 tensor
    cores with TMA-streamed weights; bfloat16 operands, float32 or bfloat16 output.
    With ``defer_sum`` and more than one K split the partial sums are returned as a
    ``SplitSum`` (no reduction is launched); otherwise ``out`` (allocated if None).
    ``swiglu``: ``w`` holds gate and up rows alternating in runs of ``SWIGLU_BLOCK``; the
    result is silu(gate) * up, [M, N / 2] (one K split, no bias).  ``x`` may be ``ScaledRows``."""
    global launch_count
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_decode_splits(N, Kd, groups)
    if swiglu:
        if splits != 1 or bias is not None or N % (2 * SWIGLU_BLOCK):
            raise ValueError("gemm_tc_decode: the fused activation needs one K split, no bias and "
                             f"a multiple of {2 * SWIGLU_BLOCK} rows")
        if out is None:
            out = torch.empty((M, N // 2), dtype=out_dtype or x.dtype, device=x.device)
    out_dtype = out.dtype if out is not None else (out_dtype or x.dtype)
    ws = torch.empty((splits, M, N), dtype=_F32, device=x.device) if splits > 1 else None
    deferred = defer_sum and splits > 1
    if out is None and not deferred:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    L.check(L.core().slb_gemm_tc_decode_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _p(out),
        out.stride(0) if out is not None else N,
        _p(bias), _p(ws), 1 if out_dtype == _F32 else 0, M, N, Kd, splits, tc_max_stages,
        1 if deferred else 0, 1 if swiglu else 0, sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_decode")
    if deferred:
        return SplitSum(ws, bias, out_dtype)
    launch_count += 1 if splits > 1 else 0
    return out


TC_MAX_CLUSTER = 8             # K splits that can share a row tile as one thread-block cluster
TC_ROPE_HEAD_DIMS = (16, 32, 64, 128)   # a 128-row tile of the q|k|v product holds whole heads


def tc_cluster_splits(n_out: int, k: int, groups: int = 1) -> int:
    return min(tc_decode_splits(n_out, k, groups), TC_MAX_CLUSTER)


def gemm_tc_cluster(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None, splits: int = 0) -> torch.Tensor:
    """out[M,N] = x . w^T (+ bias) in bfloat16 for up to 64 tokens, like
    ``gemm_tc_decode``, but the K splits of a row tile form a thread-block cluster and
    add their results up through one another's shared memory: no partial sums in
    global memory and no reduction kernel; a fixed order of additions.  ``x`` may be
    ``ScaledRows``."""
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_cluster_splits(N, Kd, groups)
    if out is None:
        out = torch.empty((M, N), dtype=_BF16, device=x.device)
    L.check(L.core().slb_gemm_tc_cluster_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), _p(bias),
        M, N, Kd, splits, _cluster_stages(M, groups), sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_cluster")
    return out


def gemm_tc_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                     positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                     page_size: int, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                     q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                     head_dim: int, splits: int = 0) -> None:
    """The q|k|v product of up to 64 tokens together with ``qkv_rope_cache``: the product's
    epilogue adds the bias, rotates q and k, writes q to ``q_out`` and k, v into the paged
    cache.  Head sizes in ``TC_ROPE_HEAD_DIMS``.  ``x`` may be ``ScaledRows``."""
    x, sumsq, tiles, eps = _row_scale(x)
    M, Kd = x.shape
    groups = tc_token_groups(M, w_qkv)
    splits = splits or tc_cluster_splits(w_qkv.shape[0], Kd, groups)
    L.check(L.core().slb_gemm_tc_qkv_rope_bf16(
        x.data_ptr(), x.stride(0), w_qkv.data_ptr(), w_qkv.stride(0),
        _p(bias), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, _num_pages(k_cache), _p(inv_freq), rotary_dim,
        q_out.data_ptr(), q_out.stride(0), _p(k_cache), _p(v_cache), M, num_heads, num_kv_heads,
        head_dim, Kd, splits, _cluster_stages(M, groups), sumsq, tiles, eps,
        tc_token_group if groups > 1 else 0, _stream()), "gemm_tc_qkv_rope")


tc_cluster_many_token_stages = 3   # ring depth of the cluster products above 16 tokens: their x tiles grow
                                   # with the tokens, and with four stages only two blocks fit on an SM,
                                   # which is fewer clusters of eight than a 36-tile product has at once
                                   # (the rest started when the first had finished: 38 against 25 us for
                                   # q|k|v at 64 tokens)


def _cluster_stages(M: int, groups: int = 1) -> int:
    if M <= 16 or (groups > 1 and tc_token_group <= 16):    # (what a block sees)
        return tc_max_stages
    return min(tc_max_stages, tc_cluster_many_token_stages)


def gemm_tc_resid_norm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                       resid: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                       splits: int = 0) -> ScaledRows:
    """The product that closes a residual branch with the add and the RMS norm that follow
    it, in one kernel: resid (float32, in place) += x . w^T (+ bias); the result is the normed
    rows in the form ``ScaledRows`` (bfloat16(resid * norm_weight) and per-tile sums of
    squares), whose factor 1 / rms the next product applies.  Up to 64 tokens."""
    M, Kd = x.shape
    N = w.shape[0]
    groups = tc_token_groups(M, w)
    splits = splits or tc_cluster_splits(N, Kd, groups)
    z = torch.empty((M, N), dtype=_BF16, device=x.device)
    sumsq = torch.empty((M, -(-N // 128)), dtype=_F32, device=x.device)
    L.check(L.core().slb_gemm_tc_resid_norm_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _p(bias), resid.data_ptr(),
        resid.stride(0), norm_weight.data_ptr(), z.data_ptr(), z.stride(0), sumsq.data_ptr(),
        M, N, Kd, splits, _cluster_stages(M, groups), tc_token_group if groups > 1 else 0,
        _stream()), "gemm_tc_resid_norm")
    return ScaledRows(z, sumsq, eps, resid, norm_weight)


def gemm_tc_status(reset: bool = False) -> int:
    """0 unless a bounded wait inside the tcgen05 kernels ran out, or the q|k|v epilogue met a
    block-table entry outside the cache (synchronises)."""
    return L.core().slb_gemm_tc_status(1 if reset else 0)

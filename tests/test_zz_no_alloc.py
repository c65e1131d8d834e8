"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of the kernel library run where cudaMalloc is not available to them: a
plugin with a fixed memory budget, a loop that must not block on the allocator, a
process on a GPU that is already full.  ``slb_decode_attention_bf16_noalloc``
serves them with a scratch array built into the library.  This test calls it
through its exported C symbol, twice in a row with different inputs (the second
call meets the first call's leftovers in the shared scratch), and compares each
result with the regular entry point's, which is given freshly allocated scratch,
and with attention written out in float32 torch operations.  A third case has a
window, so that whole splits see no key at all and the combine step has to ignore
slots of the shared array that still hold an earlier call's numbers.

The file name sorts last on purpose, so that a run that stops at the first failure
has already run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 2e-2          # the bfloat16 tolerance of the kernel tests


def _library(head_dim):
    from servelab_b200.csrc.build import attention_library
    lib = ctypes.CDLL(attention_library(head_dim))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.slb_decode_attention_bf16_noalloc.argtypes = [P, I, P, P, P, I, P, I, P, I, I, I, I, I, F, I, I, P]
    lib.slb_decode_attention_bf16_noalloc.restype = I
    lib.slb_decode_attention_bf16.argtypes = [P, I, P, P, P, I, P, I, P, P, I, I, I, I, I, F, I, I, P]
    lib.slb_decode_attention_bf16.restype = I
    lib.slb_decode_attention_scratch_bytes.argtypes = [I, I, I]
    lib.slb_decode_attention_scratch_bytes.restype = ctypes.c_longlong
    lib.slb_decode_attention_noalloc_capacity_bytes.restype = ctypes.c_longlong
    lib.slb_decode_attention_noalloc_strerror.argtypes = [I]
    lib.slb_decode_attention_noalloc_strerror.restype = ctypes.c_char_p
    return lib


def _case(seed, S, H, Hkv, D, ps, max_ctx):
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(1, max_ctx + 1, (S,), generator=g).tolist()
    ctx[0] = max_ctx
    need = [-(-c // ps) for c in ctx]
    pages = sum(need) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    width = max(need)
    table = torch.full((S, width), -1, dtype=torch.int32)
    for s, n in enumerate(need):
        table[s, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    kc = torch.randn(pages, Hkv, ps, D, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(pages, Hkv, ps, D, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(S, H * D, generator=g).to(torch.bfloat16).to(DEV)
    return q, kc, vc, table.to(DEV), torch.tensor(ctx, dtype=torch.int32, device=DEV)


def _float32_attention(q, kc, vc, table, ctx_len, H, Hkv, D, ps, window):
    """Attention of one query per request over its paged keys, in float32 torch operations."""
    g = H // Hkv
    outs = []
    for s, c in enumerate(ctx_len.tolist()):
        pages = table[s, :-(-c // ps)].long()
        k = kc[pages].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:c].float()     # [c, Hkv, D]
        v = vc[pages].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:c].float()
        qs = q[s].view(H, D).float()
        sc = torch.einsum("hd,rhd->hr", qs, k.repeat_interleave(g, 1)) / math.sqrt(D)
        if window:
            r = torch.arange(c, device=sc.device)
            sc = sc.masked_fill(((c - 1) - r >= window)[None], float("-inf"))
        outs.append(torch.einsum("hr,rhd->hd", torch.softmax(sc, -1), v.repeat_interleave(g, 1)).reshape(-1))
    return torch.stack(outs)


def test_no_alloc_entry_matches_the_regular_one_on_two_calls_in_a_row():
    H, Hkv, D, ps, S, splits = 14, 2, 64, 16, 5, 4
    lib = _library(D)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.slb_decode_attention_noalloc_capacity_bytes() == 4 << 20
    # the third call has a window of 100 keys over contexts up to 900: the first splits of the
    # long requests hold no visible key, and their slots keep the second call's numbers
    for call, (seed, max_ctx, window) in enumerate(((11, 700, 0), (12, 400, 0), (13, 900, 100))):
        q, kc, vc, table, ctx_len = _case(seed, S, H, Hkv, D, ps, max_ctx)
        scale = 1 / math.sqrt(D)
        want = torch.empty_like(q)
        scratch = torch.empty(lib.slb_decode_attention_scratch_bytes(S, H, splits) // 4,
                              dtype=torch.float32, device=DEV)
        rc = lib.slb_decode_attention_bf16(
            q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), want.data_ptr(),
            want.stride(0), table.data_ptr(), table.shape[1], ctx_len.data_ptr(),
            scratch.data_ptr(), S, H, Hkv, ps, kc.shape[0], scale, window, splits, stream)
        assert rc == 0
        exact = _float32_attention(q, kc, vc, table, ctx_len, H, Hkv, D, ps, window)
        got = torch.full_like(q, 3.0)
        torch.cuda.synchronize()
        # free device memory as the driver counts it: a cudaMalloc inside the library (which
        # links its own runtime) would not show in torch's allocator statistics, but it does here
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.slb_decode_attention_bf16_noalloc(
            q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), got.data_ptr(),
            got.stride(0), table.data_ptr(), table.shape[1], ctx_len.data_ptr(),
            S, H, Hkv, ps, kc.shape[0], scale, window, splits, stream)
        assert rc == 0, lib.slb_decode_attention_noalloc_strerror(rc)
        torch.cuda.synchronize()
        if call > 0:        # (the first call on a device loads the module and looks the array up)
            assert torch.cuda.mem_get_info()[0] >= free_before, "the call took device memory"
        err = float((got.float() - want.float()).abs().max())
        assert err <= TOL, f"call {call}: differs from the regular entry point by {err}"
        err32 = float((got.float() - exact).abs().max())
        assert err32 <= TOL, f"call {call}: differs from float32 attention by {err32}"
        assert float(exact.abs().max()) > 0.05               # a real result, not zeros


def test_no_alloc_entry_refuses_what_does_not_fit():
    D = 64
    lib = _library(D)
    H, Hkv, ps = 64, 8, 16
    S, splits = 64, 32                         # 64*64*32*(64+2)*4 bytes = 34.6 MB > 4 MiB
    assert lib.slb_decode_attention_scratch_bytes(S, H, splits) > \
        lib.slb_decode_attention_noalloc_capacity_bytes()
    q, kc, vc, table, ctx_len = _case(1, S, H, Hkv, D, ps, 40)
    out = torch.full_like(q, 5.0)
    rc = lib.slb_decode_attention_bf16_noalloc(
        q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), out.stride(0),
        table.data_ptr(), table.shape[1], ctx_len.data_ptr(), S, H, Hkv, ps, kc.shape[0], 0.125, 0,
        splits, torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    assert b"exceed the built-in scratch" in lib.slb_decode_attention_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 5.0).all()), "a refused call must not launch anything"

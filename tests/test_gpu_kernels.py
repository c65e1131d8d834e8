"""Each CUDA kernel alone against a plain float32 torch expression of the same
operation, at sizes other than the engine's tiny models (odd widths, head sizes in
steps of 16, groups that are no power of two), in float32 and bfloat16.  Inputs are
shaped so that faults show: one far key that must win the softmax, keys at page and
window edges, shuffled page tables, equal maxima for the argmax."""

import math

import numpy as np
import pytest
import torch

import plain_model as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def K():
    from servelab_b200.ops import kernels
    return kernels


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding(dtype):
    table = torch.randn(301, 72, device=DEV).to(DT[dtype])
    ids = i32([0, 300, 17, 17, 5])
    out = torch.full((5, 72), 7.0, device=DEV)
    K().embedding(ids, table, out)
    assert torch.equal(out, table.float()[ids.long()])


# ---------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("h", [72, 1000, 3584])
def test_add_rmsnorm(dtype, h):
    dt = DT[dtype]
    resid = torch.randn(9, h, device=DEV) * 3
    delta = (torch.randn(9, h, device=DEV)).to(dt)
    w = 1 + 0.1 * torch.randn(h, device=DEV)
    want_resid = resid + delta.float()
    want = P.rms_norm(want_resid, w, 1e-5)
    out = torch.empty(9, h, device=DEV, dtype=dt)
    r = resid.clone()
    K().add_rmsnorm(r, delta, w, 1e-5, out)
    assert torch.equal(r, want_resid)                       # the stream is updated in float32
    assert (out.float() - want).abs().max() <= TOL[dtype] * 4
    # without delta the stream is untouched
    r2 = resid.clone()
    K().add_rmsnorm(r2, None, w, 1e-5, out)
    assert torch.equal(r2, resid)
    assert (out.float() - P.rms_norm(resid, w, 1e-5)).abs().max() <= TOL[dtype] * 4
    # selected rows: nothing is written back
    rows = i32([8, 0, 3])
    r3 = resid.clone()
    sel = torch.empty(3, h, device=DEV, dtype=dt)
    K().add_rmsnorm(r3, delta, w, 1e-5, sel, rows)
    assert torch.equal(r3, resid)
    assert (sel.float() - want[rows.long()]).abs().max() <= TOL[dtype] * 4


@pytest.mark.parametrize("h", [64, 172, 3584, 150, 8200])
@pytest.mark.parametrize("rows,nparts", [(1, 2), (9, 5), (3, 11)])
def test_add_rmsnorm_of_split_sums(h, rows, nparts):
    """The update as float32 partial sums of a K-split product (+ bias): a cluster of
    blocks per row where the width allows, one block per row otherwise; whole rows and
    selected rows."""
    from servelab_b200.ops.kernels import SplitSum
    resid = torch.randn(rows, h, device=DEV) * 3
    parts = torch.randn(nparts, rows, h, device=DEV)
    bias = torch.randn(h, device=DEV)
    w = 1 + 0.1 * torch.randn(h, device=DEV)
    want_resid = resid + parts.sum(0) + bias
    want = P.rms_norm(want_resid, w, 1e-5)
    out = torch.empty(rows, h, device=DEV, dtype=torch.bfloat16)
    r = resid.clone()
    K().add_rmsnorm(r, SplitSum(parts, bias, torch.bfloat16), w, 1e-5, out)
    assert (r - want_resid).abs().max() <= 1e-5
    assert (out.float() - want).abs().max() <= TOL["bfloat16"] * 4
    again = torch.empty_like(out)
    r2 = resid.clone()
    K().add_rmsnorm(r2, SplitSum(parts, bias, torch.bfloat16), w, 1e-5, again)
    assert torch.equal(again, out) and torch.equal(r2, r)    # deterministic
    # a row does not depend on the rest of the batch (bit-exact)
    one = torch.empty(1, h, device=DEV, dtype=torch.bfloat16)
    K().add_rmsnorm(resid[rows - 1:].clone(), SplitSum(parts[:, rows - 1:].contiguous(), bias, torch.bfloat16),
                    w, 1e-5, one)
    assert torch.equal(one[0], out[rows - 1])
    # selected rows: nothing is written back
    sel_rows = i32([rows - 1, 0])
    r3 = resid.clone()
    sel = torch.empty(2, h, device=DEV, dtype=torch.bfloat16)
    K().add_rmsnorm(r3, SplitSum(parts, bias, torch.bfloat16), w, 1e-5, sel, sel_rows)
    assert torch.equal(r3, resid)
    assert torch.equal(sel[0], out[rows - 1]) and torch.equal(sel[1], out[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter", [173, 172, 176, 18944])      # 1, 4 and 8 elements a thread
def test_swiglu(dtype, inter):
    dt = DT[dtype]
    gu = (torch.randn(7, 2 * inter, device=DEV) * 3).to(dt)
    out = torch.empty(7, inter, device=DEV, dtype=dt)
    K().swiglu(gu, out)
    g, u = gu.float()[:, :inter], gu.float()[:, inter:]
    want = g * torch.sigmoid(g) * u
    # results reach |30|: the bound is relative (one rounding to the output dtype)
    rel = 2.0 ** -8 if dtype == "bfloat16" else 2.0 ** -21
    assert bool(((out.float() - want).abs() <= want.abs() * rel + 1e-6).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter,block", [(192, 64), (24, 3), (1280, 64), (160, 16)])
def test_swiglu_of_alternating_runs(dtype, inter, block):
    """Gates and ups alternate in runs of ``block`` columns."""
    dt = DT[dtype]
    gu = (torch.randn(5, 2 * inter, device=DEV) * 3).to(dt)
    out = torch.empty(5, inter, device=DEV, dtype=dt)
    K().swiglu(gu, out, block)
    runs = gu.float().view(5, inter // block, 2, block)
    g, u = runs[:, :, 0].reshape(5, inter), runs[:, :, 1].reshape(5, inter)
    want = g * torch.sigmoid(g) * u
    rel = 2.0 ** -8 if dtype == "bfloat16" else 2.0 ** -21
    assert bool(((out.float() - want).abs() <= want.abs() * rel + 1e-6).all())


@pytest.mark.parametrize("M,inter,Kd", [(1, 64, 64), (8, 192, 264), (16, 1088, 896), (37, 704, 512),
                                        (64, 320, 1024)])
def test_gemm_tcgen05_decode_with_activation(M, inter, Kd):
    """The product's epilogue applies silu(gate) * up when the weights' rows alternate in
    runs of 64; compared with the float64 product of the separate matrices."""
    B = K().SWIGLU_BLOCK
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    gate = (torch.randn(inter, Kd, device=DEV) * 2 / math.sqrt(Kd)).bfloat16()
    up = (torch.randn(inter, Kd, device=DEV) * 2 / math.sqrt(Kd)).bfloat16()
    w = torch.stack([gate.view(inter // B, B, Kd), up.view(inter // B, B, Kd)], dim=1).reshape(2 * inter, Kd)
    g = x.double() @ gate.double().t()
    want = (g * torch.sigmoid(g) * (x.double() @ up.double().t())).float()
    out = K().gemm_tc_decode(x, w, None, splits=1, swiglu=True, out_dtype=torch.float32)
    assert K().gemm_tc_status(True) == 0, "a bounded wait in the kernel ran out"
    assert out.shape == (M, inter)
    assert (out - want).abs().max() <= 2e-3
    ob = K().gemm_tc_decode(x, w, None, splits=1, swiglu=True)
    assert ob.dtype == torch.bfloat16
    assert bool(((ob.float() - want).abs() <= want.abs() * 2.0 ** -7 + 2e-3).all())
    # the same numbers as the product followed by the activation kernel (both round the
    # float32 sums once)
    gu = torch.empty(M, 2 * inter, device=DEV)
    K().gemm_tc_decode(x, w, gu, None, 1)
    two = torch.empty(M, inter, device=DEV)
    K().swiglu(gu, two, B)
    assert (two - out).abs().max() <= 1e-5
    with pytest.raises(ValueError):
        K().gemm_tc_decode(x, w, None, splits=2, swiglu=True)


# ------------------------------------------------------ rotary + cache write
def _paged(num_pages, Hkv, ps, D, dt):
    return (torch.zeros(num_pages, Hkv, ps, D, device=DEV, dtype=dt),
            torch.zeros(num_pages, Hkv, ps, D, device=DEV, dtype=dt))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,D,rot", [(6, 2, 48, 48), (5, 5, 16, 8), (3, 1, 80, 0),
                                         (28, 4, 128, 128), (4, 2, 64, 32), (3, 1, 40, 20)])
def test_qkv_rope_cache(dtype, H, Hkv, D, rot):
    dt = DT[dtype]
    ps, T = 4, 11
    # two requests: 7 tokens from position 5, 4 tokens from position 0
    positions = list(range(5, 12)) + list(range(0, 4))
    seq = [0] * 7 + [1] * 4
    table = i32([[9, 2, 7], [4, -1, -1]])
    qkv = torch.randn(T, (H + 2 * Hkv) * D, device=DEV).to(dt)
    bias = torch.randn((H + 2 * Hkv) * D, device=DEV)
    inv = P.rope_inv_freq(rot, 10000.0).to(DEV) if rot else None
    q_out = torch.empty(T, H * D, device=DEV, dtype=dt)
    kc, vc = _paged(12, Hkv, ps, D, dt)
    K().qkv_rope_cache(qkv, bias, i32(positions), i32(seq), table, ps, inv, rot, q_out, kc, vc,
                       H, Hkv, D)
    x = qkv.float() + bias
    q = x[:, :H * D].view(T, H, D)
    k = x[:, H * D:(H + Hkv) * D].view(T, Hkv, D)
    v = x[:, (H + Hkv) * D:].view(T, Hkv, D)
    pos_t = torch.tensor(positions)
    if rot:
        q = torch.cat([P.rope(q[..., :rot].cpu(), pos_t, inv.cpu()).to(DEV), q[..., rot:]], -1)
        k = torch.cat([P.rope(k[..., :rot].cpu(), pos_t, inv.cpu()).to(DEV), k[..., rot:]], -1)
    tol = TOL[dtype] * 8
    assert (q_out.float().view(T, H, D) - q).abs().max() <= tol
    tab = table.cpu()
    for t in range(T):
        page = int(tab[seq[t], positions[t] // ps])
        assert (kc[page, :, positions[t] % ps].float() - k[t]).abs().max() <= tol
        assert (vc[page, :, positions[t] % ps].float() - v[t]).abs().max() <= tol
    written = {int(tab[seq[t], positions[t] // ps]) for t in range(T)}
    for page in range(12):
        if page not in written:
            assert float(kc[page].abs().max()) == 0 and float(vc[page].abs().max()) == 0
    # a run that reads another layer's cache writes nothing
    kc2, vc2 = _paged(12, Hkv, ps, D, dt)
    K().qkv_rope_cache(qkv, bias, i32(positions), i32(seq), table, ps, inv, rot, q_out, None, None,
                       H, Hkv, D)
    assert float(kc2.abs().max()) == 0
    if dtype == "bfloat16":
        # the projection as three float32 partial sums of a K-split product (decode steps)
        from servelab_b200.ops.kernels import SplitSum
        p1, p2 = torch.randn_like(qkv.float()), torch.randn_like(qkv.float())
        parts = torch.stack([p1, p2, qkv.float() - p1 - p2]).contiguous()
        q3 = torch.empty(T, H * D, device=DEV, dtype=dt)
        kc3, vc3 = _paged(12, Hkv, ps, D, dt)
        K().qkv_rope_cache(SplitSum(parts, None, dt), bias, i32(positions), i32(seq), table, ps, inv,
                           rot, q3, kc3, vc3, H, Hkv, D)
        assert (q3.float() - q_out.float()).abs().max() <= tol
        assert (kc3.float() - kc.float()).abs().max() <= tol
        assert (vc3.float() - vc.float()).abs().max() <= tol


# ------------------------------------------------------------------ attention
class PagedCase:
    """Requests with dense K/V scattered into shuffled pages."""

    def __init__(self, ctx_lens, q_lens, H, Hkv, D, ps, dt, seed=0, pad_pages=3):
        g = torch.Generator().manual_seed(seed)
        self.H, self.Hkv, self.D, self.ps, self.dt = H, Hkv, D, ps, dt
        self.ctx_lens, self.q_lens = ctx_lens, q_lens
        need = [-(-c // ps) for c in ctx_lens]
        total = sum(need) + pad_pages
        perm = torch.randperm(total, generator=g).tolist()
        self.tables, self.k, self.v = [], [], []
        self.kc, self.vc = _paged(total, Hkv, ps, D, dt)
        self.kc.normal_(generator=None)                       # stale data in unused slots
        self.vc.normal_(generator=None)
        for c, n in zip(ctx_lens, need):
            pages = [perm.pop() for _ in range(n)]
            self.tables.append(pages)
            k = torch.randn(c, Hkv, D, generator=g).to(dt)
            v = torch.randn(c, Hkv, D, generator=g).to(dt)
            self.k.append(k)
            self.v.append(v)
        self.q = [torch.randn(n, H, D, generator=g).to(dt) for n in q_lens]

    def scatter(self):
        for pages, k, v in zip(self.tables, self.k, self.v):
            for p in range(k.shape[0]):
                self.kc[pages[p // self.ps], :, p % self.ps] = k[p].to(DEV)
                self.vc[pages[p // self.ps], :, p % self.ps] = v[p].to(DEV)

    def device_args(self):
        width = max(len(t) for t in self.tables)
        table = i32([t + [-1] * (width - len(t)) for t in self.tables])
        cu = [0]
        for n in self.q_lens:
            cu.append(cu[-1] + n)
        q = torch.cat(self.q).reshape(cu[-1], self.H * self.D).to(DEV)
        return q, table, i32(cu), i32(self.ctx_lens)

    def reference(self, window=None, scale=None):
        outs = []
        g = self.H // self.Hkv
        for q, k, v, c, n in zip(self.q, self.k, self.v, self.ctx_lens, self.q_lens):
            qf, kf, vf = q.float(), k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1)
            s = torch.einsum("qhd,rhd->hqr", qf, kf) * (scale or 1 / math.sqrt(self.D))
            a = torch.arange(c - n, c)[:, None]
            r = torch.arange(c)[None, :]
            mask = r > a
            if window:
                mask = mask | (a - r >= window)
            s = s.masked_fill(mask[None], float("-inf"))
            outs.append(torch.einsum("hqr,rhd->qhd", torch.softmax(s, -1), vf).reshape(n, -1))
        return torch.cat(outs)


def run_generic(case, window=0, scale=None):
    from servelab_b200.engine.batch import StepContext
    k = K()
    case.scatter()
    q, table, cu, ctx_len = case.device_args()
    ctx = StepContext(DEV)
    ctx.q_lens = case.q_lens
    tile_seq, tile_row0, n = ctx.attention_tiles(case.H // case.Hkv, k.generic_attention_tile_rows())
    out = torch.empty_like(q)
    k.paged_attention_generic(q, case.kc, case.vc, out, table, cu, ctx_len, tile_seq, tile_row0, n,
                              case.H, case.Hkv, case.D, case.ps, scale or 1 / math.sqrt(case.D),
                              window)
    return out.float().cpu()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,D,ps", [(6, 2, 16, 16), (7, 1, 64, 8), (5, 5, 48, 4),
                                        (28, 4, 128, 16), (2, 1, 256, 32), (12, 2, 80, 5)])
def test_generic_attention_mixed_batch(dtype, H, Hkv, D, ps):
    # a whole prompt, a portion in the middle of one, two single tokens, a 2-token portion
    case = PagedCase([37, 150, 1, 263, 34], [37, 19, 1, 1, 2], H, Hkv, D, ps, DT[dtype], seed=D)
    got, want = run_generic(case), case.reference()
    assert (got - want).abs().max() <= TOL[dtype] * (5 if dtype == "float32" else 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 7, 16, 33])
def test_generic_attention_window_edges(dtype, window):
    case = PagedCase([90, 41, 64], [23, 1, 64], 6, 3, 32, 8, DT[dtype], seed=window)
    # the key just outside the window would win by far if it were visible; the key
    # just inside must be seen
    for q, k, c, n in zip(case.q, case.k, case.ctx_lens, case.q_lens):
        a = c - 1                                        # last query
        if a - window >= 0:
            k[a - window] = (q[-1, 0::2].mean(0) * 50).to(k.dtype)
    got, want = run_generic(case, window=window), case.reference(window=window)
    assert (got - want).abs().max() <= TOL[dtype] * (5 if dtype == "float32" else 1)
    full = case.reference()
    assert (want - full).abs().max() > 1e-2              # the window does change the result


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("needle", [0, 15, 16, 511, 512, 700])
def test_generic_attention_finds_one_far_key(dtype, needle):
    """One key among 701 is aligned with the query and scaled so that it takes all
    the weight: the output must be that key's value (page edges included)."""
    H, Hkv, D, ps = 4, 2, 64, 16
    case = PagedCase([701], [1], H, Hkv, D, ps, DT[dtype], seed=needle)
    for kvh in range(Hkv):
        qdir = case.q[0][0, kvh * 2].float()
        case.k[0][needle, kvh] = (qdir * 40 / qdir.norm()).to(case.dt)
        case.q[0][0, kvh * 2 + 1] = case.q[0][0, kvh * 2]
    case.q[0] = (case.q[0].float() * 8).to(case.dt)
    got = run_generic(case).view(1, H, D)
    for h in range(H):
        assert (got[0, h] - case.v[0][needle, h // 2].float()).abs().max() <= 2e-2


# ------------------------------------------------------------ matrix product
@pytest.mark.parametrize("M,N,Kd", [(1, 7, 5), (33, 172, 64), (70, 65, 173), (5, 300, 129)])
def test_gemm_simt(M, N, Kd):
    a = torch.randn(M, Kd, device=DEV)
    w = torch.randn(N, Kd, device=DEV)
    b = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV)
    K().gemm_simt(a, w, out, b)
    want = (a.double() @ w.double().t() + b.double()).float()
    assert (out - want).abs().max() <= 1e-5 * math.sqrt(Kd) * 4
    # a row does not depend on the rest of the batch (bit-exact)
    one = torch.empty(1, N, device=DEV)
    K().gemm_simt(a[M - 1:M].contiguous(), w, one, b)
    assert torch.equal(one[0], out[M - 1])
    ab, wb = a.bfloat16(), w.bfloat16()
    o32 = torch.empty(M, N, device=DEV)
    K().gemm_simt(ab, wb, o32, None)
    assert (o32 - (ab.double() @ wb.double().t()).float()).abs().max() <= 1e-4 * math.sqrt(Kd)
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().gemm_simt(ab, wb, ob, None)
    assert torch.equal(ob, o32.bfloat16())


def test_bf16_linear_dispatch_shapes():
    """Aligned shapes go to the library GEMM, ragged ones to the CUDA-core kernel;
    both agree with float64 within bfloat16 rounding."""
    from servelab_b200.ops.linear import linear
    for M, N, Kd in [(40, 256, 96), (40, 172, 64), (3, 64, 172), (100, 300, 80)]:
        x = torch.randn(M, Kd, device=DEV).bfloat16()
        w = (torch.randn(N, Kd, device=DEV) * 0.05).bfloat16()
        want = (x.double() @ w.double().t()).float()
        y = linear(x, w)
        assert y.dtype == torch.bfloat16 and (y.float() - want).abs().max() <= 2e-2
        y32 = linear(x, w, out_dtype=torch.float32)
        assert y32.dtype == torch.float32 and (y32 - want).abs().max() <= 2e-3


@pytest.mark.parametrize("N,Kd", [(3584, 3584), (3584, 18944), (4608, 3584), (5120, 13824), (896, 4864)])
def test_bf16_linear_at_every_token_count_of_a_step(N, Kd):
    """``linear`` at the layer sizes of the large shapes for 1 to 80 tokens: whichever kernel
    the dispatch picks (cluster form, partial sums, vendor GEMM), the result agrees with
    float64, as a tensor and as the update a norm consumes."""
    from servelab_b200.ops.linear import linear
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    for M in (1, 8, 16, 17, 40, 64, 65, 80):
        x = torch.randn(M, Kd, device=DEV).bfloat16()
        want = (x.double() @ w.double().t()).float()
        y = linear(x, w)
        assert y.shape == (M, N) and (y.float() - want).abs().max() <= 3e-2, M
        d = linear(x, w, consumer="norm")
        resid = torch.zeros(M, N, device=DEV)
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        K().add_rmsnorm(resid, K().plain_unless(None, d) if not isinstance(d, K().SplitSum) else d,
                        torch.ones(N, device=DEV), 1e-6, out)
        assert (resid - want).abs().max() <= 3e-2, M
    assert K().gemm_tc_status(True) == 0


# ------------------------------------------------------------------- sampling
def test_argmax_takes_the_first_of_equal_maxima():
    V = 152064 + 7
    logits = torch.randn(5, V, device=DEV)
    logits[0, 1000] = logits[0, 77] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 60.0
    logits[3, :] = 1.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    K().sample_rows(logits, out)
    assert out.tolist()[:4] == [77, V - 1, 0, 0]
    assert out.tolist()[4] == int(torch.argmax(logits[4]))


def _sample(logits, temp, top_k, top_p, seed, stream, pos):
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=DEV)
    K().sample_rows(logits, out, torch.tensor(temp, dtype=torch.float32, device=DEV), i32(top_k),
                    torch.tensor(top_p, dtype=torch.float32, device=DEV),
                    torch.tensor(seed, dtype=torch.int64, device=DEV),
                    torch.tensor(stream, dtype=torch.int64, device=DEV), i32(pos))
    return out.tolist()


@pytest.mark.parametrize("mode", ["temperature", "top_k", "top_p"])
def test_sampler_matches_the_host_mirror(mode):
    V, R = 1031, 256
    g = torch.Generator().manual_seed(3)
    row = torch.randn(V, generator=g) * 2
    logits = row.repeat(R, 1).to(DEV)
    temp, top_k, top_p = 0.7, -1, 1.0
    if mode == "top_k":
        top_k = 5
    if mode == "top_p":
        top_p = 0.6
    seed, stream = 1234 + (1 << 40), 9
    got = _sample(logits, [temp] * R, [top_k] * R, [top_p] * R, [seed] * R, [stream] * R,
                  list(range(R)))
    want = [P.sample_token(row, temp, P.philox_uniform(seed, stream, i), top_k, top_p)
            for i in range(R)]
    same = sum(int(a == b) for a, b in zip(got, want))
    assert same >= R - 1, f"{R - same} draws differ from the host mirror"
    kept = (P.filtered_probs(row, temp, top_k, top_p) > 0).nonzero().flatten().tolist()
    assert set(got) <= set(kept)
    if mode == "top_k":
        assert len(kept) == 5
    # the draw depends on (seed, stream, position) only, not on the row's place in the batch
    again = _sample(logits[:3], [temp] * 3, [top_k] * 3, [top_p] * 3, [seed] * 3, [stream] * 3,
                    [200, 7, 31])
    assert again == [got[200], got[7], got[31]]
    other = _sample(logits[:64], [temp] * 64, [top_k] * 64, [top_p] * 64, [seed + 1] * 64,
                    [stream] * 64, list(range(64)))
    assert other != got[:64]


def test_sampler_mixes_greedy_and_random_rows_and_follows_the_distribution():
    V, R = 50, 4000
    row = torch.linspace(-2, 2, V)
    logits = row.repeat(R, 1).to(DEV)
    temps = [0.0 if i % 2 else 1.3 for i in range(R)]
    got = _sample(logits, temps, [-1] * R, [1.0] * R, [7] * R, [1] * R, list(range(R)))
    assert all(got[i] == V - 1 for i in range(1, R, 2))
    counts = np.bincount([got[i] for i in range(0, R, 2)], minlength=V) / (R / 2)
    want = torch.softmax(row.double() / 1.3, -1).numpy()
    assert np.abs(counts - want).max() < 0.03


# -------------------------------------------- tensor-core attention (bfloat16)
def _ctx_for(case):
    from servelab_b200.engine.batch import StepContext
    q, table, cu, ctx_len = case.device_args()
    ctx = StepContext(DEV)
    ctx.q_lens, ctx.num_seqs = case.q_lens, len(case.q_lens)
    ctx.cu_q, ctx.ctx_len = cu, ctx_len
    ctx.max_ctx_len = ctx.split_hint_len = max(case.ctx_lens)
    return ctx, q, table


@pytest.mark.parametrize("H,Hkv,D,ps", [(6, 2, 16, 16), (7, 1, 64, 8), (4, 2, 48, 4),
                                        (28, 4, 128, 16), (2, 1, 256, 32), (20, 1, 32, 16),
                                        (3, 3, 64, 64), (10, 2, 128, 128), (8, 1, 128, 32)])
@pytest.mark.parametrize("window", [0, 40])
def test_prefill_attention_tensor_cores(H, Hkv, D, ps, window):
    case = PagedCase([37, 150, 1, 263, 34, 300], [37, 19, 1, 1, 2, 300], H, Hkv, D, ps,
                     torch.bfloat16, seed=D + window)
    case.scatter()
    ctx, q, table = _ctx_for(case)
    out = torch.empty_like(q)
    from servelab_b200.ops import kernels as kernels_module
    want = case.reference(window=window or None)
    plain = run_generic(case, window=window)
    # the tcgen05 kernel (head sizes 64 and 128) and the mma.sync kernel (every head size)
    for use_tc in (True, False):
        kernels_module.use_tc_prefill = use_tc
        try:
            out = torch.full_like(q, 3.0)
            K().prefill_attention(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), window)
            assert K().prefill_attention_tc_status(D, reset=True) == 0, "a bounded wait gave up"
            assert (out.float().cpu() - want).abs().max() <= TOL["bfloat16"], f"tcgen05={use_tc}"
            assert (out.float().cpu() - plain).abs().max() <= TOL["bfloat16"], f"tcgen05={use_tc}"
        finally:
            kernels_module.use_tc_prefill = True


def test_prefill_attention_tcgen05_many_launches_of_a_long_prompt():
    """A 2,048-token prompt at the 7B head layout, 300 launches back to back with matrix
    products between them: 137,000 blocks whose roles (loader, MMA issuer, softmax
    warps) run ahead of one another by different amounts.  No bounded wait may give up
    (a barrier that wraps past a waiter shows as a status word, and as a test that takes
    seconds), and every launch gives the result of the mma.sync kernel."""
    from servelab_b200.ops import kernels as kernels_module
    H, Hkv, D, ps = 28, 4, 128, 16
    case = PagedCase([2048], [2048], H, Hkv, D, ps, torch.bfloat16, seed=5)
    case.scatter()
    ctx, q, table = _ctx_for(case)
    kernels_module.use_tc_prefill = False
    try:
        want = torch.empty_like(q)
        K().prefill_attention(ctx, q, case.kc, case.vc, want, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    finally:
        kernels_module.use_tc_prefill = True
    a = torch.randn(2048, 1024, device=DEV).bfloat16()
    b = torch.randn(1024, 3584, device=DEV).bfloat16()
    outs = [torch.empty_like(q) for _ in range(4)]
    worst = 0.0
    for i in range(300):
        out = outs[i % 4]
        if i % 3 == 0:
            torch.mm(a, b)
        K().prefill_attention(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
        if i % 50 == 49:
            assert K().prefill_attention_tc_status(D, reset=True) == 0, \
                f"a bounded wait gave up: {K().prefill_attention_tc_where(D)}"
            for o in outs:
                worst = max(worst, (o.float() - want.float()).abs().max().item())
    assert worst <= TOL["bfloat16"]


@pytest.mark.parametrize("H,Hkv,D,ps", [(6, 2, 16, 16), (7, 1, 64, 8), (4, 2, 48, 4),
                                        (28, 4, 128, 16), (2, 1, 256, 32), (20, 1, 32, 16)])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("splits", [1, 3, 32])
def test_decode_attention_tensor_cores(H, Hkv, D, ps, window, splits):
    from servelab_b200.ops import library as L
    ctxs = [1, 63, 64, 65, 700, 2049, 17]
    case = PagedCase(ctxs, [1] * len(ctxs), H, Hkv, D, ps, torch.bfloat16, seed=D + splits)
    case.scatter()
    ctx, q, table = _ctx_for(case)
    out = torch.full_like(q, 7.0)
    lib = L.attention(D)
    S = len(ctxs)
    scratch = torch.full((max(1, lib.slb_decode_attention_scratch_bytes(S, H, splits) // 4),),
                         float("nan"), device=DEV)
    L.check(lib.slb_decode_attention_bf16(
        q.data_ptr(), q.stride(0), case.kc.data_ptr(), case.vc.data_ptr(), out.data_ptr(),
        out.stride(0), table.data_ptr(), table.shape[1], ctx.ctx_len.data_ptr(),
        scratch.data_ptr(), S, H, Hkv, ps, case.kc.shape[0], 1 / math.sqrt(D), window, splits,
        torch.cuda.current_stream().cuda_stream), "decode")
    want = case.reference(window=window or None)
    assert K().attention_status(D, reset=True) == 0, "a bounded wait in the kernel gave up"
    assert (out.float().cpu() - want).abs().max() <= TOL["bfloat16"]
    # the dispatching wrapper (its own choice of splits) gives the same
    out2 = torch.empty_like(q)
    K().decode_attention(ctx, q, case.kc, case.vc, out2, table, H, Hkv, D, ps, 1 / math.sqrt(D), window)
    assert (out2.float().cpu() - want).abs().max() <= TOL["bfloat16"]


@pytest.mark.parametrize("H,Hkv,D,ps", [(7, 1, 64, 8), (28, 4, 128, 16), (2, 1, 256, 32),
                                        (20, 1, 64, 16), (16, 1, 192, 64), (9, 1, 128, 128),
                                        (24, 3, 64, 256), (48, 2, 128, 16),
                                        (6, 2, 16, 16), (4, 2, 48, 4), (16, 1, 80, 5)])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("splits,stages,coef,unsplit", [(1, 3, 0.8, 12), (3, 2, 0.0, 0), (32, 4, 0.0, 0),
                                                        (5, 3, 0.8, 12), (32, 3, 0.8, 2), (32, 3, 3.0, 0)])
def test_decode_attention_one_launch(H, Hkv, D, ps, window, splits, stages, coef, unsplit):
    """The producer/consumer decode kernel whose last block combines the splits:
    every group size (8 and 16 head rows a block, several head tiles), pages smaller
    and larger than a key tile, ring depths, more splits than tiles, requests that use
    fewer splits than were launched (each by its own length); twice in a row, so the
    arrival counters came back to 0.  Sizes it refuses reach the earlier
    kernel through the wrapper."""
    from servelab_b200.ops import library as L
    ctxs = [1, 63, 64, 65, 700, 2049, 17]
    case = PagedCase(ctxs, [1] * len(ctxs), H, Hkv, D, ps, torch.bfloat16, seed=D + splits)
    case.scatter()
    ctx, q, table = _ctx_for(case)
    lib = L.attention(D)
    if not lib.slb_decode_attention_ws_supported(ps):
        assert D % 64 or ps < 8 or ps & (ps - 1)
        out = torch.empty_like(q)
        K().decode_attention(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), window)
        assert (out.float().cpu() - case.reference(window=window or None)).abs().max() <= TOL["bfloat16"]
        return
    S = len(ctxs)
    want = case.reference(window=window or None)
    counters = torch.zeros(int(lib.slb_decode_attention_ws_counters(S, H, Hkv)), dtype=torch.int32,
                           device=DEV)
    # twice through global scratch and the arrival counters, then twice with the splits of a
    # request as thread-block clusters: up to eight splits one cluster, which needs neither;
    # beyond, several clusters a request, whose results meet in the scratch slice by slice
    most = lib.slb_decode_attention_ws_max_cluster_splits()
    for cluster in (0, 0, 1, 1):
        if cluster and splits > most and splits % most:
            continue
        bare = cluster and splits <= most
        out = torch.full_like(q, 7.0)
        scratch = torch.full((max(1, lib.slb_decode_attention_ws_scratch_bytes(S, H, splits) // 4),),
                             float("nan"), device=DEV)
        L.check(lib.slb_decode_attention_ws_bf16(
            q.data_ptr(), q.stride(0), case.kc.data_ptr(), case.vc.data_ptr(), out.data_ptr(),
            out.stride(0), table.data_ptr(), table.shape[1], ctx.ctx_len.data_ptr(),
            None if bare else scratch.data_ptr(), None if bare else counters.data_ptr(), S, H, Hkv, ps,
            case.kc.shape[0], 1 / math.sqrt(D), window, splits, stages, coef, unsplit, cluster,
            torch.cuda.current_stream().cuda_stream), "decode")
        assert K().decode_attention_status(D, reset=True) == 0, "a bounded wait in the kernel gave up"
        assert (out.float().cpu() - want).abs().max() <= TOL["bfloat16"], f"cluster={cluster}"
        assert int(counters.abs().sum()) == 0
    # the dispatching wrapper (its own choice of splits) and the earlier two-kernel form
    for fn in (K().decode_attention, K().decode_attention_split):
        out2 = torch.empty_like(q)
        fn(ctx, q, case.kc, case.vc, out2, table, H, Hkv, D, ps, 1 / math.sqrt(D), window)
        assert (out2.float().cpu() - want).abs().max() <= TOL["bfloat16"]


@pytest.mark.parametrize("ctxs", [[9000], [9000, 3000, 130], [20000, 70], [1500, 1400, 1300, 1200, 1100]])
@pytest.mark.parametrize("H,Hkv,D", [(28, 4, 128), (8, 1, 64)])
def test_decode_attention_of_few_long_requests_uses_several_clusters(ctxs, H, Hkv, D):
    """Few requests with long contexts: the wrapper launches more splits than a cluster holds,
    every cluster leaves a partial result and the last block of each slice combines them; one
    far key is made to dominate a head, so a group whose result were dropped would show.  Twice,
    bit for bit the same (the counters came back to zero)."""
    from servelab_b200.ops import kernels as kernels_module
    ps = 16
    case = PagedCase(ctxs, [1] * len(ctxs), H, Hkv, D, ps, torch.bfloat16, seed=len(ctxs) + D)
    g = H // Hkv
    for i, c in enumerate(ctxs):                            # a key that the first head of each group
        for kvh in range(Hkv):                              # attends to alone, at a different depth each
            far = (kvh + 1) * c // (Hkv + 2)
            case.k[i][far, kvh] = (4.0 * case.q[i][0, kvh * g].float()).to(torch.bfloat16)
            case.v[i][far, kvh] = 5.0
    case.scatter()
    ctx, q, table = _ctx_for(case)
    want = case.reference()
    assert float(want.view(len(ctxs), H, D)[:, ::g].min()) > 4.0       # those heads see that key only
    K().decode_attention_splits_used(D, reset=True)
    out = torch.full_like(q, 7.0)
    K().decode_attention(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    assert K().decode_attention_status(D, reset=True) == 0
    used = K().decode_attention_splits_used(D, reset=True)
    if max(ctxs) >= 9000:
        assert used > 8, used                               # more than one cluster for the long request
    assert (out.float().cpu() - want).abs().max() <= TOL["bfloat16"]
    again = torch.full_like(q, 3.0)
    K().decode_attention(ctx, q, case.kc, case.vc, again, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    assert torch.equal(again, out)
    buf = kernels_module._decode_counters.get(torch.cuda.current_device())
    assert buf is None or int(buf.abs().sum()) == 0


def test_decode_attention_many_launches_of_a_mixed_batch():
    """48 requests of very different lengths at the 7B head layout, 300 launches back to
    back with matrix products between them (producer and consumers, blocks that leave at
    once, last blocks that combine: every role runs ahead or behind by different amounts
    from launch to launch).  No bounded wait may give up, the arrival counters are zero
    again, and every launch gives bit for bit the result of the first."""
    from servelab_b200.ops import kernels as kernels_module
    H, Hkv, D, ps = 28, 4, 128, 16
    g = torch.Generator().manual_seed(3)
    ctxs = [int(x) for x in torch.randint(1, 3000, (48,), generator=g)] + [1, 64, 65, 4096]
    case = PagedCase(ctxs, [1] * len(ctxs), H, Hkv, D, ps, torch.bfloat16, seed=9)
    case.scatter()
    ctx, q, table = _ctx_for(case)
    want = case.reference()
    a = torch.randn(512, 1024, device=DEV).bfloat16()
    b = torch.randn(1024, 2048, device=DEV).bfloat16()
    first = torch.empty_like(q)
    K().decode_attention(ctx, q, case.kc, case.vc, first, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    assert (first.float().cpu() - want).abs().max() <= TOL["bfloat16"]
    outs = [torch.empty_like(q) for _ in range(4)]
    for i in range(300):
        if i % 3 == 0:
            torch.mm(a, b)
        K().decode_attention(ctx, q, case.kc, case.vc, outs[i % 4], table, H, Hkv, D, ps,
                             1 / math.sqrt(D), 0)
        if i % 60 == 59:
            assert K().decode_attention_status(D, reset=True) == 0, "a bounded wait gave up"
            assert all(torch.equal(o, first) for o in outs)
    assert all(int(c.abs().sum()) == 0 for c in kernels_module._decode_counters.values())


@pytest.mark.parametrize("H,Hkv,D,ps", [(14, 2, 128, 16), (6, 3, 32, 8), (8, 1, 64, 64)])
@pytest.mark.parametrize("window", [1, 7, 64, 65, 200])
def test_fast_attention_window_edges(H, Hkv, D, ps, window):
    """The key just outside the window of the last query would take all the weight if it
    were visible (the key just inside must be seen): prompt portions through both prefill
    kernels, single tokens through both decode kernels; windows below, at and above the
    64-key tile."""
    from servelab_b200.ops import kernels as kernels_module
    for q_lens in ([23, 1, 64, 5], [1, 1, 1, 1]):
        ctxs = [90, 341, 64, 700]
        case = PagedCase(ctxs, q_lens, H, Hkv, D, ps, torch.bfloat16, seed=window + D)
        for q, k, c in zip(case.q, case.k, case.ctx_lens):
            a = c - 1                                        # the last query's position
            if a - window >= 0:
                k[a - window] = (q[-1].float().view(Hkv, H // Hkv, D).mean(1) * 50).to(k.dtype)
        case.scatter()
        ctx, q, table = _ctx_for(case)
        want, full = case.reference(window=window), case.reference()
        assert (want - full).abs().max() > 1e-2              # the window does change the result
        if all(n == 1 for n in q_lens):
            runs = [K().decode_attention, K().decode_attention_split]
        else:
            def tc(*a):
                kernels_module.use_tc_prefill = True
                K().prefill_attention(*a)

            def mma(*a):
                kernels_module.use_tc_prefill = False
                try:
                    K().prefill_attention(*a)
                finally:
                    kernels_module.use_tc_prefill = True
            runs = [tc, mma]
        for fn in runs:
            out = torch.full_like(q, 5.0)
            fn(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), window)
            assert (out.float().cpu() - want).abs().max() <= TOL["bfloat16"], (fn, q_lens)
    assert K().prefill_attention_tc_status(D, reset=True) == 0
    assert K().decode_attention_status(D, reset=True) == 0
    assert K().attention_status(D, reset=True) == 0


@pytest.mark.parametrize("needle", [0, 63, 64, 1023, 1024, 1500])
def test_fast_attention_finds_one_far_key(needle):
    H, Hkv, D, ps = 14, 2, 128, 16
    for q_len in (1, 5):
        case = PagedCase([1501], [q_len], H, Hkv, D, ps, torch.bfloat16, seed=needle)
        for kvh in range(Hkv):
            qdir = case.q[0][-1, kvh * 7].float()
            case.k[0][needle, kvh] = (qdir * 60 / qdir.norm()).to(case.dt)
            for h in range(7):
                case.q[0][-1, kvh * 7 + h] = case.q[0][-1, kvh * 7]
        case.q[0] = (case.q[0].float() * 8).to(case.dt)
        case.scatter()
        ctx, q, table = _ctx_for(case)
        out = torch.empty_like(q)
        fn = K().decode_attention if q_len == 1 else K().prefill_attention
        fn(ctx, q, case.kc, case.vc, out, table, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
        got = out.float().cpu().view(q_len, H, D)[-1]
        for h in range(H):
            assert (got[h] - case.v[0][needle, h // 7].float()).abs().max() <= 3e-2


# ------------------------------------------------- weight-streaming product
@pytest.mark.parametrize("D", [48, 64])
def test_block_table_entries_outside_the_cache_are_skipped_and_reported(D):
    """A block table can only be wrong through a fault of the host side; the kernels then skip
    the page (no write, keys read as zeros) and set a status word instead of touching memory
    outside the pool.  Request 1's second page is given as num_pages + 3; request 0 must come
    out exactly as without the fault.  Head size 48 takes the mma.sync kernels, 64 the TMA ones."""
    H, Hkv, ps = 4, 2, 8
    dt = torch.bfloat16
    k = K()
    case = PagedCase([40, 30], [1, 1], H, Hkv, D, ps, dt, seed=D)
    case.scatter()
    num_pages = case.kc.shape[0]
    ctx, q, table = _ctx_for(case)
    bad = table.clone()
    bad[1, 1] = num_pages + 3
    want = case.reference()

    def check(out, what):
        assert torch.isfinite(out.float()).all(), what
        assert (out.float().cpu()[0] - want[0]).abs().max() <= TOL["bfloat16"], what

    # plain attention (float32 arithmetic on bfloat16 data)
    tile_seq, tile_row0, n = ctx.attention_tiles(H // Hkv, k.generic_attention_tile_rows())
    out = torch.empty_like(q)
    k.generic_attention_status(reset=True)
    k.paged_attention_generic(q, case.kc, case.vc, out, bad, ctx.cu_q, ctx.ctx_len, tile_seq, tile_row0,
                              n, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    assert k.generic_attention_status(reset=True) == 1
    check(out, "generic")
    # decode kernels: the one-launch kernel where the head size allows it, else the split form
    for fn, status in ((k.decode_attention, k.decode_attention_status if k.decode_attention_takes(D, ps)
                        else k.attention_status), (k.decode_attention_split, k.attention_status)):
        status(D, reset=True)
        out = torch.empty_like(q)
        fn(ctx, q, case.kc, case.vc, out, bad, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
        assert status(D, reset=True) == 0x40, fn.__name__
        check(out, fn.__name__)
    # prefill kernels (request 1 as a 2-token portion)
    pcase = PagedCase([40, 30], [1, 2], H, Hkv, D, ps, dt, seed=D)
    pcase.scatter()
    pctx, pq, ptable = _ctx_for(pcase)
    pbad = ptable.clone()
    pbad[1, 1] = num_pages + 3
    out = torch.empty_like(pq)
    k.prefill_attention(pctx, pq, pcase.kc, pcase.vc, out, pbad, H, Hkv, D, ps, 1 / math.sqrt(D), 0)
    assert torch.isfinite(out.float()).all()
    assert (out.float().cpu()[0] - pcase.reference()[0]).abs().max() <= TOL["bfloat16"]
    if D == 48:
        assert k.attention_status(D, reset=True) == 0x40
    # the q/k/v kernel: token 1 (request 1, position 9, second page) is not written
    kc, vc = _paged(num_pages, Hkv, ps, D, dt)
    qkv = torch.randn(2, (H + 2 * Hkv) * D, device=DEV).to(dt)
    q_out = torch.empty(2, H * D, device=DEV, dtype=dt)
    k.cache_write_status(reset=True)
    k.qkv_rope_cache(qkv, None, i32([3, 9]), i32([0, 1]), bad, ps, None, 0, q_out, kc, vc, H, Hkv, D)
    assert k.cache_write_status(reset=True) == 1
    page0 = int(bad[0, 0])
    assert float(kc[page0, :, 3].abs().max()) > 0, "the token with a good page is written"
    kc[page0, :, 3] = 0
    vc[page0, :, 3] = 0
    assert float(kc.abs().max()) == 0 and float(vc.abs().max()) == 0, "nothing else is written"


@pytest.mark.parametrize("M", [1, 5, 16, 17, 33, 64])
@pytest.mark.parametrize("N,Kd,splits", [(3584, 3584, 0), (4608, 3584, 4), (37888, 1024, 1),
                                         (1000, 152, 1), (24, 18944, 0), (300, 4096, 16)])
def test_gemm_tcgen05_decode(M, N, Kd, splits):
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV)
    want = (x.double() @ w.double().t() + b.double()).float()
    o32 = torch.full((M, N), 9.0, device=DEV)
    K().gemm_tc_decode(x, w, o32, b, splits)
    assert K().gemm_tc_status(True) == 0, "a bounded wait in the kernel ran out"
    assert (o32 - want).abs().max() <= 2e-3
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().gemm_tc_decode(x, w, ob, None, splits)
    assert (ob.float() - (want - b)).abs().max() <= 2e-2
    again = torch.empty(M, N, device=DEV)
    K().gemm_tc_decode(x, w, again, b, splits)
    assert torch.equal(again, o32)                          # deterministic
    if M >= 2:                                              # a token does not depend on its neighbours
        x2 = x.clone()
        x2[0] = 0
        other = torch.empty(M, N, device=DEV)
        K().gemm_tc_decode(x2, w, other, b, splits)
        assert torch.equal(other[1:], o32[1:])
    assert K().gemm_tc_status(True) == 0


@pytest.mark.parametrize("M", [1, 5, 8, 16, 17, 64])
@pytest.mark.parametrize("N,Kd,splits", [(3584, 3584, 0), (4608, 3584, 8), (3584, 18944, 0), (1000, 152, 1),
                                         (24, 18944, 7), (300, 4096, 3), (896, 4864, 0)])
def test_gemm_tcgen05_cluster(M, N, Kd, splits):
    """The K splits of a row tile as a thread-block cluster that adds its results up
    through shared memory: against float64, bit for bit the same on a second launch, a
    token independent of its neighbours, more tokens than ranks and fewer."""
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) / math.sqrt(Kd)).bfloat16()
    b = torch.randn(N, device=DEV)
    want = (x.double() @ w.double().t() + b.double()).float()
    out = torch.full((M, N), 9.0, device=DEV, dtype=torch.bfloat16)
    K().gemm_tc_cluster(x, w, out, b, splits)
    assert K().gemm_tc_status(True) == 0, "a bounded wait in the kernel ran out"
    assert (out.float() - want).abs().max() <= 2e-2
    again = torch.empty_like(out)
    K().gemm_tc_cluster(x, w, again, b, splits)
    assert torch.equal(again, out)
    nobias = K().gemm_tc_cluster(x, w, None, None, splits)
    assert (nobias.float() - (want - b)).abs().max() <= 2e-2
    if M >= 2:
        x2 = x.clone()
        x2[0] = 0
        other = K().gemm_tc_cluster(x2, w, None, b, splits)
        assert torch.equal(other[1:], out[1:])
    assert K().gemm_tc_status(True) == 0


@pytest.mark.parametrize("M", [1, 3, 8, 16, 23, 64])
@pytest.mark.parametrize("N,Kd,splits", [(3584, 3584, 0), (3584, 18944, 0), (896, 4864, 0), (1000, 152, 2),
                                         (24, 1024, 7), (300, 4096, 3)])
def test_gemm_tcgen05_product_with_residual_add_and_norm(M, N, Kd, splits):
    """The product that closes a residual branch, with the add and the RMS norm in its epilogue
    (the rows are left without 1 / rms), and the products that apply that factor afterwards:
    the stream, the normed rows and the three kinds of consumer against float64; one row of the
    stream is made a thousand times larger than the others, so a factor taken from a
    neighbour's row would show."""
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, Kd, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).bfloat16().to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    resid0 = torch.randn(M, N, generator=g).to(DEV)
    resid0[M // 2] *= 1000.0
    nw = (1.0 + 0.3 * torch.randn(N, generator=g)).to(DEV)
    eps = 1e-5
    want_resid = resid0.double() + x.double() @ w.double().t() + b.double()
    rstd = torch.rsqrt((want_resid * want_resid).mean(-1, keepdim=True) + eps)
    want_normed = want_resid * rstd * nw.double()
    resid = resid0.clone()
    rows = K().gemm_tc_resid_norm(x, w, b, resid, nw, eps, splits)
    assert K().gemm_tc_status(True) == 0, "a bounded wait in the kernel ran out"
    scale = want_resid.abs().amax(-1, keepdim=True).float()
    assert ((resid - want_resid.float()).abs() / scale).max() <= 1e-5
    assert torch.equal(rows.resid, resid) and rows.sumsq.shape == (M, (N + 127) // 128)
    ss = rows.sumsq.double().sum(1)
    assert ((ss - (want_resid * want_resid).sum(-1)).abs() / ss).max() <= 1e-5
    # the plain form: the norm kernel on the updated stream
    plain = rows.materialize()
    assert (plain.float() - want_normed.float()).abs().max() <= 4e-2
    # z is resid * weight in bfloat16
    assert ((rows.z.float() - (want_resid * nw.double()).float()).abs() / scale).max() <= 8e-3
    again = resid0.clone()
    rows2 = K().gemm_tc_resid_norm(x, w, b, again, nw, eps, splits)
    assert torch.equal(again, resid) and torch.equal(rows2.z, rows.z) and torch.equal(rows2.sumsq, rows.sumsq)
    # consumers: they must give what the product of the normed rows gives
    N2 = 256
    w2 = (torch.randn(N2, N, generator=g) / math.sqrt(N)).bfloat16().to(DEV)
    b2 = torch.randn(N2, generator=g).to(DEV)
    zn = rows.z.double() * rstd                             # what the consumer multiplies, exactly
    want2 = (zn @ w2.double().t() + b2.double()).float()
    if N % 8 == 0:
        two = 2 if N > 64 else 1                            # K splits cannot outnumber the k-blocks
        got = K().gemm_tc_cluster(rows, w2, None, b2, two)
        assert (got.float() - want2).abs().max() <= 3e-2
        got = torch.empty(M, N2, device=DEV)
        K().gemm_tc_decode(rows, w2, got, b2, 1)
        assert (got - want2).abs().max() <= 2e-3
        got = torch.empty(M, N2, device=DEV)
        K().gemm_tc_decode(rows, w2, got, b2, two)
        assert (got - want2).abs().max() <= 2e-3
        act = K().gemm_tc_decode(rows, w2, None, splits=1, swiglu=True)
        y = (zn @ w2.double().t()).float().view(M, N2 // 128, 2, 64)
        want_act = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, N2 // 2)
        assert (act.float() - want_act).abs().max() <= 3e-2
        # q|k|v with rotation: one head of 128 and two of keys / values ... against the plain rows
        H, Hkv, D, ps = 1, 1, 64, 4
        w3 = (torch.randn((H + 2 * Hkv) * D, N, generator=g) / math.sqrt(N)).bfloat16().to(DEV)
        positions = i32(list(range(M)))
        seq = i32([0] * M)
        table = i32([list(range((M + ps - 1) // ps))])
        inv = P.rope_inv_freq(D, 10000.0).to(DEV)
        q = torch.empty(M, H * D, device=DEV, dtype=torch.bfloat16)
        kc, vc = _paged((M + ps - 1) // ps, Hkv, ps, D, torch.bfloat16)
        K().gemm_tc_qkv_rope(rows, w3, None, positions, seq, table, ps, inv, D, q, kc, vc, H, Hkv, D, two)
        y3 = (zn @ w3.double().t()).float().cpu()
        qf = P.rope(y3[:, :D].view(M, 1, D), torch.arange(M), inv.cpu())
        assert (q.float().cpu().view(M, 1, D) - qf).abs().max() <= 3e-2
        vf = y3[:, 2 * D:]
        for t in range(M):
            assert (vc[t // ps, 0, t % ps].float().cpu() - vf[t]).abs().max() <= 3e-2
    assert K().gemm_tc_status(True) == 0


@pytest.mark.parametrize("M", [8, 16, 40])
def test_cluster_products_of_a_layer_launched_back_to_back_many_times(M):
    """The products of a decode layer one after the other, 150 times, with programmatic dependent
    launch: blocks of the next product become resident and fill their shared memory while the
    blocks of a cluster still read one another's (the closing barrier of a cluster arrives
    relaxed, after the remote values have been used).  Every round must give bit for bit the
    result of the first; no bounded wait may give up."""
    h, Hq, Hkv, D, inter, ps = 1024, 8, 2, 128, 2816, 16
    g = torch.Generator().manual_seed(M)
    def w(n, k):
        return (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16().to(DEV)
    w_qkv, w_o, w_gu, w_down = w((Hq + 2 * Hkv) * D, h), w(h, Hq * D), w(2 * inter, h), w(h, inter)
    bias = torch.randn((Hq + 2 * Hkv) * D, generator=g).to(DEV)
    nw = (1.0 + 0.1 * torch.randn(h, generator=g)).to(DEV)
    inv = P.rope_inv_freq(D, 10000.0).to(DEV)
    x0 = torch.randn(M, h, generator=g).bfloat16().to(DEV)
    attn = torch.randn(M, Hq * D, generator=g).bfloat16().to(DEV)
    resid0 = torch.randn(M, h, generator=g).to(DEV)
    positions, seq = i32(list(range(100, 100 + M))), i32([0] * M)
    pages = (100 + M) // ps + 1
    table = i32([list(range(pages))])
    first = None
    for it in range(150):
        resid = resid0.clone()
        q = torch.empty(M, Hq * D, device=DEV, dtype=torch.bfloat16)
        kc, vc = _paged(pages, Hkv, ps, D, torch.bfloat16)
        K().gemm_tc_qkv_rope(x0, w_qkv, bias, positions, seq, table, ps, inv, D, q, kc, vc, Hq, Hkv, D)
        rows = K().gemm_tc_resid_norm(attn, w_o, None, resid, nw, 1e-6)
        act = K().gemm_tc_decode(rows, w_gu, None, splits=1, swiglu=True)
        rows2 = K().gemm_tc_resid_norm(act, w_down, None, resid, nw, 1e-6)
        out = K().gemm_tc_cluster(rows2, w_qkv, None, bias)
        got = (q, kc, rows.z, rows.sumsq, act, rows2.z, rows2.sumsq, resid, out)
        if first is None:
            first = [t.clone() for t in got]
            assert all(bool(torch.isfinite(t.float()).all()) for t in first)
        elif it % 10 == 9 or it < 5:
            for a, b in zip(got, first):
                assert torch.equal(a, b), f"round {it}"
    assert K().gemm_tc_status(True) == 0


@pytest.mark.parametrize("H,Hkv,D,rot,hidden", [(28, 4, 128, 128, 3584), (14, 2, 64, 64, 896),
                                                (6, 2, 64, 32, 72), (5, 1, 32, 32, 160),
                                                (3, 3, 16, 0, 64), (9, 1, 128, 64, 1024)])
@pytest.mark.parametrize("M", [1, 8, 13, 64])
def test_gemm_tcgen05_qkv_with_rotation_and_cache_write(H, Hkv, D, rot, hidden, M):
    """The q|k|v product whose epilogue adds the bias, rotates and writes the cache, against
    the library-free path it replaces (product, then the q/k/v kernel) and against float32
    arithmetic: tokens of two requests at scattered positions, partial and no rotation, a
    run that writes no cache."""
    ps = 4
    g = torch.Generator().manual_seed(M + D)
    positions = torch.randperm(max(M, 40), generator=g)[:M].tolist()   # distinct: a slot per token
    seq = [t % 2 for t in range(M)]
    pages = max(positions) // ps + 1
    perm = torch.randperm(2 * pages, generator=g).tolist()
    table = i32([perm[:pages], perm[pages:]])
    width = (H + 2 * Hkv) * D
    x = torch.randn(M, hidden, generator=g).bfloat16().to(DEV)
    w = (torch.randn(width, hidden, generator=g) / math.sqrt(hidden)).bfloat16().to(DEV)
    bias = torch.randn(width, generator=g).to(DEV)
    inv = P.rope_inv_freq(rot, 10000.0).to(DEV) if rot else None
    # float32 arithmetic
    y = (x.double() @ w.double().t()).float() + bias
    qf = y[:, :H * D].view(M, H, D).cpu()
    kf = y[:, H * D:(H + Hkv) * D].view(M, Hkv, D).cpu()
    vf = y[:, (H + Hkv) * D:].view(M, Hkv, D).cpu()
    pos_t = torch.tensor(positions)
    if rot:
        qf = torch.cat([P.rope(qf[..., :rot], pos_t, inv.cpu()), qf[..., rot:]], -1)
        kf = torch.cat([P.rope(kf[..., :rot], pos_t, inv.cpu()), kf[..., rot:]], -1)
    q = torch.full((M, H * D), 7.0, device=DEV, dtype=torch.bfloat16)
    kc, vc = _paged(2 * pages, Hkv, ps, D, torch.bfloat16)
    K().gemm_tc_qkv_rope(x, w, bias, i32(positions), i32(seq), table, ps, inv, rot, q, kc, vc, H, Hkv, D)
    assert K().gemm_tc_status(True) == 0, "a bounded wait in the kernel ran out"
    tol = 3e-2
    assert (q.float().cpu().view(M, H, D) - qf).abs().max() <= tol
    tab = table.cpu()
    written = set()
    for t in range(M):
        page = int(tab[seq[t], positions[t] // ps])
        written.add((page, positions[t] % ps))
        assert (kc[page, :, positions[t] % ps].float().cpu() - kf[t]).abs().max() <= tol
        assert (vc[page, :, positions[t] % ps].float().cpu() - vf[t]).abs().max() <= tol
    for page in range(2 * pages):                            # no other slot is touched
        for slot in range(ps):
            if (page, slot) not in written:
                assert float(kc[page, :, slot].abs().max()) == 0 and float(vc[page, :, slot].abs().max()) == 0
    # the two-kernel path gives the same to a bfloat16 step (it rounds the product first)
    q2 = torch.empty_like(q)
    kc2, vc2 = _paged(2 * pages, Hkv, ps, D, torch.bfloat16)
    mid = K().gemm_tc_cluster(x, w, None, None)
    K().qkv_rope_cache(mid, bias, i32(positions), i32(seq), table, ps, inv, rot, q2, kc2, vc2, H, Hkv, D)
    assert (q2.float() - q.float()).abs().max() <= 2 * tol
    assert (kc2.float() - kc.float()).abs().max() <= 2 * tol
    # a run that reads another run's cache writes none
    q3 = torch.empty_like(q)
    kc3, vc3 = _paged(2 * pages, Hkv, ps, D, torch.bfloat16)
    K().gemm_tc_qkv_rope(x, w, bias, i32(positions), i32(seq), table, ps, inv, rot, q3, None, None, H, Hkv, D)
    assert torch.equal(q3, q) and float(kc3.abs().max()) == 0
    assert K().gemm_tc_status(True) == 0


def test_kernel_bench_program_runs_on_small_cases(capsys):
    """The microbenchmark module end to end on its smallest cases: every group, a table
    with one row per case, status words all zero (exit code 0)."""
    from servelab_b200.bench import kernel_bench
    rc = kernel_bench.main(["--shape", "qwen2.5-0.5b", "--batches", "2", "--contexts", "130",
                            "--prefill-lengths", "70", "--tokens", "3", "--markdown"])
    out = capsys.readouterr().out
    assert rc == 0, out
    for name in ("decode attention (one launch)", "prefill attention (tcgen05)", "q|k|v product",
                 "LM head", "residual add + RMSNorm", "SwiGLU", "sampler"):
        assert name in out, name

"""The reference's own GPU kernels beside this package's, on the same data.

The reference project cannot generate a token here (its engine imports a model package that
its tree does not contain), but its two Triton kernels import on their own:
``paged_decode_attention_triton`` and ``rmsnorm_triton``
(servelab/attention/triton/paged_attention.py:94-134).  This module calls them unmodified,
through those wrapper functions, from an installed copy of the reference (``baseline/_ref``
beside the repository root, or any folder on ``sys.path`` that holds ``servelab``), at the
sizes of the reference's own kernel benchmark (servelab/bench/kernel_bench.py:26-27,73:
32 requests x 32 / 8 heads, 1,024 keys each, head size 128, pages of 16; RMSNorm of 4,096 rows
of 4,096), and times this package's kernels on the same values.

Timing: CUDA events around ``iters`` launches after warm-up, as the reference's benchmark
does (kernel_bench.py:12-23), but every launch works on the next of several copies of the
data, so that together they exceed the L2 cache and no launch is served from it.

Layouts differ and are converted before the clock starts: the reference keeps rows
[page * page_size + slot, kv head, D]; this package keeps [page, kv head, slot, D].  The
reference's RMSNorm reads and writes 16-bit rows; this package's norm reads the float32
residual stream and writes 16-bit rows (more bytes for the same rows), so both the time and
the bytes each moved are reported.
"""

from __future__ import annotations

import math
import os
import sys
from typing import Dict, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def import_reference():
    """(module with the two wrappers, None) or (None, why not)."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref, "servelab")) and ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        from servelab.attention.triton import paged_attention as mod
    except Exception as e:                                  # noqa: BLE001 (reported, not hidden)
        return None, f"{type(e).__name__}: {e}"
    if not getattr(mod, "HAS_TRITON", False):
        return None, "the reference reports that Triton is not importable"
    return mod, None


def reference_engine_error() -> str:
    """What importing the reference's engine raises here (its public entry point)."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref, "servelab")) and ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import servelab.engine.engine  # noqa: F401
    except Exception as e:                                  # noqa: BLE001
        return f"{type(e).__name__}: {e}"
    return ""


def _time(launch, copies: int, warmup: int = 10, iters: int = 50) -> float:
    """Microseconds per launch; ``launch(i)`` works on copy i % copies."""
    import torch
    for i in range(warmup):
        launch(i % copies)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iters):
        launch(i % copies)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def compare(device: str = "cuda:0", batch: int = 32, ctx: int = 1024, heads: int = 32,
            kv_heads: int = 8, head_dim: int = 128, page: int = 16, rows: int = 4096,
            dim: int = 4096) -> Dict[str, object]:
    """Times of both arms in microseconds, the largest difference between their results, and
    the bytes each had to move.  ``{"unavailable": why}`` when the reference's kernels cannot
    be imported or run."""
    import torch
    from ..engine.batch import BatchEntry, StepContext
    from ..ops import kernels as K
    mod, why = import_reference()
    if mod is None:
        return {"unavailable": why}
    out: Dict[str, object] = {"shape": f"{batch} requests x {heads}/{kv_heads} heads, {ctx} keys, head size "
                                       f"{head_dim}, page {page}; RMSNorm {rows} x {dim}"}
    torch.manual_seed(0)
    n = ctx // page
    pages = batch * n
    copies = 4
    scale = head_dim ** -0.5
    # ---------------------------------------------------------------- paged decode attention
    try:
        tables = torch.arange(pages, dtype=torch.int32, device=device).view(batch, n)
        lens = torch.full((batch,), ctx, dtype=torch.int32, device=device)
        data = []
        for _ in range(copies):
            k = torch.randn(pages * page, kv_heads, head_dim, device=device)
            v = torch.randn(pages * page, kv_heads, head_dim, device=device)
            q = torch.randn(batch, heads, head_dim, device=device)
            data.append((q, k, v))
        kv_bytes = 2 * pages * page * kv_heads * head_dim * 2
        for name, dt in (("fp16", torch.float16), ("bf16", torch.bfloat16)):
            theirs = [(q.to(dt), k.to(dt), v.to(dt)) for q, k, v in data]
            us = _time(lambda i: mod.paged_decode_attention_triton(
                theirs[i][0], theirs[i][1], theirs[i][2], tables, lens, scale, kv_heads, page), copies)
            out[f"reference_paged_decode_{name}_us"] = round(us, 1)
            if dt == torch.bfloat16:
                ref_out = mod.paged_decode_attention_triton(theirs[0][0], theirs[0][1], theirs[0][2],
                                                            tables, lens, scale, kv_heads, page)
            del theirs
        # this package: the same values as [page, kv head, slot, D] bfloat16
        mine = []
        for q, k, v in data:
            kc = k.view(pages, page, kv_heads, head_dim).permute(0, 2, 1, 3).contiguous().bfloat16()
            vc = v.view(pages, page, kv_heads, head_dim).permute(0, 2, 1, 3).contiguous().bfloat16()
            mine.append((q.view(batch, heads * head_dim).bfloat16(), kc, vc))
        del data
        entries = [BatchEntry(tokens=[1], start=ctx - 1, want=(0,),
                              block_tables=[list(range(b * n, (b + 1) * n))], state_slot=0)
                   for b in range(batch)]
        sctx = StepContext.pack(entries, 1, device, min_table_width=n)
        o = torch.empty_like(mine[0][0])

        def ours(i):
            K.decode_attention(sctx, mine[i][0], mine[i][1], mine[i][2], o, sctx.block_tables[0],
                               heads, kv_heads, head_dim, page, scale, 0)
        us = _time(ours, copies)
        out["ours_paged_decode_bf16_us"] = round(us, 1)
        ours(0)
        torch.cuda.synchronize()
        out["paged_decode_max_abs_diff"] = round(float(
            (o.float().view(batch, heads, head_dim) - ref_out.float()).abs().max()), 5)
        out["paged_decode_kv_bytes"] = kv_bytes
        del mine
    except Exception as e:                                  # noqa: BLE001
        out["paged_decode_unavailable"] = f"{type(e).__name__}: {e}"
    torch.cuda.empty_cache()
    # -------------------------------------------------------------------------- RMSNorm
    try:
        copies = 8
        xs = [torch.randn(rows, dim, device=device) for _ in range(copies)]
        w = torch.randn(dim, device=device)
        for name, dt in (("fp16", torch.float16), ("bf16", torch.bfloat16)):
            theirs = [x.to(dt) for x in xs]
            wd = w.to(dt)
            us = _time(lambda i: mod.rmsnorm_triton(theirs[i], wd, 1e-6), copies)
            out[f"reference_rmsnorm_{name}_us"] = round(us, 1)
            if dt == torch.bfloat16:
                ref_y = mod.rmsnorm_triton(theirs[0], wd, 1e-6)
            del theirs
        out["reference_rmsnorm_bytes"] = rows * dim * 2 * 2
        ys = [torch.empty(rows, dim, device=device, dtype=torch.bfloat16) for _ in range(copies)]
        wf = w.bfloat16().float()                            # the value the reference multiplies by

        def ours_norm(i):
            K.add_rmsnorm(xs[i], None, wf, 1e-6, ys[i])
        us = _time(ours_norm, copies)
        out["ours_rmsnorm_f32_in_bf16_out_us"] = round(us, 1)
        out["ours_rmsnorm_bytes"] = rows * dim * (4 + 2)
        ours_norm(0)
        torch.cuda.synchronize()
        # the reference normalises the 16-bit rounding of x, this package x itself
        want = xs[0].bfloat16().float()
        want = want * torch.rsqrt((want * want).mean(-1, keepdim=True) + 1e-6) * wf
        out["rmsnorm_reference_max_abs_err"] = round(float((ref_y.float() - want).abs().max()), 5)
        exact = xs[0] * torch.rsqrt((xs[0] * xs[0]).mean(-1, keepdim=True) + 1e-6) * wf
        out["rmsnorm_ours_max_abs_err"] = round(float((ys[0].float() - exact).abs().max()), 5)
    except Exception as e:                                  # noqa: BLE001
        out["rmsnorm_unavailable"] = f"{type(e).__name__}: {e}"
    return out


def main(argv: Optional[list] = None) -> int:
    import json
    print(json.dumps(compare(), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())

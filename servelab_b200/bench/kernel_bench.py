"""Kernel microbenchmarks: each hot kernel of a step alone, at the sizes of a model shape,
over batch sizes and context lengths, with what it achieves against the roofline.

    python -m servelab_b200.bench.kernel_bench                         # Qwen2.5-7B sizes
    python -m servelab_b200.bench.kernel_bench --shape qwen2.5-14b --only decode_attention
    python -m servelab_b200.bench.kernel_bench --markdown > table.md

How a kernel is timed: ``copies`` launches of it, each on buffers of its own (so that
together they exceed the L2 cache and nothing is served from it twice), are captured in
one CUDA graph; the graph is replayed a few times for warm-up and then ``iters`` times
between two CUDA events.  Inside a graph the launches follow one another as they do
in a decode step (programmatic dependent launch on), so the figure is the cost of the
kernel in a step, not its cold, isolated cost.  Bytes and flops are the algorithmic ones
(every operand once).  Peaks: the JSON file given with ``--peaks`` (``hbm_gbs``,
``bf16_tflops``), by default ``MEASURED_PEAKS.json`` beside the package's parent folder when it
exists, else 6,650 GB/s and 1,590 TFLOP/s; the header line says which were used.

``--only reference_kernels`` times the reference project's own two GPU kernels (Triton; imported
unmodified from an installed copy of the reference) beside this package's on the same data
(``bench/reference_kernels.py``).

Reference analogue: servelab/bench/kernel_bench.py:12-23 (CUDA events after warm-up),
:26-70 (paged decode attention, batch x context).
"""

from __future__ import annotations

import argparse
import json
import math
import sys
from typing import Callable, Dict, List, Optional, Tuple

import os

from . import workloads as W

# hidden, heads, kv heads, head size, intermediate, vocabulary
SHAPES = {name: (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                 c["intermediate_size"], c["vocab_size"]) for name, c in W.SHAPES.items()}
PAGE = 16
DEFAULT_PEAKS = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                             "MEASURED_PEAKS.json")


class Row:
    def __init__(self, kernel: str, case: str, us: float, nbytes: float, flops: float, peaks):
        self.kernel, self.case, self.us = kernel, case, us
        self.gbs = nbytes / us / 1e3
        self.tflops = flops / us / 1e6
        mem_us = nbytes / peaks["hbm_gbs"] / 1e3
        mma_us = flops / peaks["bf16_tflops"] / 1e6
        self.bound = "hbm" if mem_us >= mma_us else "mma"
        self.frac = max(mem_us, mma_us) / us

    def cells(self) -> List[str]:
        return [self.kernel, self.case, f"{self.us:.1f}", f"{self.gbs:.0f}", f"{self.tflops:.1f}",
                self.bound, f"{self.frac:.2f}"]


HEADER = ["kernel", "case", "us", "GB/s", "TFLOP/s", "bound", "of roofline"]


def time_in_graph(make_launches: Callable[[], Callable[[], None]], iters: int = 10) -> float:
    """Milliseconds per replay of a graph holding what ``make_launches()`` launches.
    ``make_launches`` allocates the buffers and returns the function that launches."""
    import torch
    run = make_launches()
    run()                                                  # builds libraries, warms caches
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(3):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / iters
    del graph
    torch.cuda.empty_cache()
    return ms


def copies_for(nbytes_each: float, budget: float = 6e9, least: int = 4, most: int = 28) -> int:
    """How many copies of a kernel's buffers a graph holds: enough that they exceed the
    L2 cache several times, within a few GB."""
    want = int(1.0e9 // max(nbytes_each, 1)) + 1
    fit = int(budget // max(nbytes_each, 1))
    return max(least, min(most, want, max(fit, 1)))


def _decode_context(batch: int, ctx_len: int, device: str, width: int):
    from ..engine.batch import BatchEntry, StepContext
    n = -(-ctx_len // PAGE)
    entries = [BatchEntry(tokens=[1], start=ctx_len - 1, want=(0,),
                          block_tables=[list(range(b * n, (b + 1) * n))], state_slot=0)
               for b in range(batch)]
    return StepContext.pack(entries, 1, device, min_table_width=width), n


def bench_decode_attention(shape, peaks, device, batches, contexts, twin: bool) -> List[Row]:
    import torch
    from ..ops import kernels as K
    _, H, Hkv, D, _, _ = shape
    rows = []
    for B in batches:
        for c in contexts:
            kv_bytes = B * c * Hkv * D * 2 * 2
            if kv_bytes > 24e9:
                continue
            copies = copies_for(kv_bytes)
            flops = 4.0 * B * c * H * D

            def make(fn):
                def build():
                    ctx, n = _decode_context(B, c, device, -(-c // PAGE))
                    caches = [(torch.randn(B * n, Hkv, PAGE, D, device=device).bfloat16(),
                               torch.randn(B * n, Hkv, PAGE, D, device=device).bfloat16())
                              for _ in range(copies)]
                    q = torch.randn(B, H * D, device=device).bfloat16()
                    out = torch.empty_like(q)

                    def run():
                        for kc, vc in caches:
                            fn(ctx, q, kc, vc, out, ctx.block_tables[0], H, Hkv, D, PAGE,
                               1 / math.sqrt(D), 0)
                    return run
                return build
            us = time_in_graph(make(K.decode_attention)) * 1e3 / copies
            rows.append(Row("decode attention (one launch)", f"batch {B}, context {c}", us, kv_bytes,
                            flops, peaks))
            if twin:
                us = time_in_graph(make(K.decode_attention_split)) * 1e3 / copies
                rows.append(Row("decode attention (split-KV twin)", f"batch {B}, context {c}", us,
                                kv_bytes, flops, peaks))
    return rows


def bench_prefill_attention(shape, peaks, device, lengths, twin: bool) -> List[Row]:
    import torch
    from ..engine.batch import BatchEntry, StepContext
    from ..ops import kernels as K
    _, H, Hkv, D, _, _ = shape
    rows = []
    for T in lengths:
        n = -(-T // PAGE)
        nbytes = T * H * D * 2 * 2 + T * Hkv * D * 2 * 2          # q and o, K and V once
        flops = 4.0 * (T * (T + 1) / 2) * H * D
        copies = 4

        def make(use_tc):
            def build():
                ctx = StepContext.pack([BatchEntry(tokens=[1] * T, start=0, want=(T - 1,),
                                                   block_tables=[list(range(n))], state_slot=0)],
                                       1, device)
                caches = [(torch.randn(n, Hkv, PAGE, D, device=device).bfloat16(),
                           torch.randn(n, Hkv, PAGE, D, device=device).bfloat16())
                          for _ in range(copies)]
                q = torch.randn(T, H * D, device=device).bfloat16()
                out = torch.empty_like(q)

                def run():
                    K.use_tc_prefill = use_tc
                    try:
                        for kc, vc in caches:
                            K.prefill_attention(ctx, q, kc, vc, out, ctx.block_tables[0], H, Hkv, D,
                                                PAGE, 1 / math.sqrt(D), 0)
                    finally:
                        K.use_tc_prefill = True
                return run
            return build
        us = time_in_graph(make(True)) * 1e3 / copies
        rows.append(Row("prefill attention (tcgen05)", f"{T} tokens", us, nbytes, flops, peaks))
        if twin:
            us = time_in_graph(make(False)) * 1e3 / copies
            rows.append(Row("prefill attention (mma.sync twin)", f"{T} tokens", us, nbytes, flops, peaks))
    return rows


def bench_products(shape, peaks, device, token_counts, only: Optional[List[str]] = None,
                   fused_only: bool = False) -> List[Row]:
    """The matrix products of a layer and the LM head as the engine dispatches them
    (``ops.linear``): this package's tcgen05 kernel for few tokens, the vendor GEMM above."""
    import torch
    from ..ops import kernels as K
    from ..ops.linear import gated_linear, linear
    h, H, Hkv, D, inter, vocab = shape
    products = [("q|k|v product", (H + 2 * Hkv) * D, h, "rope"), ("o product", h, H * D, "norm"),
                ("gate|up product + SwiGLU", 2 * inter, h, "swiglu"), ("down product", h, inter, "norm"),
                ("LM head", vocab, h, "f32")]
    rows = []
    if only:
        products = [p for p in products if any(o in p[0] for o in only)]
    for name, N, Kd, kind in products:
        for M in token_counts:
            if kind == "f32" and M > 64:
                continue                                   # logits are wanted for few rows
            w_bytes = N * Kd * 2
            out_cols = N // 2 if kind == "swiglu" else N
            nbytes = w_bytes + M * Kd * 2 + M * out_cols * (4 if kind == "f32" else 2)
            flops = 2.0 * M * N * Kd
            copies = copies_for(w_bytes)

            def build():
                ws = [(torch.randn(N, Kd, device=device) * 0.02).bfloat16() for _ in range(copies)]
                x = torch.randn(M, Kd, device=device).bfloat16()

                def run():
                    for w in ws:
                        if kind == "swiglu":
                            gated_linear(x, w, K.SWIGLU_BLOCK)
                        elif kind == "f32":
                            linear(x, w, out_dtype=torch.float32)
                        else:
                            y = linear(x, w, consumer=kind)
                            if isinstance(y, K.DeferredLinear):      # timed as the plain product
                                y.materialize()
                return run
            if not fused_only:
                us = time_in_graph(build) * 1e3 / copies
                rows.append(Row(name, f"{M} tokens [{N} x {Kd}]", us, nbytes, flops, peaks))
            if kind != "norm" or M > K.TC_MAX_TOKENS:
                continue
            # the product with the residual add and the RMS norm that follow it: as two kernels
            # (product, then add + norm) and as the one kernel that carries both in its epilogue
            # (float32 stream read and written, normed rows out: 10 more bytes an element)

            def build_pair(fused):
                ws = [(torch.randn(N, Kd, device=device) * 0.02).bfloat16() for _ in range(copies)]
                x = torch.randn(M, Kd, device=device).bfloat16()
                resid = torch.randn(M, N, device=device)
                weight = torch.ones(N, device=device)
                out = torch.empty(M, N, device=device, dtype=torch.bfloat16)

                def run():
                    for w in ws:
                        if fused:
                            K.gemm_tc_resid_norm(x, w, None, resid, weight, 1e-6)
                        else:
                            K.add_rmsnorm(resid, K.gemm_tc_cluster(x, w), weight, 1e-6, out)
                return run
            for fused in ((True,) if fused_only else (False, True)):
                us = time_in_graph(lambda: build_pair(fused)) * 1e3 / copies
                label = name + (" + add + norm (one kernel)" if fused else " + add + norm (two kernels)")
                rows.append(Row(label, f"{M} tokens [{N} x {Kd}]", us, nbytes + M * N * 10, flops, peaks))
    return rows


def bench_elementwise(shape, peaks, device, token_counts) -> List[Row]:
    import torch
    from ..ops import kernels as K
    h, H, Hkv, D, inter, vocab = shape
    rows = []
    for T in token_counts:
        # residual add + RMSNorm: float32 stream read and written, bfloat16 update in, rows out
        nbytes = T * h * (4 + 4 + 2 + 2)
        copies = copies_for(nbytes, least=8)

        def build_norm():
            bufs = [(torch.randn(T, h, device=device), torch.randn(T, h, device=device).bfloat16(),
                     torch.empty(T, h, device=device, dtype=torch.bfloat16)) for _ in range(copies)]
            weight = torch.ones(h, device=device)

            def run():
                for resid, delta, out in bufs:
                    K.add_rmsnorm(resid, delta, weight, 1e-6, out)
            return run
        us = time_in_graph(build_norm) * 1e3 / copies
        rows.append(Row("residual add + RMSNorm", f"{T} tokens", us, nbytes, 0.0, peaks))

        # q/k/v bias + rotation + cache write
        width = (H + 2 * Hkv) * D
        nbytes = T * width * 2 * 2
        copies = copies_for(nbytes, least=8)
        n = -(-T // PAGE)

        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))

        def build_rope():
            bufs = [(torch.randn(T, width, device=device).bfloat16(),
                     torch.empty(T, H * D, device=device, dtype=torch.bfloat16),
                     torch.zeros(n, Hkv, PAGE, D, device=device, dtype=torch.bfloat16),
                     torch.zeros(n, Hkv, PAGE, D, device=device, dtype=torch.bfloat16))
                    for _ in range(copies)]
            bias = torch.randn(width, device=device)
            pos = torch.arange(T, dtype=torch.int32, device=device)
            seq = torch.zeros(T, dtype=torch.int32, device=device)
            table = torch.arange(n, dtype=torch.int32, device=device)[None].contiguous()
            inv_d = inv.to(device)

            def run():
                for qkv, q, kc, vc in bufs:
                    K.qkv_rope_cache(qkv, bias, pos, seq, table, PAGE, inv_d, D, q, kc, vc, H, Hkv, D)
            return run
        us = time_in_graph(build_rope) * 1e3 / copies
        rows.append(Row("q/k/v bias + rotation + cache write", f"{T} tokens", us, nbytes, 0.0, peaks))

        # SwiGLU as a kernel of its own (steps of many tokens)
        nbytes = T * inter * 2 * 3
        copies = copies_for(nbytes, least=4)

        def build_act():
            bufs = [(torch.randn(T, 2 * inter, device=device).bfloat16(),
                     torch.empty(T, inter, device=device, dtype=torch.bfloat16)) for _ in range(copies)]

            def run():
                for gu, out in bufs:
                    K.swiglu(gu, out, K.SWIGLU_BLOCK)
            return run
        us = time_in_graph(build_act) * 1e3 / copies
        rows.append(Row("SwiGLU", f"{T} tokens", us, nbytes, 0.0, peaks))
    for R in (8, 64):
        nbytes = R * vocab * 4
        copies = copies_for(nbytes, least=8)

        def build_sample():
            bufs = [torch.randn(R, vocab, device=device) for _ in range(copies)]
            out = torch.empty(R, dtype=torch.int32, device=device)

            def run():
                for logits in bufs:
                    K.sample_rows(logits, out)
            return run
        us = time_in_graph(build_sample) * 1e3 / copies
        rows.append(Row("sampler (greedy rows)", f"{R} rows of {vocab}", us, nbytes, 0.0, peaks))
    return rows


GROUPS = ("decode_attention", "prefill_attention", "products", "elementwise")
EXTRA_GROUPS = ("reference_kernels",)       # only when asked for


def render(rows: List[Row], markdown: bool) -> str:
    table = [HEADER] + [r.cells() for r in rows]
    if markdown:
        lines = ["| " + " | ".join(table[0]) + " |", "|" + "---|" * len(HEADER)]
        lines += ["| " + " | ".join(r) + " |" for r in table[1:]]
        return "\n".join(lines)
    widths = [max(len(r[i]) for r in table) for i in range(len(HEADER))]
    return "\n".join("  ".join(c.ljust(w) for c, w in zip(r, widths)) for r in table)


def _ints(text: str) -> List[int]:
    return [int(v) for v in text.split(",") if v]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="qwen2.5-7b", choices=sorted(SHAPES))
    ap.add_argument("--only", default="", help="comma-separated groups: " + ", ".join(GROUPS))
    ap.add_argument("--batches", default="1,8,64", help="decode attention: requests in the step")
    ap.add_argument("--contexts", default="512,2048,8192,32768", help="decode attention: keys a request")
    ap.add_argument("--prefill-lengths", default="512,2048,8192", help="prefill attention: prompt tokens")
    ap.add_argument("--tokens", default="1,8,16,64,2048", help="products and element-wise kernels")
    ap.add_argument("--products", default="", help="products: only those whose name contains one of "
                    "these comma-separated pieces (q|k|v, o product, gate|up, down, LM head)")
    ap.add_argument("--fused-only", action="store_true",
                    help="products: only the o and down products with add and norm in their epilogue")
    ap.add_argument("--no-twins", action="store_true", help="skip the plain twins of the attention kernels")
    ap.add_argument("--force-splits", type=int, default=0,
                    help="decode attention: launch this many key splits instead of the launcher's choice")
    ap.add_argument("--no-cluster", action="store_true",
                    help="decode attention: combine the splits through the arrival counter, not clusters")
    ap.add_argument("--peaks", default=DEFAULT_PEAKS, help="JSON file with hbm_gbs and bf16_tflops")
    ap.add_argument("--markdown", action="store_true")
    args = ap.parse_args(argv)

    peaks = W.load_peaks(args.peaks)
    from ..ops import kernels as K
    K.require_cuda()
    K.decode_ws_force_splits = args.force_splits
    K.decode_ws_cluster = not args.no_cluster
    device = "cuda:0"
    shape = SHAPES[args.shape]
    groups = [g for g in args.only.split(",") if g] or list(GROUPS)
    unknown = [g for g in groups if g not in GROUPS + EXTRA_GROUPS]
    if unknown:
        raise SystemExit(f"unknown group(s) {unknown}; known: {', '.join(GROUPS + EXTRA_GROUPS)}")
    rows: List[Row] = []
    for g in groups:
        print(f"[kernel_bench] {g} ...", file=sys.stderr, flush=True)
        if g == "decode_attention":
            rows += bench_decode_attention(shape, peaks, device, _ints(args.batches),
                                           _ints(args.contexts), not args.no_twins)
        elif g == "prefill_attention":
            rows += bench_prefill_attention(shape, peaks, device, _ints(args.prefill_lengths),
                                            not args.no_twins)
        elif g == "reference_kernels":
            from .reference_kernels import compare
            print("reference kernels beside this package's:", json.dumps(compare(device), indent=1))
        elif g == "products":
            rows += bench_products(shape, peaks, device, _ints(args.tokens),
                                   [p for p in args.products.split(",") if p], args.fused_only)
        else:
            rows += bench_elementwise(shape, peaks, device, _ints(args.tokens))
    print(f"{args.shape}: hidden {shape[0]}, heads {shape[1]}/{shape[2]} x {shape[3]}, intermediate "
          f"{shape[4]}, vocabulary {shape[5]}; page {PAGE}; peaks ({peaks['source']}) "
          f"{peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops']:.0f} TFLOP/s")
    print(render(rows, args.markdown))
    status = {"gemm_tc": K.gemm_tc_status(), "attention": K.attention_status(shape[3]),
              "prefill_attention_tc": K.prefill_attention_tc_status(shape[3]),
              "decode_attention": K.decode_attention_status(shape[3])}
    print("kernel status words (0 = no bounded wait gave up):", json.dumps(status))
    return 0 if not any(status.values()) else 1


if __name__ == "__main__":
    sys.exit(main())

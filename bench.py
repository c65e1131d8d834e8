#!/usr/bin/env python3
"""Benchmark of the serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the
Qwen2.5-7B shape with random weights, a batch of 8 requests with 2,048-token
prompts (context limit 4,096, page size 16).  It prints ONE JSON line:
decoded tokens per second timed on the device (``value``), the same through the
Python entry point with host tokens in and out (``e2e``), a 2,048-token prefill
(``prefill``), the decode step's memory roofline (``roofline``) and decoding at
batch 1 and 64 (``points``).  Weights (14 GB) are larger than the L2 cache, so
every timed step reads them from HBM; no extra flush is needed.

More than one GPU is not supported: one line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 28,
    "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 32768,
    "use_sliding_window": False, "torch_dtype": "bfloat16", "eos_token_id": 151645,
}
PROMPT_LEN, CONTEXT, PAGE = 2048, 4096, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max([int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()] or [0])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": reasons, "samples": len(sm)}


def weight_bytes_per_step(cfg, layers):
    h, H, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"],
                          cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"],
                          cfg["vocab_size"])
    per_layer = (H + 2 * Hkv) * D * h + H * D * h + 3 * I * h
    return 2 * (layers * per_layer + V * h), per_layer


def kv_bytes_per_token(cfg, layers):
    return 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, T):
    _, per_layer = weight_bytes_per_step(cfg, layers)
    lin = 2 * T * layers * per_layer
    attn = layers * 4 * (T * (T + 1) // 2) * cfg["num_attention_heads"] * cfg["head_dim"]
    return lin + attn + 2 * cfg["vocab_size"] * cfg["hidden_size"]


_T0 = time.perf_counter()


def note(msg: str) -> None:
    """Progress on stderr (the JSON line on stdout stays alone)."""
    print(f"[bench +{time.perf_counter() - _T0:6.1f}s] {msg}", file=sys.stderr, flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0 = all)")
    ap.add_argument("--skip-points", action="store_true", help="no batch 1/64 and no prefill")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill"],
                    help="profiling aid: run only the decode loop or only the prefill")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: launch kernels eagerly")
    ap.add_argument("--tune", action="append", default=[], metavar="NAME=VALUE",
                    help="measurement aid: set a dispatch tunable (skinny_max_tokens, "
                         "decode_ctas_per_sm, pdl)")
    ap.add_argument("--profile-region", action="store_true",
                    help="profiling aid: cudaProfilerStart/Stop around the device-timed region")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference's engine imports servelab.models, a package its tree "
                          "does not contain (excluded by its own .gitignore), so it cannot run"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from servelab_b200.config import CacheConfig, SchedulerConfig, config_from_dict
    from servelab_b200.engine.llm_engine import LLMEngine
    from servelab_b200.models import declare_tensors
    from servelab_b200.ops import kernels as K
    from servelab_b200.sampling import SamplingParams
    from servelab_b200.weights import RandomSource

    from servelab_b200.ops import linear as linear_ops
    for item in args.tune:
        name, value = item.split("=")
        if name == "skinny_max_tokens":
            linear_ops.skinny_max_tokens = int(value)
        elif name in ("tc_max_tokens", "tc_wide_max_tokens"):
            setattr(linear_ops, name, int(value))
        elif name in ("defer_rope", "defer_norm"):
            linear_ops.defer_split_sums[name[6:]] = bool(int(value))
        elif name == "tc_max_stages":
            K.tc_max_stages = int(value)
        elif name == "decode_ctas_per_sm":
            K.decode_ctas_per_sm = int(value)
        elif name in ("decode_ws_stages", "decode_ws_force_splits", "decode_ws_unsplit_tiles"):
            setattr(K, name, int(value))
        elif name == "decode_ws_split_coef":
            K.decode_ws_split_coef = float(value)
        elif name in ("tc_prefetch_bytes", "tc_prefetch_chunk", "tc_blocks_per_sm"):
            setattr(K, name, int(value))
        elif name in ("fuse_swiglu", "cluster_sums", "fuse_qkv_rope", "fuse_resid_norm"):
            setattr(linear_ops, name, bool(int(value)))
        elif name in ("cluster_max_kblocks", "cluster_long_k_max_tokens"):
            setattr(linear_ops, name, int(value))
        elif name == "tc_max_cluster":                      # at most 8, the portable cluster size
            K.TC_MAX_CLUSTER = int(value)
        elif name == "use_tc_prefill":
            K.use_tc_prefill = bool(int(value))
        elif name == "fuse_decode_qkv":
            from servelab_b200.ops import attention as attention_ops
            attention_ops.fuse_decode_qkv = bool(int(value))
        elif name == "pdl":
            from servelab_b200.ops import library as kernel_library
            kernel_library.set_pdl(bool(int(value)))
        else:
            raise SystemExit(f"unknown tunable {name}")

    cfg = dict(QWEN25_7B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    config = config_from_dict(cfg)
    peaks = load_peaks()
    if args.only:
        args.skip_points = True
    max_batch = 64 if not args.skip_points else max(args.batch, 1)
    max_batch = max(max_batch, args.batch)
    pages = max_batch * (CONTEXT // PAGE) + 64
    note("building the engine (random weights on the device, cache pool)")
    source = RandomSource(declare_tensors(config.to_model_spec()), seed=0, device="cuda:0",
                          dtype=torch.bfloat16)
    engine = LLMEngine(config, CacheConfig(block_size=PAGE, num_blocks=pages),
                       SchedulerConfig(max_num_seqs=max_batch, max_num_batched_tokens=PROMPT_LEN),
                       dtype="bfloat16", weights=source, cuda_graphs=not args.no_graphs,
                       max_model_len=CONTEXT)
    runner = engine.runner
    note("engine ready")
    gen = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def prompts(n):
        return [torch.randint(0, V, (PROMPT_LEN,), generator=gen).tolist() for _ in range(n)]

    def run_decode(batch, steps, warmup, clocks=None):
        """Prefill ``batch`` prompts through the engine, then time decode steps
        (a) on the device through the step function and (b) end to end through
        engine.step() with host tokens in and out."""
        sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN - 8, ignore_eos=True)
        for p in prompts(batch):
            engine.add_request(prompt_token_ids=p, sampling_params=sp)
        while any(not s.is_decoding() for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        assert len(engine.scheduler.running) == batch
        note(f"batch {batch}: prompts prefilled, timing {steps} decode steps end to end and on the device")
        # (b) end to end: schedule, pack, H2D, graph replay, sample, D2H, bookkeeping
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        # (a) device time of the same step: replay with CUDA events around it
        seqs = list(engine.scheduler.running)
        entries = []
        for s in seqs:
            runner.cache.ensure(s.request_id, s.get_len())
            entries.append(runner.entry(s.request_id, [s.token_ids[-1]], s.get_len() - 1, (0,)))
        out_ids = torch.empty(batch, dtype=torch.int32, device="cuda:0")
        for _ in range(warmup):
            K.sample_rows(runner.step(entries), out_ids)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0 = K.launch_count
        if args.profile_region:
            torch.cuda.profiler.start()
        start.record()
        for _ in range(steps):
            K.sample_rows(runner.step(entries), out_ids)
        stop.record()
        torch.cuda.synchronize()
        if args.profile_region:
            torch.cuda.profiler.stop()
        dev_ms = start.elapsed_time(stop) / steps
        clk = clocks.stop() if clocks else None
        ctx_tokens = sum(s.get_len() for s in seqs)
        per_graph = getattr(runner, "graph_kernel_launches", {}).get(batch, 0)
        launches = (K.launch_count - k0) + per_graph * steps
        desc_bytes = engine.runner._graphs[batch][1]._dev.numel() * 4 if batch in runner._graphs else 0
        for s in seqs:
            engine.abort_request(s.request_id)
        return {"dev_ms": dev_ms, "e2e_ms": e2e_s * 1000 / steps, "ctx_tokens": ctx_tokens,
                "launches": launches, "h2d": desc_bytes, "d2h": batch * 4, "clocks": clk}

    def run_prefill():
        """One 2,048-token prompt through the step function, timed on the device
        (median of the runs after two warm-ups)."""
        ids = prompts(1)[0]
        times = []
        for i in range(5):
            rid = f"prefill-{i}"
            runner.cache.open(rid)
            runner.cache.ensure(rid, PROMPT_LEN)
            entry = runner.entry(rid, ids, 0, (PROMPT_LEN - 1,))
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if args.profile_region and i == 4:
                torch.cuda.profiler.start()
            start.record()
            runner.step([entry])
            stop.record()
            torch.cuda.synchronize()
            if args.profile_region and i == 4:
                torch.cuda.profiler.stop()
            times.append(start.elapsed_time(stop))
            runner.cache.release(rid)
        ms = sorted(times[2:])[len(times[2:]) // 2]
        flops = prefill_flops(cfg, layers, PROMPT_LEN)
        return {"value": round(PROMPT_LEN / (ms * 1e-3), 1), "tokens": PROMPT_LEN,
                "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    def kernel_status():
        """Status words of the kernels with bounded waits (0 = no wait gave up)."""
        D = cfg["head_dim"]
        status = {"gemm_tc": K.gemm_tc_status(), "attention": K.attention_status(D),
                  "prefill_attention_tc": K.prefill_attention_tc_status(D),
                  "decode_attention": K.decode_attention_status(D)}
        if status["prefill_attention_tc"]:
            note(f"tcgen05 prefill attention gave up a wait: {K.prefill_attention_tc_where(D)}")
        return status

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": layers, "prefill": run_prefill(),
                          "kernel_status": kernel_status()}))
        return 0
    clocks = ClockSampler()
    note(f"decode at batch {args.batch}")
    main_run = run_decode(args.batch, args.steps, args.warmup, clocks)
    wbytes, _ = weight_bytes_per_step(cfg, layers)
    step_bytes = wbytes + main_run["ctx_tokens"] * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (main_run["dev_ms"] * 1e-3) / 1e9
    value = args.batch / (main_run["dev_ms"] * 1e-3)
    result = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B shape, 2048-token prompts",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["dev_ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, token ids uniform over the vocabulary",
        "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "layers": layers, "layers_of_shape": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "page_size": PAGE,
                   "parallelism": "single GPU", "cuda_graphs": not args.no_graphs,
                   "l2": "weights (14 GB) exceed L2; no flush", "peaks": peaks["source"]},
        "e2e": {"value": round(args.batch / (main_run["e2e_ms"] * 1e-3), 1), "unit": "tok/s",
                "ms_per_step": round(main_run["e2e_ms"], 4),
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": main_run["clocks"],
    }
    if not args.skip_points:
        note("prefill of one prompt")
        result["prefill"] = run_prefill()
        points = {}
        for b in (1, 64):
            r = run_decode(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (r["dev_ms"] * 1e-3), 1)
            sb = wbytes + r["ctx_tokens"] * kv_bytes_per_token(cfg, layers)
            points[f"decode_b{b}_hbm_frac"] = round(sb / (r["dev_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            points[f"decode_b{b}_e2e"] = round(b / (r["e2e_ms"] * 1e-3), 1)
        result["points"] = points
    result["kernel_status"] = kernel_status()
    note("done")
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())

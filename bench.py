#!/usr/bin/env python3
"""Benchmark of the serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the
Qwen2.5-7B shape with random weights, a batch of 8 requests with 2,048-token
prompts (context limit 4,096, page size 16).  It prints ONE JSON line:
decoded tokens per second timed on the device (``value``: the median of
``--rounds`` timed regions of ``--steps`` steps each), the same through the Python
entry point with host tokens in and out (``e2e``), a 2,048-token prefill
(``prefill``), the decode step's memory roofline (``roofline``), and under
``points``: decoding at batch 1 and 64, at contexts of 512, 8,192 and 32,768 tokens
for batch 8 (the longest also for one request), the continuous-batching workloads of the 0.5B and 14B shapes with their
roofline fractions, and the largest difference between the logits of a graph-replayed
decode step and the same step run eagerly through the plain twin kernels.  Weights
(14 GB) are larger than the L2 cache, so every timed step reads them from HBM; no
extra flush is needed.

``--impl reference``: the reference's engine cannot run (the line says what its import
raises); its two GPU kernels can, and are timed beside this package's on the same data.

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

PROMPT_LEN, CONTEXT, PAGE = 2048, 4096, 16
SWEEP_CONTEXTS = (512, 8192, 32768)


class ClockSampler:
    """Samples SM clocks and throttle reasons of the GPU in use with nvidia-smi (a read-only
    query) while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: str = "0"):
        """``gpu``: what ``nvidia-smi -i`` takes; the UUID of the CUDA device, because index 0 of
        nvidia-smi need not be the device this process was given."""
        self.gpu, self.rows, self.proc = gpu, [], None

    @staticmethod
    def current_gpu() -> str:
        try:
            import torch
            return "GPU-" + str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
        except Exception:                                   # noqa: BLE001 (older torch: no uuid)
            return "0"

    def start(self):
        self.rows = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, args=(self.proc, self.rows), daemon=True).start()
        except OSError:
            self.proc = None

    @staticmethod
    def _read(proc, rows):
        for line in proc.stdout:
            rows.append([c.strip() for c in line.split(",")])

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


_T0 = time.perf_counter()


def note(msg: str) -> None:
    """Progress on stderr (the JSON line on stdout stays alone)."""
    print(f"[bench +{time.perf_counter() - _T0:6.1f}s] {msg}", file=sys.stderr, flush=True)


def reference_arm() -> int:
    """The reference through its own public API: its engine does not import; its two Triton
    kernels do and are timed on the reference's own benchmark shapes."""
    from servelab_b200.bench import reference_kernels as R
    why = R.reference_engine_error() or "the reference's engine imported, which was not expected"
    line = {"impl": "reference",
            "unavailable": "the reference's engine cannot be imported (its tree lacks the model "
                           "package it imports, excluded by its own .gitignore): " + why}
    try:
        import torch
        if torch.cuda.is_available():
            line["kernel_level"] = R.compare()
    except Exception as e:                                  # noqa: BLE001
        line["kernel_level"] = {"unavailable": f"{type(e).__name__}: {e}"}
    print(json.dumps(line))
    return 0


TUNABLES = """tc_max_tokens tc_wide_max_tokens cluster_max_kblocks cluster_long_k_max_tokens
cluster_max_tokens_per_block (ints, ops.linear); defer_rope defer_norm fuse_swiglu cluster_sums fuse_qkv_rope fuse_resid_norm (0/1, ops.linear); tc_max_stages
tc_blocks_per_sm decode_ctas_per_sm decode_ws_stages decode_ws_force_splits decode_ws_unsplit_tiles
tc_max_cluster (ints, ops.kernels); decode_ws_split_coef (float); use_tc_prefill decode_ws_cluster pdl
pdl_early evict_first (0/1)"""


def apply_tunables(items):
    from servelab_b200.ops import kernels as K
    from servelab_b200.ops import library as kernel_library
    from servelab_b200.ops import linear as linear_ops
    for item in items:
        name, value = item.split("=")
        if name in ("tc_max_tokens", "tc_wide_max_tokens", "cluster_max_kblocks", "cluster_long_k_max_tokens",
                    "cluster_max_tokens_per_block"):
            setattr(linear_ops, name, int(value))
        elif name in ("defer_rope", "defer_norm"):
            linear_ops.defer_split_sums[name[6:]] = bool(int(value))
        elif name in ("fuse_swiglu", "cluster_sums", "fuse_qkv_rope", "fuse_resid_norm"):
            setattr(linear_ops, name, bool(int(value)))
        elif name in ("tc_max_stages", "tc_token_group", "tc_token_group_bytes", "tc_blocks_per_sm", "decode_ctas_per_sm", "decode_ws_stages",
                      "decode_ws_force_splits", "decode_ws_unsplit_tiles"):
            setattr(K, name, int(value))
        elif name == "tc_max_cluster":                      # at most 8, the portable cluster size
            K.TC_MAX_CLUSTER = int(value)
        elif name == "decode_ws_split_coef":
            K.decode_ws_split_coef = float(value)
        elif name in ("use_tc_prefill", "decode_ws_cluster"):
            setattr(K, name, bool(int(value)))
        elif name == "pdl":
            kernel_library.set_pdl(bool(int(value)))
        elif name == "pdl_early":
            kernel_library.set_pdl_early(bool(int(value)))
        elif name == "evict_first":
            kernel_library.set_evict_first(bool(int(value)))
        else:
            raise SystemExit(f"unknown tunable {name}; known: {TUNABLES}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=3, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0 = all)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline, its e2e and roofline")
    ap.add_argument("--skip-workloads", action="store_true", help="no 0.5B / 14B serving workloads")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill"],
                    help="profiling aid: run only the decode loop or only the prefill")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: launch kernels eagerly")
    ap.add_argument("--tune", action="append", default=[], metavar="NAME=VALUE",
                    help="measurement aid: set a dispatch tunable: " + TUNABLES)
    ap.add_argument("--profile-region", action="store_true",
                    help="profiling aid: cudaProfilerStart/Stop around the device-timed region")
    ap.add_argument("--timeline", default="", metavar="FILE",
                    help="measurement aid: record when every block of the decode kernels started, got "
                         "past its wait for the preceding kernel and ended (the device's own timer) "
                         "for one replayed step; rows per launch to FILE (JSON), the first to stderr")
    ap.add_argument("--profile-steps", type=int, default=0, metavar="N",
                    help="also run N decode steps and one prefill eagerly with a CUDA event after "
                         "every kernel and print the per-kernel table (stderr; 'step_profile' in the line)")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.rounds = max(args.rounds, 1)

    import torch
    from servelab_b200.bench import workloads as W
    from servelab_b200.ops import attention as attention_ops
    from servelab_b200.ops import kernels as K
    from servelab_b200.ops import linear as linear_ops
    from servelab_b200.ops.profile import StepProfile
    from servelab_b200.sampling import SamplingParams
    apply_tunables(args.tune)
    timeline = None
    if args.timeline:
        from servelab_b200.ops.timeline import DeviceTimeline
        timeline = DeviceTimeline()
        timeline.__enter__()           # before the graphs are captured: the buffer is a launch argument

    cfg = dict(W.SHAPES["qwen2.5-7b"])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    peaks = W.load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    if args.only:
        args.skip_points = True
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    pages = max_batch * (CONTEXT // PAGE) + 64
    note("building the engine (random weights on the device, cache pool)")
    engine = W.make_engine(cfg, pages, max_batch, PROMPT_LEN, CONTEXT, weights_seed=0, page_size=PAGE,
                           cuda_graphs=not args.no_graphs)
    runner = engine.runner
    note("engine ready")
    gen = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]
    clocks = ClockSampler(ClockSampler.current_gpu())
    wbytes = W.weight_bytes_per_step(cfg, layers)
    kvb = W.kv_bytes_per_token(cfg, layers)

    def prompts(n, length=PROMPT_LEN):
        return [torch.randint(0, V, (length,), generator=gen).tolist() for _ in range(n)]

    def timed_rounds(run_step, steps, rounds, with_clocks, warmup=0, profile=False):
        """``warmup`` untimed steps, then ``rounds`` regions of ``steps`` steps between CUDA events;
        (ms per step of each region, one clock record over warm-up and regions: the sampler's
        own start takes longer than a short region)."""
        if with_clocks:
            clocks.start()
        for _ in range(warmup):
            run_step()
        if profile:
            torch.cuda.profiler.start()
        times = []
        for _ in range(rounds):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                run_step()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) / steps)
        if profile:
            torch.cuda.profiler.stop()
        return times, (clocks.stop() if with_clocks else None)

    def decode_entries(seqs):
        entries = []
        for s in seqs:
            runner.cache.ensure(s.request_id, s.get_len())
            entries.append(runner.entry(s.request_id, [s.token_ids[-1]], s.get_len() - 1, (0,)))
        return entries

    def logit_check(entries):
        """The largest difference between the logits of the replayed graph and of the same step
        run eagerly through the plain twin kernels (CUDA-core attention; K-split sums through
        global memory instead of clusters)."""
        fast = runner.step(entries).clone()
        saved = (runner.cuda_graphs, attention_ops.force_generic, linear_ops.cluster_sums)
        runner.cuda_graphs, attention_ops.force_generic, linear_ops.cluster_sums = False, True, False
        try:
            plain = runner.step(entries)
        finally:
            runner.cuda_graphs, attention_ops.force_generic, linear_ops.cluster_sums = saved
        differ = fast.argmax(-1) != plain.argmax(-1)
        top2 = plain.topk(2, dim=-1).values
        out = {"max_abs_diff": round(float((fast - plain).abs().max()), 5),
               "largest_logit": round(float(plain.abs().max()), 3),
               "same_argmax_rows": int((~differ).sum()), "rows": fast.shape[0]}
        if bool(differ.any()):      # rows whose two best logits are closer than the rounding noise
            out["widest_top2_gap_of_differing_rows"] = round(float((top2[:, 0] - top2[:, 1])[differ].max()), 5)
        return out

    def run_decode(batch, steps, warmup, rounds=1, with_clocks=False):
        """Prefill ``batch`` prompts through the engine, then time decode steps
        (a) end to end through engine.step() with host tokens in and out and (b) on the
        device through the step function."""
        sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN - 8, ignore_eos=True)
        for p in prompts(batch):
            engine.add_request(prompt_token_ids=p, sampling_params=sp)
        while any(not s.is_decoding() for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        assert len(engine.scheduler.running) == batch
        note(f"batch {batch}: prompts prefilled, timing {rounds} x {steps} decode steps end to end and on the device")
        # (a) end to end: schedule, pack, H2D, graph replay, sample, D2H, bookkeeping
        for _ in range(warmup):
            engine.step()
        e2e = []
        for _ in range(rounds):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            e2e.append((time.perf_counter() - t0) * 1e3 / steps)
        # (b) device time of the same step: replay with CUDA events around it
        seqs = list(engine.scheduler.running)
        entries = decode_entries(seqs)
        out_ids = torch.empty(batch, dtype=torch.int32, device="cuda:0")

        def one_step():
            K.sample_rows(runner.step(entries), out_ids)
        for _ in range(3):
            one_step()
        k0 = K.launch_count
        dev, record = timed_rounds(one_step, steps, rounds, with_clocks, profile=args.profile_region,
                                   warmup=max(0, warmup - 3) + (200 if with_clocks and not args.profile_region else 0))
        ctx_tokens = sum(s.get_len() for s in seqs)
        per_graph = runner.graph_kernel_launches.get(batch, 0)
        ran = steps * rounds + max(0, warmup - 3) + (200 if with_clocks and not args.profile_region else 0)
        launches = round(((K.launch_count - k0) + per_graph * ran) / ran * steps)   # of one timed region
        desc_bytes = runner._graphs[batch][1]._dev.numel() * 4 if batch in runner._graphs else 0
        if timeline is not None and with_clocks:
            one_step()
            timeline.reset()
            one_step()
            rows = timeline.launches()
            with open(args.timeline, "w") as f:
                json.dump(rows, f)
            note(f"timeline of one replayed decode step at batch {batch} ({len(rows)} launches; "
                 f"microseconds):\n" + timeline.render(40))
        check = logit_check(entries)
        profile = None
        if args.profile_steps:
            saved, runner.cuda_graphs = runner.cuda_graphs, False
            try:
                one_step()
                with StepProfile() as prof:
                    for _ in range(args.profile_steps):
                        one_step()
            finally:
                runner.cuda_graphs = saved
            note(f"per-kernel times of an eager decode step at batch {batch}:\n" + prof.render(args.profile_steps))
            profile = prof.summary(args.profile_steps)
        for s in seqs:
            engine.abort_request(s.request_id)
        med = sorted(dev)[len(dev) // 2]
        return {"dev_ms": med, "dev_ms_rounds": [round(t, 4) for t in dev],
                "e2e_ms": sorted(e2e)[len(e2e) // 2], "ctx_tokens": ctx_tokens, "launches": launches,
                "h2d": desc_bytes, "d2h": batch * 4, "clocks": record, "logit_check": check,
                "profile": profile}

    def run_context(batch, ctx_len, steps, warmup):
        """A decode step of ``batch`` requests that each hold ``ctx_len`` tokens.  The pages are
        taken, not prefilled: the step's time does not depend on the values of the cache."""
        ids = []
        for b in range(batch):
            rid = f"ctx-{ctx_len}-{b}"
            if not (runner.cache.open(rid) and runner.cache.ensure(rid, ctx_len)):
                raise RuntimeError(f"no room for {batch} requests of {ctx_len} tokens")
            ids.append(rid)
        entries = [runner.entry(rid, [1 + b], ctx_len - 1, (0,)) for b, rid in enumerate(ids)]
        out_ids = torch.empty(batch, dtype=torch.int32, device="cuda:0")

        def one_step():
            K.sample_rows(runner.step(entries), out_ids)
        dev, _ = timed_rounds(one_step, steps, 1, False, warmup=warmup)
        for rid in ids:
            runner.cache.release(rid)
        nbytes = wbytes + batch * ctx_len * kvb
        return dev[0], nbytes / (dev[0] * 1e-3) / 1e9 / peaks["hbm_gbs"]

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
            if args.profile_steps and i == 4:
                saved, runner.cuda_graphs = runner.cuda_graphs, False    # (launched one by one)
                try:
                    with StepProfile() as prof:
                        runner.step([entry])
                finally:
                    runner.cuda_graphs = saved
                note("per-kernel times of the 2,048-token prefill:\n" + prof.render())
            runner.cache.release(rid)
        ms = sorted(times[2:])[len(times[2:]) // 2]
        flops = W.prefill_flops(cfg, layers, PROMPT_LEN)
        out = {"value": round(PROMPT_LEN / (ms * 1e-3), 1), "tokens": PROMPT_LEN,
               "ms": round(ms, 3),
               "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
        if peaks.get("bf16_tflops_sustained"):      # beside it: of the GEMM rate a seconds-long loop holds
            out["frac_of_sustained"] = round(flops / (ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
        return out

    def kernel_status():
        """Status words of the kernels with bounded waits and page checks (0 = nothing happened)."""
        D = cfg["head_dim"]
        status = {"gemm_tc": K.gemm_tc_status(), "attention": K.attention_status(D),
                  "prefill_attention_tc": K.prefill_attention_tc_status(D),
                  "decode_attention": K.decode_attention_status(D),
                  "cache_write": K.cache_write_status()}
        if status["prefill_attention_tc"]:
            note(f"tcgen05 prefill attention gave up a wait: {K.prefill_attention_tc_where(D)}")
        return status

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": layers, "prefill": run_prefill(),
                          "kernel_status": kernel_status()}))
        return 0
    note(f"decode at batch {args.batch}")
    main_run = run_decode(args.batch, args.steps, args.warmup, args.rounds, with_clocks=True)
    step_bytes = wbytes + main_run["ctx_tokens"] * kvb
    achieved = step_bytes / (main_run["dev_ms"] * 1e-3) / 1e9
    value = args.batch / (main_run["dev_ms"] * 1e-3)
    clock_line = main_run["clocks"]
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
                   "l2": "weights (14 GB) exceed L2; no flush", "peaks": peaks["source"],
                   "rounds": args.rounds},
        "rounds_ms_per_step": main_run["dev_ms_rounds"],
        "e2e": {"value": round(args.batch / (main_run["e2e_ms"] * 1e-3), 1), "unit": "tok/s",
                "ms_per_step": round(main_run["e2e_ms"], 4),
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": clock_line,
        "logit_check": {f"decode_b{args.batch}": main_run["logit_check"]},
    }
    if main_run["profile"]:
        result["step_profile"] = main_run["profile"]
    if not args.skip_points:
        note("prefill of one prompt")
        result["prefill"] = run_prefill()
        points = {}
        for b in (1, 64):
            r = run_decode(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (r["dev_ms"] * 1e-3), 1)
            sb = wbytes + r["ctx_tokens"] * kvb
            points[f"decode_b{b}_hbm_frac"] = round(sb / (r["dev_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            points[f"decode_b{b}_e2e"] = round(b / (r["e2e_ms"] * 1e-3), 1)
            result["logit_check"][f"decode_b{b}"] = r["logit_check"]
        result["points"] = points
    result["kernel_status"] = kernel_status()
    del runner, engine
    torch.cuda.empty_cache()
    if not args.skip_points:
        # decode at other contexts: an engine whose cache holds 8 requests of 32,768 tokens
        note("decode at batch 8 over contexts " + ", ".join(str(c) for c in SWEEP_CONTEXTS))
        long_ctx = max(SWEEP_CONTEXTS) + PAGE
        engine = W.make_engine(cfg, 8 * (long_ctx // PAGE) + 8, 8, PROMPT_LEN, long_ctx, weights_seed=0,
                               page_size=PAGE, cuda_graphs=not args.no_graphs)
        runner = engine.runner
        for c in SWEEP_CONTEXTS:
            ms, frac = run_context(8, c, max(16, args.steps // 2), args.warmup)
            result["points"][f"decode_b8_ctx{c}"] = round(8 / (ms * 1e-3), 1)
            result["points"][f"decode_b8_ctx{c}_hbm_frac"] = round(frac, 4)
        # one request with a long context: its keys are split over several clusters of blocks
        ms, frac = run_context(1, max(SWEEP_CONTEXTS), max(16, args.steps // 2), args.warmup)
        result["points"][f"decode_b1_ctx{max(SWEEP_CONTEXTS)}"] = round(1 / (ms * 1e-3), 1)
        result["points"][f"decode_b1_ctx{max(SWEEP_CONTEXTS)}_hbm_frac"] = round(frac, 4)
        st = K.decode_attention_status(cfg["head_dim"])
        result["kernel_status"]["decode_attention"] = result["kernel_status"]["decode_attention"] or st
        del runner, engine
        torch.cuda.empty_cache()
        if not args.skip_workloads:
            for shape, key in (("qwen2.5-0.5b", "serve_0.5b"), ("qwen2.5-14b", "serve_14b")):
                note(f"continuous-batching workload of the {shape} shape")
                r = W.run_workload(shape, peaks, note=note)
                result["points"][f"{key}_gen_tok_s"] = r["generated_tokens_per_s"]
                result["points"][f"{key}_total_tok_s"] = r["total_tokens_per_s"]
                result["points"][f"{key}_roofline_frac"] = r["roofline_frac"]
                result["points"][f"{key}_ms_per_step"] = r["ms_per_step"]
                result["points"][f"{key}_ok"] = bool(r["ok"])
    note("done")
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())

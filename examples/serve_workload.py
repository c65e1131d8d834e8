"""Continuous batching on a model shape with random weights: many requests of random
prompt lengths, chunked prefill beside decoding, throughput and roofline fraction at the end.

    python examples/serve_workload.py --shape qwen2.5-0.5b        # 64 requests, prompts 16..1024, 128 new tokens
    python examples/serve_workload.py --shape qwen2.5-14b         # 32 requests, prompts 512..4096, 256 new tokens
    python examples/serve_workload.py --shape qwen2.5-7b --requests 16 --prompt-len 100:900 --max-tokens 64

Weights are drawn on the device (nothing is written to disk); token ids are uniform
over the vocabulary.  Prints one JSON line: requests, prompt and generated tokens,
seconds, tokens a second, steps, preemptions, whether every page came back, and the
workload's floor (the sum over its steps of the time the bytes and flops of the step need
at the machine's measured peaks) over the measured time.
"""
import argparse
import json
import os
import sys

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
sys.path.insert(0, ROOT)


def main(argv=None) -> int:
    from servelab_b200.bench import workloads as W
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="qwen2.5-0.5b", choices=sorted(W.SHAPES))
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--prompt-len", default="", help="LOW:HIGH, uniform")
    ap.add_argument("--max-tokens", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=-1.0)
    ap.add_argument("--max-batched-tokens", type=int, default=0, help="the prefill chunk")
    ap.add_argument("--max-num-seqs", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=0, help="0 = enough for every request at once")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--warmup", type=int, default=1,
                    help="untimed passes of the same workload first (graphs of the decode batch sizes "
                         "are captured at their first use)")
    ap.add_argument("--peaks", default=os.path.join(ROOT, "MEASURED_PEAKS.json"),
                    help="JSON file with hbm_gbs and bf16_tflops (else the stated fallback)")
    args = ap.parse_args(argv)
    span = tuple(int(v) for v in args.prompt_len.split(":")) if args.prompt_len else None
    result = W.run_workload(
        args.shape, W.load_peaks(args.peaks), layers=args.layers, requests=args.requests,
        prompt_len=span, max_tokens=args.max_tokens, temperature=args.temperature,
        chunk=args.max_batched_tokens, max_num_seqs=args.max_num_seqs, page_size=args.block_size,
        num_blocks=args.num_blocks, dtype=args.dtype, warmup=args.warmup,
        note=lambda m: print(f"[serve_workload] {m}", file=sys.stderr, flush=True))
    print(json.dumps(result))
    return 0 if result["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())

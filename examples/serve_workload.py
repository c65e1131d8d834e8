"""Continuous batching on a model shape with random weights: many requests of random
prompt lengths, chunked prefill beside decoding, throughput at the end.

    python examples/serve_workload.py --shape qwen2.5-0.5b        # 64 requests, prompts 16..1024, 128 new tokens
    python examples/serve_workload.py --shape qwen2.5-14b         # 32 requests, prompts 512..4096, 256 new tokens
    python examples/serve_workload.py --shape qwen2.5-7b --requests 16 --prompt-len 100:900 --max-tokens 64

Weights are drawn on the device (nothing is written to disk); token ids are uniform
over the vocabulary.  Prints one JSON line: requests, prompt and generated tokens,
seconds, tokens a second, steps, preemptions, and whether every page came back.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

QWEN2 = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rope_theta": 1000000.0,
         "rms_norm_eps": 1e-6, "max_position_embeddings": 32768, "use_sliding_window": False,
         "torch_dtype": "bfloat16", "eos_token_id": 151645}
SHAPES = {
    "qwen2.5-0.5b": dict(QWEN2, num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                         num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                         tie_word_embeddings=True),
    "qwen2.5-7b": dict(QWEN2, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
                       num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
                       tie_word_embeddings=False),
    "qwen2.5-14b": dict(QWEN2, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40,
                        num_key_value_heads=8, head_dim=128, intermediate_size=13824, vocab_size=152064,
                        tie_word_embeddings=False),
}
# requests, prompt lengths, new tokens, temperature, prefill chunk, weights seed, sampler seed
WORKLOADS = {
    "qwen2.5-0.5b": (64, (16, 1024), 128, 0.0, 512, 5, 0),
    "qwen2.5-7b": (32, (512, 2048), 128, 0.0, 2048, 0, 0),
    "qwen2.5-14b": (32, (512, 4096), 256, 1.0, 2048, 6, 7),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="qwen2.5-0.5b", choices=sorted(SHAPES))
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
    args = ap.parse_args(argv)

    import torch
    from servelab_b200.config import CacheConfig, SchedulerConfig, config_from_dict
    from servelab_b200.engine.llm_engine import LLMEngine
    from servelab_b200.models import declare_tensors
    from servelab_b200.sampling import SamplingParams
    from servelab_b200.weights import RandomSource

    n, (lo, hi), new, temp, chunk, wseed, sseed = WORKLOADS[args.shape]
    n = args.requests or n
    if args.prompt_len:
        lo, hi = (int(v) for v in args.prompt_len.split(":"))
    new = args.max_tokens or new
    temp = args.temperature if args.temperature >= 0 else temp
    chunk = args.max_batched_tokens or chunk
    cfg = dict(SHAPES[args.shape])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg)

    gen = torch.Generator().manual_seed(1)
    lengths = torch.randint(lo, hi + 1, (n,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist() for length in lengths]
    ps = args.block_size
    need = sum(-(-(length + new) // ps) for length in lengths)
    pages = args.num_blocks or need + 8
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    print(f"[serve_workload] {args.shape}: {n} requests, prompts {lo}..{hi} ({sum(lengths)} tokens), "
          f"{new} new tokens each, chunk {chunk}, {pages} pages of {ps}", file=sys.stderr, flush=True)
    source = RandomSource(declare_tensors(config.to_model_spec()), seed=wseed, device="cuda:0", dtype=dt)
    engine = LLMEngine(config, CacheConfig(block_size=ps, num_blocks=pages),
                       SchedulerConfig(max_num_seqs=args.max_num_seqs or n, max_num_batched_tokens=chunk),
                       dtype=args.dtype, weights=source, max_model_len=hi + new + ps, seed=sseed)
    sp = SamplingParams(temperature=temp, max_tokens=new, ignore_eos=True)
    free_before = engine.runner.cache.stats()["pages_free"]
    for _ in range(args.warmup):
        engine.generate(prompts, sp)
    steps0, ahead0, preempt0 = engine.num_steps, engine.num_lookahead_steps, engine.scheduler.num_preemptions
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, sp)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    generated = sum(len(o.outputs[0].token_ids) for o in outs)
    result = {
        "shape": args.shape, "layers": cfg["num_hidden_layers"], "dtype": args.dtype, "requests": n,
        "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(seconds, 3),
        "generated_tokens_per_s": round(generated / seconds, 1),
        "total_tokens_per_s": round((generated + sum(lengths)) / seconds, 1),
        "steps": engine.num_steps - steps0, "lookahead_steps": engine.num_lookahead_steps - ahead0,
        "preemptions": engine.scheduler.num_preemptions - preempt0,
        "all_pages_returned": engine.runner.cache.stats()["pages_free"] == free_before,
    }
    print(json.dumps(result))
    ok = generated == n * new and result["all_pages_returned"]
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

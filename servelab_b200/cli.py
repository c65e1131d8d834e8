"""Command line: offline generation on the engine, in the manner of the
reference's demo (examples/run_engine.py:27-72).

Options the reference has keep their names and meanings: --model (checkpoint
folder; empty = a tiny random model is written and used), --prompt (text; needs a
tokenizer in the folder), --max-tokens (default 32), --block-size (16),
--num-blocks (0 = from free memory).  Its --no-prefix-cache and --kv-cache-dtype
belong to features this engine does not have and are accepted only with their
neutral values.  Added: --prompt-ids, --dtype, --temperature, --top-k, --top-p,
--seed, --ignore-eos, --max-num-seqs, --max-batched-tokens, --random-weights,
--weights-seed.  As in the reference the scheduler runs with max_num_seqs 16 and
max_num_batched_tokens 1024 unless told otherwise, and sampling temperature
defaults to 1.0 (run_engine.py:57,66).
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile

TINY_CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 32,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 8,
    "intermediate_size": 64, "vocab_size": 96, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "max_position_embeddings": 512, "tie_word_embeddings": False, "torch_dtype": "float32",
    "eos_token_id": 95,
}   # the sizes of the reference's tiny test model (tests/helpers_tiny_model.py:7-30)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="servelab_b200", description="offline generation")
    ap.add_argument("--model", default="", help="checkpoint dir; empty = tiny random model")
    ap.add_argument("--prompt", default="The meaning of life is")
    ap.add_argument("--prompt-ids", default="", help="comma-separated token ids (overrides --prompt)")
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--no-prefix-cache", action="store_true",
                    help="accepted for compatibility: there is no prefix cache")
    ap.add_argument("--kv-cache-dtype", default="auto",
                    help="only 'auto' (the cache follows the compute dtype)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=0, help="0 = auto")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=1234, help="sampler seed")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--max-num-seqs", type=int, default=16)
    ap.add_argument("--max-batched-tokens", type=int, default=1024)
    ap.add_argument("--random-weights", default="",
                    help="a config.json: write a random model folder from it and use that")
    ap.add_argument("--weights-seed", type=int, default=0)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.kv_cache_dtype != "auto":
        print("error: --kv-cache-dtype: only 'auto' is supported", file=sys.stderr)
        return 2
    from .config import CacheConfig, SchedulerConfig, config_from_dict
    from .engine.llm_engine import LLMEngine
    from .sampling import SamplingParams
    from .weights import write_random_model

    model, tokenizer = args.model, None
    if args.random_weights or not model:
        cfg = TINY_CONFIG
        if args.random_weights:
            with open(args.random_weights) as f:
                cfg = json.load(f)
        model = tempfile.mkdtemp(prefix="servelab_b200_model_")
        write_random_model(model, config_from_dict(cfg), args.weights_seed)
        print(f"[servelab_b200] wrote random model to {model}")
    else:
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(model, trust_remote_code=True)
        except Exception as e:  # tokenizer is optional
            print(f"[warn] no tokenizer: {e}")

    engine = LLMEngine(
        model, CacheConfig(block_size=args.block_size, num_blocks=args.num_blocks or None),
        SchedulerConfig(max_num_seqs=args.max_num_seqs,
                        max_num_batched_tokens=args.max_batched_tokens),
        seed=args.seed, dtype=args.dtype, tokenizer=tokenizer)

    if args.prompt_ids:
        prompts = [[int(t) for t in args.prompt_ids.split(",")]]
    elif tokenizer is not None:
        prompts = [args.prompt]
    else:
        prompts = [list(range(10, 40))]            # token ids for the tiny model
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    for out in engine.generate(prompts, params, verbose=True):
        comp = out.outputs[0]
        print(f"[{out.request_id}] finish={comp.finish_reason} -> {comp.text or comp.token_ids}")
    print("stats:", engine.stats())
    return 0


if __name__ == "__main__":
    sys.exit(main())

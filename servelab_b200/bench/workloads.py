"""Model shapes, serving workloads and the roofline arithmetic the benchmarks share.

A decode step has to read every weight it uses once and the cached keys and values of the
live requests; a step with prompt portions also has arithmetic to do.  Its floor is the
slower of the two, the reference's own cost model (servelab/simulator/model_cost.py:64-75:
t = max(2 P tokens / F, (2 P + kv bytes) / BW)) with the attention flops added; a
workload's floor is the sum over its steps, and its roofline fraction the floor over the
measured time.
"""

from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks(path: str) -> Dict[str, object]:
    """Measured copy bandwidth and bf16 GEMM throughput of the machine from a JSON file with
    ``hbm_gbs`` and ``bf16_tflops``; the stated fallback if the file is absent."""
    import json
    try:
        with open(path) as f:
            d = json.load(f)
        out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
               "source": "measured"}
        if d.get("bf16_tflops_sustained"):                  # the same GEMM back to back under the power cap
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        return out
    except Exception:                                       # noqa: BLE001 (absent or unreadable)
        return dict(FALLBACK_PEAKS, source="fallback")


def layer_params(cfg: dict) -> int:
    h, H, Hkv, D, inter = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"])
    return (H + 2 * Hkv) * D * h + H * D * h + 3 * inter * h


def weight_bytes_per_step(cfg: dict, layers: int, itemsize: int = 2) -> int:
    """Every matrix a step multiplies by, once: the layers and the LM head (tied or not, the
    head is read; the embedding rows of the step's tokens are negligible)."""
    return itemsize * (layers * layer_params(cfg) + cfg["vocab_size"] * cfg["hidden_size"])


def kv_bytes_per_token(cfg: dict, layers: int, itemsize: int = 2) -> int:
    return 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * itemsize


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    lin = 2.0 * T * layers * layer_params(cfg)
    attn = layers * 4.0 * (T * (T + 1) // 2) * cfg["num_attention_heads"] * cfg["head_dim"]
    return lin + attn + 2.0 * cfg["vocab_size"] * cfg["hidden_size"]


def step_floor_seconds(cfg: dict, layers: int, tokens: int, kv_tokens: int, pair_count: float,
                       logit_rows: int, peaks: Dict[str, float]) -> float:
    """The least time a step can take: ``tokens`` run, ``kv_tokens`` cached keys and values are
    read (the sum of the context lengths of the step's requests), ``pair_count`` query-key pairs
    are scored, ``logit_rows`` rows go through the LM head."""
    nbytes = weight_bytes_per_step(cfg, layers) + kv_tokens * kv_bytes_per_token(cfg, layers)
    flops = (2.0 * tokens * layers * layer_params(cfg)
             + layers * 4.0 * pair_count * cfg["num_attention_heads"] * cfg["head_dim"]
             + 2.0 * logit_rows * cfg["vocab_size"] * cfg["hidden_size"])
    return max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12))


def make_engine(cfg: dict, pages: int, max_num_seqs: int, chunk: int, max_model_len: int,
                weights_seed: int = 0, sampler_seed: int = 1234, page_size: int = 16,
                dtype: str = "bfloat16", cuda_graphs: bool = True):
    """An engine of this shape with weights drawn on the device (nothing is written to disk)."""
    import torch
    from ..config import CacheConfig, SchedulerConfig, config_from_dict
    from ..engine.llm_engine import LLMEngine
    from ..models import declare_tensors
    from ..weights import RandomSource
    config = config_from_dict(cfg)
    dt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    source = RandomSource(declare_tensors(config.to_model_spec()), seed=weights_seed, device="cuda:0",
                          dtype=dt)
    return LLMEngine(config, CacheConfig(block_size=page_size, num_blocks=pages),
                     SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=chunk),
                     dtype=dtype, weights=source, cuda_graphs=cuda_graphs, max_model_len=max_model_len,
                     seed=sampler_seed)


def run_workload(shape: str, peaks: Dict[str, float], layers: int = 0, requests: int = 0,
                 prompt_len: Optional[Tuple[int, int]] = None, max_tokens: int = 0,
                 temperature: float = -1.0, chunk: int = 0, max_num_seqs: int = 0, page_size: int = 16,
                 num_blocks: int = 0, dtype: str = "bfloat16", warmup: int = 1, note=None,
                 repeats: int = 3, portion_graphs: bool = True) -> dict:
    """The continuous-batching workload of a shape through ``LLMEngine.generate`` (host token
    ids in, host token ids out), timed by the wall clock around it after ``warmup`` untimed
    passes (graphs of the decode batch sizes are captured at their first use).  The pass is
    timed ``repeats`` times and the median reported with all times beside it: the steps of a
    small model are bound by the host, whose speed varied by half between runs on shared
    machines."""
    import torch
    from ..sampling import SamplingParams
    n, (lo, hi), new, temp, wchunk, wseed, sseed = WORKLOADS[shape]
    n = requests or n
    lo, hi = prompt_len or (lo, hi)
    new = max_tokens or new
    temp = temperature if temperature >= 0 else temp
    chunk = chunk or wchunk
    cfg = dict(SHAPES[shape])
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    layers = cfg["num_hidden_layers"]
    gen = torch.Generator().manual_seed(1)
    lengths = torch.randint(lo, hi + 1, (n,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist() for length in lengths]
    need = sum(-(-(length + new) // page_size) for length in lengths)
    pages = num_blocks or need + 8
    if note:
        note(f"{shape}: {n} requests, prompts {lo}..{hi} ({sum(lengths)} tokens), {new} new tokens "
             f"each, chunk {chunk}, {pages} pages of {page_size}")
    engine = make_engine(cfg, pages, max_num_seqs or n, chunk, hi + new + page_size, wseed, sseed,
                         page_size, dtype)
    engine.runner.portion_graphs = engine.runner.portion_graphs and portion_graphs
    sp = SamplingParams(temperature=temp, max_tokens=new, ignore_eos=True)
    free_before = engine.runner.cache.stats()["pages_free"]
    for _ in range(warmup):
        engine.generate(prompts, sp)
    steps0, ahead0, preempt0 = engine.num_steps, engine.num_lookahead_steps, engine.scheduler.num_preemptions
    times = []
    for _ in range(max(1, repeats)):
        steps0, ahead0, preempt0 = (engine.num_steps, engine.num_lookahead_steps,
                                    engine.scheduler.num_preemptions)
        engine.step_trace = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = engine.generate(prompts, sp)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        trace, engine.step_trace = engine.step_trace, None
    seconds = sorted(times)[len(times) // 2]
    floor = sum(step_floor_seconds(cfg, layers, t, kv, pairs, rows, peaks) for t, kv, pairs, rows in trace)
    generated = sum(len(o.outputs[0].token_ids) for o in outs)
    result = {
        "shape": shape, "layers": layers, "layers_of_shape": full_layers, "dtype": dtype, "requests": n,
        "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(seconds, 4),
        "seconds_of_each_pass": [round(t, 4) for t in times],
        "generated_tokens_per_s": round(generated / seconds, 1),
        "total_tokens_per_s": round((generated + sum(lengths)) / seconds, 1),
        "steps": engine.num_steps - steps0, "lookahead_steps": engine.num_lookahead_steps - ahead0,
        "ms_per_step": round(seconds * 1e3 / max(1, engine.num_steps - steps0), 4),
        "preemptions": engine.scheduler.num_preemptions - preempt0,
        "all_pages_returned": engine.runner.cache.stats()["pages_free"] == free_before,
        "floor_seconds": round(floor, 4), "roofline_frac": round(floor / seconds, 4),
        "peaks": peaks.get("source", "given"),
        "portion_graph_replays": engine.runner.portion_graph_replays,
        "portion_graphs_held": len(engine.runner._portion_graphs),
    }
    result["ok"] = generated == n * new and result["all_pages_returned"]
    del engine
    torch.cuda.empty_cache()
    return result

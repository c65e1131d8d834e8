"""Shared test material: tiny configurations, random model folders, trace builders.

The tiny configurations differ in every size and option: layers, width, head
counts and groups, head size, intermediate size (172 is no multiple of 8), vocabulary
(300 is no power of two), rope theta, norm eps, tying, page size, and windowed
layers (configuration C, whose q width 4*48 also differs from its hidden size).
Configuration D has head size 64, which the fastest attention kernels take; E has head
size 128, a long position limit and weights that make the attention peaked.
"""

from __future__ import annotations

import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import plain_model

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 172, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "torch_dtype": "float32", "eos_token_id": 255,
    "use_sliding_window": False,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "torch_dtype": "float32", "eos_token_id": [510, 511],
    "use_sliding_window": False,
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 120, "vocab_size": 300,
    "rope_theta": 500000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 384, "torch_dtype": "float32", "eos_token_id": 299,
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 2,
}
# head size 64: the tensor-core kernels that the large shapes use (tcgen05 prefill, one-launch
# decode from the q|k|v product) run inside a tiny model, one layer of it windowed
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 72, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 200, "vocab_size": 384,
    "rope_theta": 20000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 320, "torch_dtype": "float32", "eos_token_id": 383,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
# head size 128 and a position limit beyond 768, so that the kernels of the benchmark's shape
# run inside a tiny model and a request can be long enough for its decode steps to be split
# over the keys; its queries and keys are drawn large (``PEAKED``): the scores then have a
# standard deviation of several units, the softmax is peaked, and a key that is lost, seen
# twice or rotated by the wrong angle moves the logits far beyond bfloat16 rounding
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 208, "vocab_size": 320,
    "rope_theta": 100000.0, "rms_norm_eps": 4e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 1280, "torch_dtype": "float32", "eos_token_id": 319,
    "use_sliding_window": False,
}
PEAKED = {"q_proj.weight": 0.2, "k_proj.weight": 0.2, "v_proj.weight": 0.1, "lm_head.weight": 0.1,
          "embed_tokens.weight": 0.1}
CONFIGS = {"A": (TINY_A, 0, 16), "B": (TINY_B, 2, 8), "C": (TINY_C, 7, 16),
           "D": (TINY_D, 11, 8), "E": (TINY_E, 13, 16)}  # cfg, seed, page
STD_OF = {"E": PEAKED}           # per-tensor standard deviations of a configuration's weights


def make_model(folder: str, cfg: dict, seed: int, std_of=None) -> str:
    from servelab_b200.config import config_from_dict
    from servelab_b200.weights import write_random_model
    if std_of is None:
        std_of = next((STD_OF[k] for k, v in CONFIGS.items() if v[0] is cfg and k in STD_OF), None)
    return write_random_model(folder, config_from_dict(cfg), seed, std_of=std_of)


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(folder: str, ids: Sequence[int], dtype=torch.float32) -> np.ndarray:
    cfg, w = plain_model.load_folder(folder, dtype)
    return plain_model.forward_logits(cfg, w, ids).to(torch.float32).numpy()


# ------------------------------------------------------------------ traces
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for rid, ids in requests.items():
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def trace_bulk_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps = []
    for rid, ids in requests.items():
        n = max(1, len(ids) - tail)
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": ids[:n], "want": list(range(n))}], "end": []})
        for i in range(n, len(ids)):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": [ids[i]], "want": [0]}],
                "end": [rid] if i == len(ids) - 1 else []})
    return steps


PORTIONS = [7, 2, 16, 3, 2, 5, 33, 2, 9, 2, 17, 4]


def trace_portions(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for k, (rid, ids) in enumerate(requests.items()):
        pos, j = 0, k
        while pos < len(ids):
            n = PORTIONS[j % len(PORTIONS)]
            j += 1
            if len(ids) - pos - n == 1:     # never leave a single token for a "portion"
                n += 1
            n = min(n, len(ids) - pos)
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}],
                "end": [rid] if pos + n == len(ids) else []})
            pos += n
    return steps


def trace_mixed(requests: Dict[str, List[int]], seed: int, max_live: int = 4,
                tail: int = 32) -> List[dict]:
    """Up to ``max_live`` requests at a time; each step every live request either
    sits out, feeds a prompt portion (2..20 tokens) or, in its last ``tail``
    tokens, a single token; finished requests end and the next one starts."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: List[Tuple[str, List[int], int]] = []
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live.append((rid, ids, 0))
        entries, ends, nxt = [], [], []
        for rid, ids, pos in live:
            if rng.random() < 0.2 and len(live) > 1 and len(entries) + 1 < len(live):
                nxt.append((rid, ids, pos))
                continue
            left = len(ids) - pos
            if left <= tail:
                n = 1
            else:
                n = min(rng.randint(2, 20), left - tail)
                if n == 1:
                    n = 2 if left - tail >= 2 else 1
            entries.append({"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))})
            if pos + n == len(ids):
                ends.append(rid)
            else:
                nxt.append((rid, ids, pos + n))
        live = nxt
        if entries:
            rng.shuffle(entries)
            steps.append({"step": len(steps), "entries": entries, "end": ends})
    return steps


def peak_tokens(steps: List[dict], round_to: int = 64) -> int:
    """--max-tokens a trace needs: the peak over steps of the live requests'
    token counts, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: List[dict], outputs: Dict[int, np.ndarray], vocab: int) -> Dict[str, Dict[int, np.ndarray]]:
    """(request -> position -> logits row) from per-step outputs."""
    held: Dict[str, int] = {}
    got: Dict[str, Dict[int, np.ndarray]] = {}
    for st in steps:
        out = outputs.get(st["step"])
        row = 0
        for e in st["entries"]:
            start = held.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[start + w] = out[row]
                row += 1
            held[e["id"]] = start + len(e["tokens"])
        if out is not None:
            assert row == out.shape[0] and out.shape[1] == vocab
        for rid in st["end"]:
            held.pop(rid, None)
    return got


def run_session(session, steps: List[dict]) -> Dict[int, np.ndarray]:
    outputs = {}
    for st in steps:
        res = session.run_step(st)
        if res is not None:
            outputs[st["step"]] = res.copy()
    return outputs

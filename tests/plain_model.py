"""Plain, slow, whole-sequence implementation of the Qwen2 dense decoder.

This file is the tests' oracle.  It shares no code with the product path
(``servelab_b200``): it reads a model folder by itself, keeps no cache, and runs
a whole sequence at once on the CPU with one small function per part.

It rests on the formulas of the reference's in-tree restatements of its decoder
(the reference's own ``servelab/models`` package is absent from its tree, so it
cannot be imported and compared here); every function cites the lines it was
written from, as paths inside the reference project.

All arithmetic runs in the dtype of the tensors handed in (float32 by default,
float64 on request) so that faults hidden by bfloat16 show.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

# --------------------------------------------------------------------------- #
# reading a model folder (own reader: no code shared with the product loader)
# --------------------------------------------------------------------------- #

_ST_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "F64": torch.float64, "I32": torch.int32, "I64": torch.int64,
}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Read every tensor of one safetensors file (8-byte header length, JSON
    header with dtype/shape/data_offsets, then raw little-endian data)."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        t = torch.frombuffer(bytearray(blob[base + lo:base + hi]), dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder: str, dtype: torch.dtype = torch.float32):
    """Return (config dict, tensors converted to ``dtype``) of a model folder."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = read_safetensors(os.path.join(folder, "model.safetensors"))
    return cfg, {k: v.to(dtype) for k, v in raw.items()}


# --------------------------------------------------------------------------- #
# one function per part
# --------------------------------------------------------------------------- #

def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """hidden[t] = E[ids[t]]  (servelab/parallel/tp_model.py:123,
    scripts/debug/debug_layer_bisect.py:42)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, no bias, no mean-centering
    (tests/test_triton_kernels.py:57-59;
    servelab/attention/triton/paged_attention.py:86-91)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor,
           bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b), weights stored [out, in]
    (servelab/parallel/tp_model.py:48-53, tests/helpers_tiny_model.py:37-46)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_i = theta^(-2i/D), built in float32
    (servelab/parallel/tp_model.py:94-95)."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """NeoX rotate-half on [T, heads, D]: with x = [x1 | x2] (halves),
    x' = [x1 cos - x2 sin | x2 cos + x1 sin], angle = pos * inv_freq
    (docs/architecture.md:69, docs/knowledge_checklist.md:12; call site
    servelab/parallel/tp_model.py:128).  The angle is formed in float32."""
    ang = positions.to(torch.float32)[:, None] * inv_freq.to(positions.device)[None, :]   # [T, D/2]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None) -> torch.Tensor:
    """Whole-sequence grouped-query attention, q [T,H,D], k/v [T,Hkv,D].

    Query head j uses kv head j // g; scores = q.k * D^-1/2; key r is masked
    for query a when r > a; softmax over keys; o = P.v
    (servelab/parallel/tp_model.py:136-157, servelab/engine/speculative.py:72-84).
    ``window`` (not in the reference, which has no windowed layers) further
    masks keys with a - r >= window.
    """
    T, H, D = q.shape
    g = H // k.shape[1]
    k = k.repeat_interleave(g, dim=1)
    v = v.repeat_interleave(g, dim=1)
    scores = torch.einsum("qhd,rhd->hqr", q, k) * (1.0 / math.sqrt(D))
    a = torch.arange(T, device=q.device)[:, None]
    r = torch.arange(T, device=q.device)[None, :]
    mask = r > a
    if window is not None:
        mask = mask | (a - r >= window)
    scores = scores.masked_fill(mask[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqr,rhd->qhd", probs, v).reshape(T, H * D)


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
           w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z), no biases
    (servelab/parallel/tp_model.py:67-68)."""
    gate = linear(x, w_gate)
    return linear(gate * torch.sigmoid(gate) * linear(x, w_up), w_down)


# --------------------------------------------------------------------------- #
# the whole model
# --------------------------------------------------------------------------- #

def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Window of a layer from the Qwen2 config keys.  The reference reads none
    of them (servelab/config.py:48-72); the rule is the keys' documented
    meaning: with use_sliding_window, layers >= max_window_layers see only the
    last sliding_window keys."""
    if not cfg.get("use_sliding_window", False):
        return None
    if layer < cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return None
    return int(cfg["sliding_window"])


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] of one whole sequence, no cache
    (layer body: servelab/parallel/tp_model.py:121-134; LM head and tying:
    servelab/parallel/tp_model.py:112-119)."""
    H = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", H)
    D = cfg.get("head_dim", cfg["hidden_size"] // H)
    eps = cfg["rms_norm_eps"]
    inv_freq = rope_inv_freq(D, cfg.get("rope_theta", 1000000.0))
    device = w["model.embed_tokens.weight"].device          # tensors may live on any device
    ids_t = torch.tensor(list(ids), dtype=torch.long, device=device)
    T = ids_t.numel()
    pos = torch.arange(T, device=device)

    hidden = embed(ids_t, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        residual = hidden
        x = rms_norm(hidden, w[p + "input_layernorm.weight"], eps)
        q = linear(x, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, H, D)
        k = linear(x, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, Hkv, D)
        v = linear(x, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, Hkv, D)
        q = rope(q, pos, inv_freq)
        k = rope(k, pos, inv_freq)
        attn = causal_attention(q, k, v, layer_window(cfg, i))
        hidden = residual + linear(attn, w[p + "self_attn.o_proj.weight"])
        residual = hidden
        x = rms_norm(hidden, w[p + "post_attention_layernorm.weight"], eps)
        hidden = residual + swiglu(x, w[p + "mlp.gate_proj.weight"],
                                   w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    hidden = rms_norm(hidden, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(hidden, head)


# --------------------------------------------------------------------------- #
# sampling (host mirror of the engine's counter-based sampler)
# --------------------------------------------------------------------------- #

def greedy_token(logits: torch.Tensor) -> int:
    """argmax, the first index among equal maxima (servelab/engine/sampler.py:23-24)."""
    return int(torch.argmax(logits).item())


_M32 = 0xFFFFFFFF


def _mulhilo(a: int, b: int):
    p = a * b
    return (p >> 32) & _M32, p & _M32


def philox_uniform(seed: int, stream: int, counter: int) -> float:
    """Philox-4x32-10 keyed by the 64-bit ``seed``, counter words
    (counter, stream_lo, stream_hi, 0); the first output word becomes a float
    in [0, 1) with 24 bits.  Written from the published Philox constants; the
    engine's device sampler uses the same construction, so that a draw depends
    only on (seed, request stream, output position) and not on the batch.
    The reference instead draws from one CPU generator in batch order
    (servelab/engine/sampler.py:11-13,29-45)."""
    k0, k1 = seed & _M32, (seed >> 32) & _M32
    c = [counter & _M32, stream & _M32, (stream >> 32) & _M32, 0]
    for _ in range(10):
        hi0, lo0 = _mulhilo(0xD2511F53, c[0])
        hi1, lo1 = _mulhilo(0xCD9E8D57, c[2])
        c = [(hi1 ^ c[1] ^ k0) & _M32, lo1, (hi0 ^ c[3] ^ k1) & _M32, lo0]
        k0 = (k0 + 0x9E3779B9) & _M32
        k1 = (k1 + 0xBB67AE85) & _M32
    return (c[0] >> 8) * (1.0 / 16777216.0)


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int = -1,
                   top_p: float = 1.0) -> torch.Tensor:
    """softmax(logits / max(T, 1e-6)); then top-k (keep the k largest,
    renormalise) OR ELSE top-p (sort descending, drop entries whose inclusive
    cumulative sum exceeds p, except the first; renormalise)
    (servelab/engine/sampler.py:29-45: top-k takes precedence over top-p)."""
    probs = torch.softmax(logits.double() / max(temperature, 1e-6), dim=-1)
    if top_k > 0:
        k = min(top_k, probs.numel())
        kth = torch.topk(probs, k).values[-1]
        probs = torch.where(probs >= kth, probs, torch.zeros_like(probs))
    elif top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cut = torch.cumsum(sp, dim=-1) > top_p
        cut[0] = False
        sp[cut] = 0.0
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
    return probs / probs.sum()


def sample_token(logits: torch.Tensor, temperature: float, u: float,
                 top_k: int = -1, top_p: float = 1.0) -> int:
    """Inverse-CDF draw in index order: the first index whose inclusive
    cumulative probability exceeds u."""
    if temperature == 0.0:
        return greedy_token(logits)
    cdf = torch.cumsum(filtered_probs(logits, temperature, top_k, top_p), dim=-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype), right=True).item())
    return min(idx, logits.numel() - 1)


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int],
                    max_tokens: int) -> List[int]:
    """Greedy continuation by full recomputation each token (the reference's
    cross-check runner does the same with a growing cache,
    servelab/engine/speculative.py:89-97)."""
    ids = list(prompt)
    out = []
    for _ in range(max_tokens):
        tok = greedy_token(forward_logits(cfg, w, ids)[-1])
        out.append(tok)
        ids.append(tok)
    return out

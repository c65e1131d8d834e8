"""The plain implementation checked against itself and its golden file (CPU)."""

import importlib.util
import math
import os

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as P

HERE = os.path.dirname(os.path.abspath(__file__))


def test_golden_file_still_matches():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    now = mod.compute()
    gold = np.load(os.path.join(HERE, "golden", "plain_tiny.npz"))
    # every configuration of the tests, not whatever the file happens to hold
    assert sorted(gold.files) == sorted(f"{name}_{what}" for name in H.CONFIGS for what in ("ids", "logits_rows"))
    for name, (cfg, _, _) in H.CONFIGS.items():
        scale = float(np.abs(gold[f"{name}_logits_rows"]).max())
        assert np.array_equal(now[f"{name}_ids"], gold[f"{name}_ids"]), name
        np.testing.assert_allclose(now[f"{name}_logits_rows"], gold[f"{name}_logits_rows"], rtol=0,
                                   atol=2e-6 * max(1.0, scale), err_msg=name)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[6.0 / r, 2.0 / r]]))
    w = torch.eye(2)
    out = P.swiglu(torch.tensor([[1.0, -2.0]]), w, w, w)
    silu = lambda z: z / (1 + math.exp(-z))
    assert torch.allclose(out, torch.tensor([[silu(1.0) * 1.0, silu(-2.0) * -2.0]]))


def test_rope_is_a_rotation_of_half_pairs_and_relative():
    inv = P.rope_inv_freq(8, 10000.0)
    assert torch.allclose(inv, torch.tensor([1.0, 0.1, 0.01, 0.001]))
    x = torch.randn(5, 2, 8)
    pos = torch.arange(5)
    y = P.rope(x, pos, inv)
    assert torch.allclose(y[0], x[0])                              # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    a = 3 * inv[1]
    assert torch.allclose(y[3, 0, 1], x[3, 0, 1] * torch.cos(a) - x[3, 0, 5] * torch.sin(a), atol=1e-6)
    assert torch.allclose(y[3, 0, 5], x[3, 0, 5] * torch.cos(a) + x[3, 0, 1] * torch.sin(a), atol=1e-6)
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    d1 = (P.rope(q, torch.tensor([7]), inv) * P.rope(k, torch.tensor([4]), inv)).sum()
    d2 = (P.rope(q, torch.tensor([13]), inv) * P.rope(k, torch.tensor([10]), inv)).sum()
    assert torch.allclose(d1, d2, atol=1e-5)                       # depends on distance only


def test_attention_is_causal_grouped_and_windowed():
    T, H_, Hkv, D = 6, 4, 2, 8
    q, k, v = torch.randn(T, H_, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    out = P.causal_attention(q, k, v).view(T, H_, D)
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)          # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    out2 = P.causal_attention(q, k2, v2).view(T, H_, D)
    assert torch.allclose(out[:4], out2[:4])                      # the future does not leak
    s = (q[5, 2] @ k[:, 1].t()) / math.sqrt(D)                    # head 2 reads kv head 1
    ref = torch.softmax(s, -1) @ v[:, 1]
    assert torch.allclose(out[5, 2], ref, atol=1e-6)
    w = P.causal_attention(q, k, v, window=2).view(T, H_, D)
    s2 = (q[5, 0] @ k[4:6, 0].t()) / math.sqrt(D)
    assert torch.allclose(w[5, 0], torch.softmax(s2, -1) @ v[4:6, 0], atol=1e-6)


def test_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    folder = H.make_model(str(tmp_path), H.TINY_C, 7)
    cfg, w = P.load_folder(folder)
    ids = H.random_ids(50, cfg["vocab_size"], 1)
    full = P.forward_logits(cfg, w, ids)
    part = P.forward_logits(cfg, w, ids[:31])
    assert torch.allclose(full[:31], part, atol=1e-6)
    assert P.layer_window(cfg, 1) is None and P.layer_window(cfg, 2) == 24
    f64 = P.forward_logits(cfg, {k: v.double() for k, v in w.items()}, ids)
    assert float((f64.float() - full).abs().max()) < 1e-5


def test_sampling_mirror():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0, 0.5])
    assert P.greedy_token(logits) == 1                             # first of equal maxima
    u = [P.philox_uniform(5, 1, i) for i in range(2000)]
    assert all(0.0 <= x < 1.0 for x in u) and abs(np.mean(u) - 0.5) < 0.03
    assert P.philox_uniform(5, 1, 0) != P.philox_uniform(5, 2, 0) != P.philox_uniform(6, 1, 0)
    p = P.filtered_probs(logits, 1.0, top_k=2)
    assert p[0] == 0 and abs(float(p[1]) - 0.5) < 1e-9
    p = P.filtered_probs(logits, 1.0, top_p=0.5)
    assert int((p > 0).sum()) == 1                                 # only the first survives
    counts = np.zeros(5)
    for i in range(4000):
        counts[P.sample_token(logits, 0.7, P.philox_uniform(1, 0, i))] += 1
    want = torch.softmax(logits.double() / 0.7, -1).numpy()
    assert np.abs(counts / 4000 - want).max() < 0.03

"""The kernels at the benchmark's layer sizes (Qwen2.5-7B shape: hidden 3584, 28
heads in 4 groups of 7, head size 128, intermediate 18944, vocabulary 152064),
with two layers so that it stays small.  float32 against the plain implementation
(run with the same tensors on the GPU in plain float32 torch operations, TF32 off),
bit-identical logits however the prompt is cut, and bfloat16 within tolerance."""

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as P

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2,
    "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
    "use_sliding_window": False,
}
LENGTHS = [150, 67, 300]


@pytest.fixture(scope="module")
def big():
    from servelab_b200.config import config_from_dict
    from servelab_b200.models import declare_tensors
    from servelab_b200.weights import RandomSource
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    config = config_from_dict(SHAPE)
    source = RandomSource(declare_tensors(config.to_model_spec()), seed=0, device="cuda:0",
                          dtype=torch.float32)
    reqs = {f"q{i}": H.random_ids(n, SHAPE["vocab_size"], 70 + i) for i, n in enumerate(LENGTHS)}
    w = {n: source.read(n) for n in source.names()}
    with torch.no_grad():
        ref = {rid: P.forward_logits(SHAPE, w, ids).float().cpu().numpy() for rid, ids in reqs.items()}
    del w
    torch.cuda.empty_cache()
    return {"config": config, "source": source, "reqs": reqs, "ref": ref}


def _run(big, dtype, steps):
    from servelab_b200.config import CacheConfig
    from servelab_b200.engine.runner import ModelRunner
    from servelab_b200.replay import TraceSession
    sess = TraceSession.__new__(TraceSession)
    sess.max_tokens, sess.max_live = H.peak_tokens(steps), 4
    sess.runner = ModelRunner(big["config"], big["source"], dtype=dtype,
                              cache_config=CacheConfig(block_size=16, num_blocks=sess.max_tokens // 16),
                              max_num_seqs=4)
    sess.cache, sess.held = sess.runner.cache, {}
    got = H.collect(steps, H.run_session(sess, steps), SHAPE["vocab_size"])
    sess.cache.check_invariants()
    del sess
    torch.cuda.empty_cache()
    return got


def _worst(big, got):
    worst = 0.0
    for rid, ids in big["reqs"].items():
        for pos in range(len(ids)):
            worst = max(worst, float(np.abs(got[rid][pos] - big["ref"][rid][pos]).max()))
    return worst


def test_float32_matches_plain_and_is_cut_invariant(big):
    whole = _run(big, "float32", H.trace_whole(big["reqs"]))
    err = _worst(big, whole)
    scale = max(float(np.abs(r).max()) for r in big["ref"].values())
    print(f"7B-shape float32: worst abs logit error {err:.3e} (largest logit {scale:.2f})")
    assert err <= 1e-3
    mixed = _run(big, "float32", H.trace_mixed(big["reqs"], seed=9, max_live=3))
    tail = _run(big, "float32", H.trace_bulk_tail(big["reqs"]))
    for rid in whole:
        for pos in whole[rid]:
            assert np.array_equal(whole[rid][pos], mixed[rid][pos]), (rid, pos)
            assert np.array_equal(whole[rid][pos], tail[rid][pos]), (rid, pos)


def test_bfloat16_within_tolerance_in_every_mode(big):
    # logits here reach |7|; bfloat16 rounds every activation to 8 bits of mantissa
    # (0.4 % each), so the bound is relative to the largest logit: 3 % of it
    scale = max(float(np.abs(r).max()) for r in big["ref"].values())
    for name, steps in (("whole", H.trace_whole(big["reqs"])),
                        ("bulk+tail", H.trace_bulk_tail(big["reqs"])),
                        ("portions", H.trace_portions(big["reqs"])),
                        ("mixed", H.trace_mixed(big["reqs"], seed=9, max_live=3))):
        err = _worst(big, _run(big, "bfloat16", steps))
        print(f"7B-shape bfloat16 {name}: worst abs logit error {err:.3e} (largest logit {scale:.2f})")
        assert err <= 0.03 * scale, name

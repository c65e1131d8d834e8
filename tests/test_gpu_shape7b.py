"""The kernels at the benchmark's layer sizes (Qwen2.5-7B shape: hidden 3584, 28
heads in 4 groups of 7, head size 128, intermediate 18944, vocabulary 152064),
with two layers so that it stays small.  float32 against the plain implementation
(run with the same tensors on the GPU in plain float32 torch operations, TF32 off),
bit-identical logits however the prompt is cut, and bfloat16 within tolerance.

The second half runs where the benchmark runs: requests of 2,100 to 2,400 tokens whose
decoded tokens sit beyond 2,048 keys (the decode kernel then splits every request and the
block that arrives last combines the splits; rotation angles are in the thousands), the same
through replayed CUDA graphs, and steps of more than 16 single tokens (where the narrow
products leave this package's kernels for the library's)."""

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
LONG = [2150, 2400, 2290]
TAIL = 32                 # tokens of a long request decoded one by one
KEEP = TAIL + 8           # rows of a long request whose logits are compared (its end)
MANY = 22                 # live requests of the wide decode steps


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
    long = {f"L{i}": H.random_ids(n, SHAPE["vocab_size"], 170 + i) for i, n in enumerate(LONG)}
    many = {f"m{i:02d}": H.random_ids(24 + 3 * i, SHAPE["vocab_size"], 270 + i) for i in range(MANY)}
    w = {n: source.read(n) for n in source.names()}
    with torch.no_grad():
        ref = {rid: P.forward_logits(SHAPE, w, ids).float().cpu().numpy() for rid, ids in reqs.items()}
        ref.update({rid: P.forward_logits(SHAPE, w, ids).float().cpu().numpy() for rid, ids in many.items()})
        # of a long request only the last rows are kept (a whole one is 1.4 GB of logits)
        long_ref = {rid: P.forward_logits(SHAPE, w, ids)[-KEEP:].float().cpu().numpy()
                    for rid, ids in long.items()}
    del w
    torch.cuda.empty_cache()
    return {"config": config, "source": source, "reqs": reqs, "ref": ref, "long": long,
            "long_ref": long_ref, "many": many}


def _run(big, dtype, steps, max_live=4, cuda_graphs=False):
    from servelab_b200.config import CacheConfig
    from servelab_b200.engine.runner import ModelRunner
    from servelab_b200.replay import TraceSession
    max_tokens = H.peak_tokens(steps)
    runner = ModelRunner(big["config"], big["source"], dtype=dtype,
                         cache_config=CacheConfig(block_size=16, num_blocks=max_tokens // 16,
                                                  poison_cache=True),
                         max_num_seqs=max_live, cuda_graphs=cuda_graphs)
    sess = TraceSession(None, dtype, max_tokens, max_live=max_live, runner=runner)
    got = H.collect(steps, H.run_session(sess, steps), SHAPE["vocab_size"])
    sess.cache.check_invariants()
    del sess
    torch.cuda.empty_cache()
    return got


def _worst(big, got, which="reqs"):
    worst = 0.0
    for rid, ids in big[which].items():
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


# ------------------------------------------------- where the benchmark runs
def _long_trace(reqs, cuts=None):
    """Each request alone: all but the last TAIL tokens in one step (or cut at ``cuts``), the
    rest one by one; logits wanted for the last KEEP positions only."""
    steps = []
    for rid, ids in reqs.items():
        n = len(ids) - TAIL
        edges = [0] + [c for c in (cuts or []) if c < n] + [n]
        for a, b in zip(edges, edges[1:]):
            want = [p - a for p in range(max(a, len(ids) - KEEP), b)]
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[a:b], "want": want}],
                          "end": []})
        for i in range(n, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}],
                          "end": [rid] if i == len(ids) - 1 else []})
    return steps


def _long_worst(big, got):
    worst = 0.0
    for rid, ids in big["long"].items():
        first = len(ids) - KEEP
        assert sorted(got[rid]) == list(range(first, len(ids))), rid
        for pos in range(first, len(ids)):
            worst = max(worst, float(np.abs(got[rid][pos] - big["long_ref"][rid][pos - first]).max()))
    return worst


def test_long_contexts_float32_match_plain_and_are_cut_invariant(big):
    a = _run(big, "float32", _long_trace(big["long"]), max_live=2)
    err = _long_worst(big, a)
    print(f"7B-shape float32, contexts {LONG}: worst abs logit error {err:.3e}")
    assert err <= 1e-3
    b = _run(big, "float32", _long_trace(big["long"], cuts=[700, 702, 1601, 2047]), max_live=2)
    for rid in a:
        for pos in a[rid]:
            assert np.array_equal(a[rid][pos], b[rid][pos]), (rid, pos)


def test_long_contexts_bfloat16_split_decode_eager_and_graphs(big):
    """Decoded tokens beyond 2,048 keys: every request is split over several blocks (asserted
    through the kernel's own counter), eagerly and through replayed graphs, whose launches are
    sized for the longest request the engine admits, and with the plain twin kernels."""
    from servelab_b200.ops import attention as A
    from servelab_b200.ops import kernels as K
    from servelab_b200.ops import linear as linear_ops
    scale = max(float(np.abs(r).max()) for r in big["long_ref"].values())
    D = SHAPE["head_dim"]
    steps = _long_trace(big["long"])
    outs = {}
    for name, graphs in (("eager", False), ("graphs", True)):
        K.decode_attention_splits_used(D, reset=True)
        outs[name] = _run(big, "bfloat16", steps, max_live=2, cuda_graphs=graphs)
        used = K.decode_attention_splits_used(D, reset=True)
        assert used > 1, f"{name}: no request was split"
        assert K.decode_attention_status(D, reset=True) == 0 and K.gemm_tc_status(True) == 0
        err = _long_worst(big, outs[name])
        print(f"7B-shape bfloat16 {name}, contexts {LONG}: worst abs logit error {err:.3e} "
              f"(largest logit {scale:.2f}, most splits {used})")
        assert err <= 0.03 * scale, name
    A.force_generic, saved = True, linear_ops.cluster_sums
    linear_ops.cluster_sums = False
    try:
        plain = _run(big, "bfloat16", steps, max_live=2)
    finally:
        A.force_generic, linear_ops.cluster_sums = False, saved
    assert _long_worst(big, plain) <= 0.03 * scale
    # the fast and the plain kernels see the same rounded inputs: they agree more closely
    # with one another than either does with float32
    worst = max(float(np.abs(outs["graphs"][rid][pos] - plain[rid][pos]).max())
                for rid in plain for pos in plain[rid])
    print(f"7B-shape bfloat16 graphs against the plain twin kernels: {worst:.3e}")
    assert worst <= 0.02 * scale


def _wide_trace(reqs, decode_steps=12):
    """All requests live at once: prompts in steps of several portions, then ``decode_steps``
    steps in which every request feeds one token (steps of len(reqs) single tokens)."""
    steps, items = [], list(reqs.items())
    for k in range(0, len(items), 5):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": ids[:len(ids) - decode_steps],
             "want": list(range(len(ids) - decode_steps))} for rid, ids in items[k:k + 5]]})
    for j in range(decode_steps, 0, -1):
        steps.append({"step": len(steps), "end": list(reqs) if j == 1 else [], "entries": [
            {"id": rid, "tokens": [ids[len(ids) - j]], "want": [0]} for rid, ids in items]})
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_more_than_sixteen_requests(big, dtype):
    """22 live requests: their decode steps have 22 tokens, where the q|k|v and o products go to
    the library's GEMM and the down product to the cluster form; eagerly and through graphs."""
    from servelab_b200.ops import kernels as K
    steps = _wide_trace(big["many"])
    scale = max(float(np.abs(big["ref"][rid]).max()) for rid in big["many"])
    bound = 1e-3 if dtype == "float32" else 0.03 * scale
    for graphs in (False, True):
        got = _run(big, dtype, steps, max_live=MANY + 2, cuda_graphs=graphs)
        err = _worst(big, got, "many")
        print(f"7B-shape {dtype}, {MANY} live requests (graphs={graphs}): worst abs logit error {err:.3e}")
        assert err <= bound
        assert K.gemm_tc_status(True) == 0

"""Which kernel a matrix product of a step goes to (``ops.linear.which_kernel``), decided
on the host from shapes alone: checked here without a GPU for the layer sizes of the three
large shapes, with the SM count of a B200."""

import pytest
import torch

from servelab_b200.ops import kernels as K
from servelab_b200.ops import linear as L

SHAPES = {  # hidden, q width, q|k|v width, intermediate, vocabulary
    "0.5b": (896, 896, 1152, 4864, 151936),
    "7b": (3584, 3584, 4608, 18944, 152064),
    "14b": (5120, 5120, 7168, 13824, 152064),
}


@pytest.fixture(autouse=True)
def b200(monkeypatch):
    monkeypatch.setattr(K, "_sm_count", 148)


def _ops(m, n, k, dtype=torch.bfloat16):
    return (torch.empty((m, k), dtype=dtype, device="meta"), torch.empty((n, k), dtype=dtype, device="meta"))


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_decode_steps_run_this_package_s_tensor_core_kernels(shape):
    h, q, qkv, inter, vocab = SHAPES[shape]
    for m in (1, 8, 16):
        assert L.which_kernel(*_ops(m, qkv, h)) == "tc_cluster"
        assert L.which_kernel(*_ops(m, h, q)) == "tc_cluster"
        if shape == "0.5b":      # 76 row tiles: three K splits still fit; the activation is a kernel
            assert L.which_kernel(*_ops(m, 2 * inter, h)) == "tc_cluster"
        else:                    # wide: no K split, the activation in the product's epilogue
            assert L.which_kernel(*_ops(m, 2 * inter, h)) == "tc"
            assert K.tc_decode_splits(2 * inter, h) == 1
        assert L.which_kernel(*_ops(m, vocab, h), out_dtype=torch.float32) == "tc"
    # Above 16 tokens the cluster form stays while a block finishes at most 8 tokens in its
    # epilogue: 8 K splits (7B: every narrow product) reach 64 tokens.  Matrices of at most 20 MB
    # (every one of the 0.5B shape) are instead read once per group of 16 tokens, so a block
    # never sees more than 16: they stay on this package's kernels up to 64 tokens too.
    kinds = {m: L.which_kernel(*_ops(m, h, inter)) for m in (8, 32, 64, 65)}
    assert kinds == {8: "tc_cluster", 32: "tc_cluster", 64: "tc_cluster", 65: "vendor"}   # down: 7 to 8 splits
    if shape == "0.5b":
        for n, k in ((qkv, h), (h, q), (h, inter)):
            w = _ops(64, n, k)[1]
            assert K.tc_token_groups(64, w) == 4 and K.tc_token_groups(16, w) == 1
            assert L.which_kernel(*_ops(64, n, k)) == "tc_cluster" and L.which_kernel(*_ops(65, n, k)) == "vendor"
        # gate|up: 76 row tiles x 4 groups fill the GPU without a K split: the activation is fused
        assert L.which_kernel(*_ops(64, 2 * inter, h)) == "tc"
        assert K.tc_decode_splits(2 * inter, h, 4) == 1
    else:
        for n, k in ((qkv, h), (h, q)):
            assert K.tc_token_groups(64, _ops(64, n, k)[1]) == 1
            splits = min(K.tc_decode_splits(n, k), K.TC_MAX_CLUSTER)
            reach = min(64, 8 * splits)
            assert L.which_kernel(*_ops(max(16, reach), n, k)) == "tc_cluster"
            assert L.which_kernel(*_ops(max(16, reach) + 1, n, k)) == "vendor"
    if shape == "7b":
        assert L.which_kernel(*_ops(64, qkv, h)) == "tc_cluster" and L.which_kernel(*_ops(64, h, q)) == "tc_cluster"


def test_many_tokens_go_to_the_vendor_gemm_and_ragged_or_float32_ones_to_cuda_cores():
    h, q, qkv, inter, vocab = SHAPES["7b"]
    for m in (65, 512, 2048):
        for n, k in ((qkv, h), (h, q), (2 * inter, h), (h, inter)):
            assert L.which_kernel(*_ops(m, n, k)) == "vendor"
    assert L.which_kernel(*_ops(100, 172, 64)) == "simt"                    # 172 rows: not a multiple of 8
    assert L.which_kernel(*_ops(40, 172, 64)) == "tc"                       # ... which the tcgen05 kernel takes
    assert L.which_kernel(*_ops(3, 64, 172)) == "simt"                      # K = 172: rows not 16-byte aligned
    assert L.which_kernel(*_ops(8, h, q, torch.float32)) == "simt"          # the 32-bit path
    assert L.which_kernel(*_ops(0, h, q)) == "empty"
    # gate|up and the LM head stay on the tcgen05 kernel up to 64 tokens
    assert L.which_kernel(*_ops(64, 2 * inter, h)) == "tc"


def test_switches_change_the_decision(monkeypatch):
    h, q, qkv, inter, vocab = SHAPES["7b"]
    monkeypatch.setattr(L, "cluster_max_tokens_per_block", 2)
    assert L.which_kernel(*_ops(16, h, q)) == "tc_cluster" and L.which_kernel(*_ops(17, h, q)) == "vendor"
    assert L.which_kernel(*_ops(64, h, inter)) == "tc_cluster"          # long K ranges keep it
    monkeypatch.setattr(L, "cluster_sums", False)
    assert L.which_kernel(*_ops(8, h, q)) == "tc"
    assert L.which_kernel(*_ops(32, h, inter)) == "vendor"
    assert L.which_kernel(*_ops(17, h, q)) == "vendor"
    monkeypatch.setattr(L, "tc_max_tokens", 4)
    assert L.which_kernel(*_ops(8, h, q)) == "vendor"

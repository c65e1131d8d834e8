"""The arithmetic of the kernel microbenchmark's table (no GPU): achieved rates, which
roof binds, the fraction of it, how many copies a graph holds, and the two renderings."""

from servelab_b200.bench import kernel_bench as kb

PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def test_a_row_reports_rates_and_the_binding_roof():
    # 66.5 MB in 20 us: 3,325 GB/s, half of the memory roof; flops negligible
    r = kb.Row("copy", "case", 20.0, 66.5e6, 1e6, PEAKS)
    assert abs(r.gbs - 3325.0) < 1e-6 and r.bound == "hbm" and abs(r.frac - 0.5) < 1e-9
    # 1.59 TFLOP in 2 ms: 795 TFLOP/s, half of the MMA roof; bytes negligible
    r = kb.Row("gemm", "case", 2000.0, 1e6, 1.59e12, PEAKS)
    assert abs(r.tflops - 795.0) < 1e-6 and r.bound == "mma" and abs(r.frac - 0.5) < 1e-9
    assert r.cells()[0:2] == ["gemm", "case"] and r.cells()[-2:] == ["mma", "0.50"]


def test_copies_exceed_the_l2_cache_within_a_few_gigabytes():
    for nbytes in (1e5, 33e6, 272e6, 1.09e9, 4.3e9):
        n = kb.copies_for(nbytes)
        assert 4 <= n <= 28
        assert n * nbytes >= min(1e9, 4 * nbytes)           # several times the 126 MB cache
    assert kb.copies_for(1e5, least=8) == 28
    assert kb.copies_for(4.3e9) == 4


def test_renderings():
    rows = [kb.Row("k", "c", 10.0, 1e6, 0.0, PEAKS)]
    md = kb.render(rows, markdown=True).splitlines()
    assert md[0].startswith("| kernel | case | us |") and md[1].startswith("|---") and md[2].startswith("| k | c | 10.0 |")
    txt = kb.render(rows, markdown=False).splitlines()
    assert txt[0].split()[:3] == ["kernel", "case", "us"] and txt[1].split()[:3] == ["k", "c", "10.0"]
    assert kb._ints("1,8,64") == [1, 8, 64] and kb._ints("") == []

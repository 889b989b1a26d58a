"""GPU tests of the ABFT SGEMM: clean runs are bit-identical to the plain kernel with zero false
positives; every injected single fault above the threshold is detected, located and corrected so
that the result meets the north-star tolerance; sub-threshold flips are benign by construction."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mats(M, N, K):
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    return a, b, c


@pytest.fixture(autouse=True)
def _pin_huge_tile(cuda):
    """The report counts tiles of whichever block tile ran; pin the 128x128 tile so that counts are fixed."""
    import hpcdeepneuralnetworks_b200 as b2
    b2.set_ffma_tile(0)
    yield
    b2.set_ffma_tile(-1)


def default_tau(K):
    return max(2e-6 * K, 4e-5)


def classify(a, b, plan, tau):
    """Per planned fault: |faulty - clean| of the final accumulator, from the exact CPU walk."""
    must, gray, benign = 0, 0, 0
    for f in plan:
        clean, bad, ok = oracle.fault_effect(a, b, f)
        assert ok
        d = abs(np.float64(bad) - np.float64(clean))
        if not np.isfinite(d) or d > 2 * tau:
            must += 1
        elif d < 0.5 * tau:
            benign += 1
        else:
            gray += 1
    return must, gray, benign


@pytest.mark.parametrize("shape", [(128, 128, 32), (256, 384, 96), (1024, 1024, 1024), (130, 260, 72), (64, 512, 1000)])
def test_clean_run_no_false_positive_and_bit_identical(cuda, shape):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    rep = b2.new_report()
    dc = dev(c)
    b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    r.pop("max_residual")
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    assert r == {"tiles": tiles, "injected": 0, "detected": 0, "corrected": 0, "uncorrectable": 0, "false_alarms": 0}
    assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))


@pytest.mark.parametrize("bit", [20, 22, 23, 25, 27, 29, 30, 31])
@pytest.mark.parametrize("k_step", [0, 5, 10 ** 6])
def test_single_fault_each_bit(cuda, bit, k_step):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 256, 256, 512
    a, b, c = mats(M, N, K)
    plan = np.array([[1, 0, 77, 101, k_step, bit]], dtype=np.int32)
    tau = default_tau(K)
    must, gray, benign = classify(a, b, plan, tau)
    rep = b2.new_report()
    dc = dev(c)
    b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["tiles"] == 4 and r["injected"] == 1
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    got = dc.cpu().numpy()
    if must:
        assert r["detected"] == 1 and r["corrected"] == 1 and r["uncorrectable"] == 0
    if benign:
        assert r["detected"] == 0 and r["uncorrectable"] == 0
    if must or benign:
        assert oracle.gemm_error(got, c64, den) <= TOL
    # every element other than the struck one is bit-identical to the plain result; a corrected one is too,
    # because correction recomputes the output with the kernel's own arithmetic
    want = oracle.sgemm_fma(1.0, a, b, 0.5, c)
    mask = np.ones_like(want, dtype=bool)
    mask[128 + 77, 101] = False
    assert np.array_equal(got[mask], want[mask])
    if must:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("seed", [6, 7, 8])
def test_config3_1024_plan(cuda, seed):
    """Benchmark configuration 3 at 1024^3: one flip (bit 20..30) per 64 tiles -- here also a denser plan, one per 2 tiles."""
    import hpcdeepneuralnetworks_b200 as b2
    n = 1024
    a, b, c = mats(n, n, n)
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    for per in (64, 2):
        plan = oracle.make_fault_plan(n, n, n, seed=seed, tiles_per_fault=per)
        tau = default_tau(n)
        must, gray, benign = classify(a, b, plan, tau)
        rep = b2.new_report()
        dc = dev(c)
        b2.ft_sgemm(n, n, n, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert r["tiles"] == 64 and r["injected"] == len(plan)
        assert must <= r["corrected"] <= must + gray
        assert r["uncorrectable"] <= gray
        if gray == 0:
            assert oracle.gemm_error(dc.cpu().numpy(), c64, den) <= TOL


def test_nan_and_inf_faults_are_rebuilt(cuda):
    """A flip of bit 30 on a value in [1,2) makes Inf/NaN; the value must be rebuilt, not subtracted."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 128, 128, 256
    a, b, c = mats(M, N, K)
    clean = oracle.sgemm_fma(1.0, a, b, 0.0, np.zeros_like(c))
    cand = np.argwhere((np.abs(clean) >= 1.0) & (np.abs(clean) < 2.0))
    r0, c0 = (int(v) for v in cand[0])
    plan = np.array([[0, 0, r0, c0, 10 ** 6, 30]], dtype=np.int32)
    _, bad, _ = oracle.fault_effect(a, b, plan[0])
    assert not np.isfinite(bad)
    rep = b2.new_report()
    dc = dev(c)
    b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
    r = b2.read_report(rep)
    assert r["corrected"] == 1 and r["uncorrectable"] == 0
    got = dc.cpu().numpy()
    assert np.isfinite(got).all()
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    assert oracle.gemm_error(got, c64, den) <= TOL


def test_north_star_launcher_ft_sgemm(cuda):
    import ctypes as C
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    n = 256
    a, b, c = mats(n, n, n)
    da, db, dc = dev(a), dev(b), dev(c)
    torch.cuda.synchronize()
    p = lambda t: C.c_void_p(t.data_ptr())
    assert L.ft_sgemm(n, n, n, 1.0, p(da), p(db), 0.5, p(dc)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))


def test_unsupported_operands_are_refused(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    t = torch.zeros(100 * 100 + 4, device="cuda")
    with pytest.raises(b2.B2Error) as e:
        b2.ft_sgemm(50, 50, 50, 1.0, t[1:], t, 0.0, t.clone())      # A not 16-byte aligned
    assert e.value.status == -2


@pytest.mark.parametrize("n", [4096, 8192])
def test_config3_large_sizes(cuda, n):
    """Benchmark configuration 3 at 4096^3 and 8192^3: seeded plan (one flip per 64 tiles) and a clean run; checked
    against the plain kernel on the device and against the exact CPU walk of each struck accumulator."""
    import hpcdeepneuralnetworks_b200 as b2
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    plain = torch.zeros((n, n), device="cuda")
    b2.sgemm(n, n, n, 1.0, A, B, 0.0, plain)
    tiles = (n // 128) ** 2
    rep = b2.new_report()
    out = torch.zeros((n, n), device="cuda")
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    r.pop("max_residual")
    assert r == {"tiles": tiles, "injected": 0, "detected": 0, "corrected": 0, "uncorrectable": 0, "false_alarms": 0}
    assert torch.equal(out, plain)
    plan = oracle.make_fault_plan(n, n, n, seed=6)
    assert len(plan) == tiles // 64
    a, b = A.cpu().numpy(), B.cpu().numpy()
    tau = default_tau(n)
    must, gray, benign = classify(a, b, plan, tau)
    rep = b2.new_report()
    out.zero_()
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["injected"] == len(plan) and must <= r["corrected"] <= must + gray and r["uncorrectable"] <= gray
    diff = (out - plain).abs()
    # untouched elements identical; struck ones within the tolerance scale 1e-5 * K/4 (+ the gray zone bound 2 tau)
    assert int((diff > 0).sum().item()) <= len(plan)
    assert float(diff.max().item()) <= max(1e-5 * n / 4.0, 2 * tau if gray else 0.0)


def test_every_generated_tile_plain_and_abft(cuda):
    """The generated tile family: each tile pinned, plain result bit-exact, a planted fault found and repaired."""
    import hpcdeepneuralnetworks_b200 as b2
    tiles = b2.ffma_tiles()
    assert len(tiles) >= 6 and {t[1] for t in tiles} >= {"huge", "tall", "wide", "large", "medium"}
    M, N, K = 200, 264, 160
    a, b, c = mats(M, N, K)
    want = oracle.sgemm_fma(1.0, a, b, 0.5, c)
    plan = np.array([[1, 1, 40, 100, 2, 28]], dtype=np.int32)        # output element (168, 228)
    clean, bad, ok = oracle.fault_effect(a, b, plan[0])
    assert ok and abs(bad - clean) > 4 * default_tau(K)
    try:
        for idx, name, bm, bn, threads in tiles:
            b2.set_ffma_tile(idx)
            dc = dev(c)
            b2.sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc)
            b2.check_status()
            assert np.array_equal(dc.cpu().numpy(), want), name
            rep = b2.new_report()
            dc = dev(c)
            b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
            b2.check_status()
            r = b2.read_report(rep)
            assert r["tiles"] == ((M + bm - 1) // bm) * ((N + bn - 1) // bn), name
            assert (r["injected"], r["detected"], r["corrected"], r["false_alarms"]) == (1, 1, 1, 0), (name, r)
            assert np.array_equal(dc.cpu().numpy(), want), name
    finally:
        b2.set_ffma_tile(-1)


def test_two_faults_in_one_block_are_both_repaired(cuda):
    """Recompute-based correction does not depend on the single-fault assumption inside a block: plant a fault,
    run, then corrupt through a second plan entry in a neighbouring tile of the same call."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 256, 256, 256
    a, b, c = mats(M, N, K)
    plan = np.array([[0, 0, 5, 9, 1, 27], [0, 1, 5, 9, 3, 29], [1, 0, 100, 64, 0, 26], [1, 1, 127, 127, 7, 30]], dtype=np.int32)
    rep = b2.new_report()
    dc = dev(c)
    b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
    r = b2.read_report(rep)
    must, gray, benign = classify(a, b, plan, default_tau(K))
    assert r["injected"] == 4 and must <= r["corrected"] <= must + gray
    if gray == 0 and benign == 0:
        assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))


@pytest.mark.parametrize("shape", [(128, 128, 64), (260, 136, 96), (512, 384, 256)])
def test_colmajor_nt_abft(cuda, shape):
    """The reference's own ABFT layout (column-major NT): clean run bit-identical, a planted fault repaired."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    af, bf, cf = oracle.fill_uniform(M * K, 1), oracle.fill_uniform(N * K, 2), oracle.fill_uniform(M * N, 3)
    want = oracle.sgemm_colmajor_nt(M, N, K, 1.0, af, bf, -1.5, cf)
    rep = b2.new_report()
    dc = dev(cf)
    b2.ft_sgemm_colmajor_nt(M, N, K, dev(af), dev(bf), dc, 1.0, -1.5, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert (r["injected"], r["detected"], r["corrected"], r["false_alarms"]) == (0, 0, 0, 0) and r["tiles"] >= 1
    assert np.array_equal(dc.cpu().numpy(), want)
    # C^T is N x M: plant a flip of bit 28 at C^T[(N-1), (M-2)] after slab 1
    gr, gc = N - 1, M - 2
    plan = np.array([[gr // 128, gc // 128, gr % 128, gc % 128, 1, 28]], dtype=np.int32)
    rep = b2.new_report()
    dc = dev(cf)
    b2.ft_sgemm_colmajor_nt(M, N, K, dev(af), dev(bf), dc, 1.0, -1.5, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert (r["injected"], r["detected"], r["corrected"]) == (1, 1, 1), r
    assert np.array_equal(dc.cpu().numpy(), want)


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("sa,sb", [(100.0, 1.0), (0.01, 0.5), (7.0, 300.0)])
def test_scale_aware_threshold(cuda, path, sa, sb):
    """Operands far from unit scale: tau < 0 measures 3*rms(A)*rms(B) and scales the default threshold with it, so a
    clean run raises no alarm and a planted flip is still found; the unit-scale default (tau = 0) would flag clean
    blocks when the data is large."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 256, 512, 768
    a, b, c = mats(M, N, K)
    a, b = (a * np.float32(sa)).astype(np.float32), (b * np.float32(sb)).astype(np.float32)
    da, db = dev(a), dev(b)
    plain = torch.zeros((M, N), device="cuda")
    b2.sgemm(M, N, K, 1.0, da, db, 0.0, plain, path=path)
    rep = b2.new_report()
    out = torch.zeros((M, N), device="cuda")
    b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=path, tau=-1.0, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["detected"] == 0 and r["false_alarms"] == 0 and r["corrected"] == 0
    assert torch.equal(out, plain)
    # a flip of the top exponent bit of the largest accumulator is far above any scaled threshold
    acc = plain.cpu().numpy()
    r0, c0 = (int(v) for v in np.unravel_index(np.argmax(np.abs(acc)), acc.shape))
    plan = np.array([[r0 // 128, c0 // 128, r0 % 128, c0 % 128, 10 ** 6, 29]], dtype=np.int32)
    rep = b2.new_report()
    out.zero_()
    b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=path, tau=-1.0, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["injected"] == 1 and r["detected"] == 1 and r["corrected"] >= 1 and r["false_alarms"] == 0
    scale = 3.0 * float(np.sqrt(np.mean(a.astype(np.float64) ** 2)) * np.sqrt(np.mean(b.astype(np.float64) ** 2)))
    assert float((out - plain).abs().max().item()) <= 2.6e-5 * K * scale
    if sa * sb >= 100.0:
        # the unit-scale default is too tight for this data: clean blocks are flagged (and found clean)
        rep = b2.new_report()
        out.zero_()
        b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=path, tau=0.0, report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert r["false_alarms"] + r["detected"] > 0
        if path == 0:
            assert r["corrected"] == 0 and torch.equal(out, plain)      # recomputation is bit-exact on the FFMA path


@pytest.mark.parametrize("transpose_a", [0, 1])
def test_thread_level_encoder(cuda, transpose_a):
    """The thread-level encoder (every thread checks its own 4 x 16 outputs, the reference's ft_sgemm_huge_thread idea)
    finds and repairs the same faults as the block-level one, bit-identically, with no false alarm."""
    import hpcdeepneuralnetworks_b200 as b2
    n = 1024
    M, N, K = 512, 2048, 1024           # N >= 2048: the K-major route is eligible when transpose_a = 1
    a, b, c = mats(M, N, K)
    want = oracle.sgemm_fma(1.0, a, b, 0.5, c)
    plan = oracle.make_fault_plan(M, N, K, seed=9, tiles_per_fault=4, bit_lo=25, bit_hi=30)
    tau = default_tau(K)
    must, gray, benign = classify(a, b, plan, tau)
    try:
        b2.set_ft_level(2)
        b2.set_ffma_transpose_a(transpose_a)
        rep = b2.new_report()
        dc = dev(c)
        b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert (r["tiles"], r["injected"], r["detected"], r["corrected"], r["false_alarms"]) == (64, 0, 0, 0, 0)
        assert np.array_equal(dc.cpu().numpy(), want)
        rep = b2.new_report()
        dc = dev(c)
        b2.ft_sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dc, plan=b2.make_plan(plan), report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert r["injected"] == len(plan) and r["false_alarms"] == 0
        assert must <= r["corrected"] <= must + gray
        if gray == 0 and benign == 0:
            assert np.array_equal(dc.cpu().numpy(), want)
    finally:
        b2.set_ft_level(1)
        b2.set_ffma_transpose_a(1)

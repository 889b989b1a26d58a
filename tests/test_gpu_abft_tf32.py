"""GPU tests of the ABFT SGEMM on the 3xTF32 tensor-core path: a clean run is bit-identical to the plain
3xTF32 kernel with no detection and no false alarm; a flipped accumulator bit whose effect is above the
threshold is found and the output rebuilt so that the result meets the 3xTF32 tolerance; a flip below the
threshold is left alone.  The accumulators live in tensor memory, so what a fault does to one of them is
known from the plain kernel's own output (alpha = 1, beta = 0)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = 2e-5          # max|C - C_ref| / (|A| |B|) that the 3xTF32 path has to meet


TAU_PER_K = 2.5e-6       # default threshold per unit of K: half the accuracy bound of uniform [-1, 1) operands (5e-6 * K)
TAU_FLOOR = 6e-5
ELEM = 0.75              # an output further than this fraction of tau from its recomputed value is replaced


@pytest.fixture(autouse=True, params=[(2, 1), (2, 0), (0, 0)],
                ids=["cta_pair_persistent", "cta_pair_one_tile_per_cluster", "single_cta"])
def _kernel_form(request, cuda):
    """Every test runs on the persistent CTA-pair kernel (the default for large problems: 256 x 256 tiles), on the
    one-tile-per-cluster CTA-pair kernel and on the single-CTA kernel (128 x 256 tiles).  The ABFT kernels accumulate
    over all of K in one go, so the plain products they are compared with here are made the same way (no chunks, no
    cut of the last round)."""
    import hpcdeepneuralnetworks_b200 as b2
    pair, persistent = request.param
    b2.set_tf32_pair(pair)
    b2.set_tf32_persistent(persistent)
    b2.set_tf32_chunk(0)
    b2.set_tf32_tail_split(0)      # one accumulation per tile, as in the plain products compared with (the cut has its own test)
    yield
    b2.set_tf32_pair(1)
    b2.set_tf32_persistent(1)
    b2.set_tf32_chunk(-1)
    b2.set_tf32_tail_split(1)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mats(M, N, K):
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    return a, b, c


def default_tau(K):
    return max(TAU_PER_K * K, TAU_FLOOR)


def elem_tol(K):
    """How far a repaired output (an FP32 recomputation) may sit from the tensor-core value it replaces."""
    return ELEM * default_tau(K)


def flip(x, bit):
    """float32 array/scalar with one bit flipped."""
    return (np.asarray(x, dtype=np.float32).view(np.uint32) ^ np.uint32(1 << bit)).view(np.float32)


def classify(acc, plan, tau):
    """(must, gray, benign) index lists of a plan, from the size of each flip on the accumulator `acc`."""
    must, gray, benign = [], [], []
    for i, f in enumerate(plan):
        r, c = f[0] * 128 + f[2], f[1] * 128 + f[3]
        with np.errstate(all="ignore"):
            d = abs(np.float64(flip(acc[r, c], int(f[5]))) - np.float64(acc[r, c]))
        (must if (not np.isfinite(d) or d > 2 * tau) else benign if d < 0.5 * tau else gray).append(i)
    return must, gray, benign


def counts(r):
    return {k: r[k] for k in ("tiles", "injected", "detected", "corrected", "uncorrectable", "false_alarms")}


@pytest.mark.parametrize("shape", [(128, 256, 32), (256, 384, 96), (1024, 1024, 1024), (130, 260, 72), (64, 512, 1000),
                                   (300, 100, 40), (129, 257, 33)])
def test_clean_run_bit_identical_to_plain_3xtf32(cuda, shape):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    da, db = dev(a), dev(b)
    plain, out = dev(c), dev(c)
    b2.set_tf32_tile_n(256)
    try:
        b2.sgemm(M, N, K, 1.25, da, db, 0.5, plain, path=b2.PATH_3XTF32)
    finally:
        b2.set_tf32_tile_n(0)
    rep = b2.new_report()
    b2.ft_sgemm(M, N, K, 1.25, da, db, 0.5, out, path=b2.PATH_3XTF32, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    assert counts(r) == {"tiles": tiles, "injected": 0, "detected": 0, "corrected": 0, "uncorrectable": 0, "false_alarms": 0}
    assert 0.0 <= r["max_residual"] <= 0.5 * default_tau(K)
    assert torch.equal(out, plain)
    c64, den = oracle.sgemm_f64(1.25, a, b, 0.5, c)
    assert oracle.gemm_error(out.cpu().numpy(), c64, den) <= TOL


@pytest.mark.parametrize("bit", [12, 18, 21, 23, 25, 27, 29, 30, 31])
def test_single_fault_each_bit(cuda, bit):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 256, 512, 512
    a, b, _ = mats(M, N, K)
    da, db = dev(a), dev(b)
    acc = torch.zeros((M, N), device="cuda")
    b2.sgemm(M, N, K, 1.0, da, db, 0.0, acc, path=b2.PATH_3XTF32)
    acc = acc.cpu().numpy()
    plan = np.array([[1, 2, 77, 101, 0, bit]], dtype=np.int32)      # element (205, 357)
    tau = default_tau(K)
    must, gray, benign = classify(acc, plan, tau)
    rep = b2.new_report()
    out = torch.zeros((M, N), device="cuda")
    b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    got = out.cpu().numpy()
    assert r["tiles"] == 4 and r["injected"] == 1 and r["false_alarms"] == 0
    mask = np.ones_like(acc, dtype=bool)
    mask[205, 357] = False
    assert np.array_equal(got[mask], acc[mask])                      # nothing else moved
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.0, np.zeros_like(acc))
    if must:
        assert r["detected"] == 1 and r["corrected"] == 1
        assert abs(float(got[205, 357]) - float(acc[205, 357])) <= elem_tol(K)
        assert oracle.gemm_error(got, c64, den) <= TOL
    if benign:
        assert r["detected"] == 0 and r["corrected"] == 0
        assert got[205, 357].view(np.uint32) == flip(acc[205, 357], bit).view(np.uint32)


@pytest.mark.parametrize("seed", [6, 7, 8])
def test_config3_1024_plan(cuda, seed):
    """Benchmark configuration 3 at 1024^3 on the tensor-core path: one flip (bit 20..30) per 64 tiles of 128 x 128, and a
    denser plan of one per 2 tiles."""
    import hpcdeepneuralnetworks_b200 as b2
    n = 1024
    a, b, _ = mats(n, n, n)
    da, db = dev(a), dev(b)
    acc_d = torch.zeros((n, n), device="cuda")
    b2.sgemm(n, n, n, 1.0, da, db, 0.0, acc_d, path=b2.PATH_3XTF32)
    acc = acc_d.cpu().numpy()
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.0, np.zeros_like(acc))
    tau = default_tau(n)
    for per in (64, 2):
        plan = oracle.make_fault_plan(n, n, n, seed=seed, tiles_per_fault=per)
        must, gray, benign = classify(acc, plan, tau)
        rep = b2.new_report()
        out = torch.zeros((n, n), device="cuda")
        b2.ft_sgemm(n, n, n, 1.0, da, db, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert r["tiles"] == 32 and r["injected"] == len(plan) and r["false_alarms"] == 0
        assert len(must) <= r["corrected"] <= len(must) + len(gray)
        got = out.cpu().numpy()
        changed = np.argwhere(got.view(np.uint32) != acc.view(np.uint32))
        struck = {(int(f[0]) * 128 + int(f[2]), int(f[1]) * 128 + int(f[3])) for f in plan}
        assert {tuple(int(v) for v in rc) for rc in changed} <= struck
        for i in must:
            f = plan[i]
            rr, cc = f[0] * 128 + f[2], f[1] * 128 + f[3]
            assert abs(float(got[rr, cc]) - float(acc[rr, cc])) <= elem_tol(n)
        if not gray:
            # benign flips stay in the output: each is below tau / 2 by construction
            assert np.abs(got.astype(np.float64) - acc.astype(np.float64)).max() <= elem_tol(n)
        if not gray and not benign:
            assert oracle.gemm_error(got, c64, den) <= TOL


def test_nan_and_inf_faults_are_rebuilt(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 128, 256, 256
    a, b, _ = mats(M, N, K)
    da, db = dev(a), dev(b)
    acc_d = torch.zeros((M, N), device="cuda")
    b2.sgemm(M, N, K, 1.0, da, db, 0.0, acc_d, path=b2.PATH_3XTF32)
    acc = acc_d.cpu().numpy()
    cand = np.argwhere((np.abs(acc) >= 1.0) & (np.abs(acc) < 2.0))
    r0, c0 = (int(v) for v in cand[0])
    with np.errstate(all="ignore"):
        assert not np.isfinite(flip(acc[r0, c0], 30))
    plan = np.array([[0, c0 // 128, r0, c0 % 128, 0, 30]], dtype=np.int32)
    rep = b2.new_report()
    out = torch.zeros((M, N), device="cuda")
    b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
    r = b2.read_report(rep)
    assert r["injected"] == 1 and r["detected"] == 1 and r["corrected"] == 1
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.0, np.zeros_like(acc))
    assert oracle.gemm_error(got, c64, den) <= TOL


def test_faults_in_both_halves_of_a_tile_and_in_one_group(cuda):
    """Two planned tiles of 128 columns share one 256-column kernel tile; two struck rows share one group of 32
    columns.  All four flips are applied and repaired."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 128, 256, 384
    a, b, _ = mats(M, N, K)
    da, db = dev(a), dev(b)
    acc = torch.zeros((M, N), device="cuda")
    b2.sgemm(M, N, K, 1.0, da, db, 0.0, acc, path=b2.PATH_3XTF32)
    plan = np.array([[0, 0, 5, 40, 0, 29], [0, 1, 5, 9, 0, 28], [0, 0, 17, 33, 0, 29], [0, 1, 90, 127, 0, 27]], dtype=np.int32)
    rep = b2.new_report()
    out = torch.zeros((M, N), device="cuda")
    b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert counts(r) == {"tiles": 1, "injected": 4, "detected": 4, "corrected": 4, "uncorrectable": 0, "false_alarms": 0}
    assert float((out - acc).abs().max().item()) <= elem_tol(K)


def test_threshold_override_leaves_small_faults_alone(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 128, 256, 128
    a, b, _ = mats(M, N, K)
    da, db = dev(a), dev(b)
    acc_d = torch.zeros((M, N), device="cuda")
    b2.sgemm(M, N, K, 1.0, da, db, 0.0, acc_d, path=b2.PATH_3XTF32)
    acc = acc_d.cpu().numpy()
    r0, c0 = (int(v) for v in np.unravel_index(np.argmax(np.abs(acc)), acc.shape))
    bad = flip(acc[r0, c0], 22)                                     # top mantissa bit: a quarter of the value or more
    assert abs(float(bad) - float(acc[r0, c0])) > 2 * default_tau(K)
    plan = np.array([[0, c0 // 128, r0, c0 % 128, 0, 22]], dtype=np.int32)
    for tau, found in ((1e9, 0), (0.0, 1)):
        rep = b2.new_report()
        out = torch.zeros((M, N), device="cuda")
        b2.ft_sgemm(M, N, K, 1.0, da, db, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), tau=tau, report=rep)
        r = b2.read_report(rep)
        assert r["injected"] == 1 and r["detected"] == found and r["corrected"] == found and r["false_alarms"] == 0
        got = out.cpu().numpy()
        if found:
            assert abs(float(got[r0, c0]) - float(acc[r0, c0])) <= elem_tol(K)
        else:
            assert got[r0, c0].view(np.uint32) == bad.view(np.uint32)


def test_degenerate_products_take_the_scaling_route(cuda):
    """K = 0 or alpha = 0: C <- beta*C without touching the tensor cores, still through b2_ft_sgemm."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N = 96, 160
    _, _, c = mats(M, N, 8)
    a, b, _ = mats(M, N, 64)
    out = dev(c)
    b2.ft_sgemm(M, N, 0, 1.0, dev(a), dev(b), 0.5, out, path=b2.PATH_3XTF32, lda=64, ldb=N)
    assert np.array_equal(out.cpu().numpy(), (np.float32(0.5) * c).astype(np.float32))
    out = dev(c)
    b2.ft_sgemm(M, N, 64, 0.0, dev(a), dev(b), -2.0, out, path=b2.PATH_3XTF32)
    assert np.array_equal(out.cpu().numpy(), (np.float32(-2.0) * c).astype(np.float32))


@pytest.mark.parametrize("n", [4096, 8192])
def test_config3_large_sizes(cuda, n):
    """Benchmark configuration 3 at 4096^3 and 8192^3: a clean run and the seeded plan (one flip per 64 tiles), checked
    against the plain 3xTF32 kernel on the device."""
    import hpcdeepneuralnetworks_b200 as b2
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    plain = torch.zeros((n, n), device="cuda")
    b2.set_tf32_tile_n(256)
    try:
        b2.sgemm(n, n, n, 1.0, A, B, 0.0, plain, path=b2.PATH_3XTF32)
    finally:
        b2.set_tf32_tile_n(0)
    tau = default_tau(n)
    rep = b2.new_report()
    out = torch.zeros((n, n), device="cuda")
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert counts(r) == {"tiles": (n // 128) * (n // 256), "injected": 0, "detected": 0, "corrected": 0, "uncorrectable": 0,
                         "false_alarms": 0}
    assert r["max_residual"] <= 0.4 * tau                         # margin of the default threshold on clean data
    assert torch.equal(out, plain)
    plan = oracle.make_fault_plan(n, n, n, seed=6)
    acc = plain.cpu().numpy()
    must, gray, benign = classify(acc, plan, tau)
    rep = b2.new_report()
    out.zero_()
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["injected"] == len(plan) and r["false_alarms"] == 0
    assert len(must) <= r["corrected"] <= len(must) + len(gray)
    diff = (out - plain).abs()
    assert int((diff > 0).sum().item()) <= len(plan)
    # repaired outputs carry the FP32 recomputation (within tau/2 of the tensor-core value); flips that stay are below 2 tau
    assert float(diff.max().item()) <= (2 * tau if gray else elem_tol(n))


@pytest.mark.parametrize("n", [2304, 4096])
def test_abft_with_the_last_round_cut_along_k(cuda, n):
    """The persistent ABFT kernel cuts a partial last round of tiles along K like the plain kernel (2304: 81 tiles, the last
    7 in five runs each; 4096: 256 tiles, the last 34 in two): every run is verified and repaired against the checksums
    of its own k range, then the runs are added.  Clean: every tile counted once, no alarm, the result as close to the uncut
    one as the path's own error at this K.  Seeded flips (one per 64 tiles, bits 20..30, striking a tile's first run): all
    injected, no false alarm, and the repaired result meets the path's accuracy contract everywhere."""
    import hpcdeepneuralnetworks_b200 as b2
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    uncut = torch.zeros((n, n), device="cuda")
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, uncut, path=b2.PATH_3XTF32)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        den = A.abs() @ B.abs()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    try:
        b2.set_tf32_tail_split(1)
        rep = b2.new_report()
        out = torch.zeros((n, n), device="cuda")
        b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert counts(r) == {"tiles": ((n + 127) // 128) * ((n + 255) // 256), "injected": 0, "detected": 0, "corrected": 0,
                             "uncorrectable": 0, "false_alarms": 0}
        assert bool(((out - uncut).abs() <= 3e-6 * den).all().item())      # runs lose less to the tensor cores' truncation than one long accumulation
        plan = oracle.make_fault_plan(n, n, n, seed=6)
        rep = b2.new_report()
        hit = torch.zeros((n, n), device="cuda")
        b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, hit, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
        b2.check_status()
        r = b2.read_report(rep)
        assert r["injected"] == len(plan) and r["false_alarms"] == 0 and r["uncorrectable"] == 0, r
        assert bool(((hit - uncut).abs() <= TOL * den).all().item())
    finally:
        b2.set_tf32_tail_split(0)


def _smallest_flip_beyond(v, tol):
    """Lowest bit (0..30) of float32 v whose flip moves v by more than tol, and the size of that move."""
    for bit in range(0, 31):
        with np.errstate(all="ignore"):
            d = abs(np.float64(flip(v, bit)) - np.float64(v))
        if not np.isfinite(d) or d > tol:
            return bit, d
    return 30, np.inf


@pytest.mark.parametrize("n", [1024, 4096, 8192])
def test_every_flip_beyond_the_path_tolerance_is_repaired(cuda, n):
    """The accuracy contract of the path is max|C - C_ref| <= 2e-5 * sum_k |a_ik||b_kj| per element.  One element in
    every fourth 128 x 128 tile gets the SMALLEST single-bit flip that breaks that bound for it (the flip moves it by
    one to two times the bound): every one of them has to be found and rebuilt, and nothing else may move."""
    import hpcdeepneuralnetworks_b200 as b2
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    plain = torch.zeros((n, n), device="cuda")
    b2.sgemm(n, n, n, 1.0, A, B, 0.0, plain, path=b2.PATH_3XTF32)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        den = A.abs() @ B.abs()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    rng = np.random.default_rng(n)
    tiles = n // 128
    plan, moves = [], []
    for t in range(0, tiles * tiles, 4):
        tm, tn = divmod(t, tiles)
        r, c = int(rng.integers(0, 128)), int(rng.integers(0, 128))
        v = np.float32(plain[tm * 128 + r, tn * 128 + c].item())
        bound = TOL * float(den[tm * 128 + r, tn * 128 + c].item())
        bit, d = _smallest_flip_beyond(v, bound)
        plan.append([tm, tn, r, c, 0, bit])
        moves.append(d / bound)
    plan = np.array(plan, dtype=np.int32)
    assert 1.0 < min(moves) and np.median(moves) <= 2.0
    rep = b2.new_report()
    out = torch.zeros((n, n), device="cuda")
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["injected"] == len(plan) and r["detected"] == len(plan) and r["corrected"] == len(plan), r
    assert r["false_alarms"] == 0
    diff = (out - plain).abs()
    assert int((diff > 0).sum().item()) <= len(plan)
    assert float(diff.max().item()) <= elem_tol(n)
    # the repaired result meets the contract everywhere
    assert bool(((out - plain).abs() <= TOL * den).all().item())


@pytest.mark.parametrize("n,scale", [(1024, 0.01), (1024, 300.0), (4096, 0.01), (4096, 300.0), (8192, 1.0)])
def test_clean_runs_raise_no_alarm_at_any_data_scale(cuda, n, scale):
    """tau < 0 scales the default threshold by 3 * rms(A) * rms(B): no false alarm, no repair, bit-identical output."""
    import hpcdeepneuralnetworks_b200 as b2
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 11) * scale
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 12)
    plain = torch.zeros((n, n), device="cuda")
    b2.set_tf32_tile_n(256)
    try:
        b2.sgemm(n, n, n, 1.0, A, B, 0.0, plain, path=b2.PATH_3XTF32)
    finally:
        b2.set_tf32_tile_n(0)
    rep = b2.new_report()
    out = torch.zeros((n, n), device="cuda")
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, tau=-1.0, report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    assert r["detected"] == 0 and r["corrected"] == 0 and r["false_alarms"] == 0, r
    assert r["max_residual"] <= 0.5 * default_tau(n) * scale
    assert torch.equal(out, plain)


@pytest.mark.parametrize("K", [1024, 8192])
def test_truncation_model_shrinks_the_clean_residual(cuda, K):
    """The check expects a group's sum to fall short of its checksum by the built-in fraction of the group's running sum
    (the tensor cores' truncating accumulation).  On clean data, with the threshold out of the way, the largest residual
    with that model is several times smaller than with a plain checksum (coefficient 0), and below a fifth of the
    default threshold."""
    import hpcdeepneuralnetworks_b200 as b2
    M = N = 2048
    A = b2.fill_uniform(torch.empty((M, K), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((K, N), device="cuda"), 2)
    worst = {}
    try:
        for bias in (0.0, -1.0):           # 0: plain checksum; negative: the built-in coefficient
            b2.set_tf32_abft_bias(bias)
            rep = b2.new_report()
            out = torch.zeros((M, N), device="cuda")
            b2.ft_sgemm(M, N, K, 1.0, A, B, 0.0, out, path=b2.PATH_3XTF32, tau=1e30, report=rep)
            b2.check_status()
            worst[bias] = b2.read_report(rep)["max_residual"]
    finally:
        b2.set_tf32_abft_bias(-1.0)
    assert worst[-1.0] <= 0.2 * default_tau(K)
    assert worst[0.0] >= 4.0 * worst[-1.0], worst

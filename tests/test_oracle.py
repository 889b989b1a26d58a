"""CPU tests of the oracle: pinned against the reference's compiled cpu_gemm (when oracle/_ref is
built) and against the committed golden fixtures; internal consistency of the restated loops."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def inputs(n, beta):
    a = oracle.fill_uniform(n * n, 1).reshape(n, n)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    c = np.zeros((n, n), np.float32) if beta == 0.0 else oracle.fill_uniform(n * n, 3).reshape(n, n)
    return a, b, c


def test_rng_matches_golden_and_c():
    for seed, vals in GOLD["rng"].items():
        assert [float(x) for x in oracle.fill_uniform(8, int(seed))] == vals
    v = oracle.fill_uniform(1 << 20, 1)
    assert digest(v) == GOLD["rng_sha_seed1_1M"]
    assert np.array_equal(v[:4096], oracle.fill_uniform_c(4096, 1))
    assert v.min() >= -1.0 and v.max() < 1.0
    # offset form is the same stream
    assert np.array_equal(oracle.fill_uniform(100, 7, offset=50), oracle.fill_uniform(150, 7)[50:])
    assert abs(float(v.mean())) < 5e-3 and abs(float(v.var()) - 1.0 / 3.0) < 5e-3


@pytest.mark.parametrize("entry", GOLD["cpu_gemm"], ids=lambda e: f"n{e['n']}_a{e['alpha']}_b{e['beta']}")
def test_cpu_gemm_matches_reference_golden(entry):
    a, b, c = inputs(entry["n"], entry["beta"])
    got = oracle.cpu_gemm(entry["alpha"], entry["beta"], a, b, c)
    assert digest(got) == entry["sha256"]
    assert [float(x) for x in got[0, :8]] == entry["first_row"]
    if "full" in entry:
        assert [float(x) for x in got.ravel()] == entry["full"]


@pytest.mark.skipif(oracle.ref_lib() is None, reason="oracle/_ref not built (no reference tree)")
@pytest.mark.parametrize("n,alpha,beta", [(16, 1.0, 0.0), (96, 0.5, -1.5), (256, 1.0, 0.5)])
def test_cpu_gemm_bit_equal_to_compiled_reference(n, alpha, beta):
    a, b, c = inputs(n, beta)
    assert np.array_equal(oracle.cpu_gemm(alpha, beta, a, b, c), oracle.ref_cpu_gemm(alpha, beta, a, b, c))


def test_general_f32_gemm_equals_cpu_gemm_on_squares():
    a, b, c = inputs(128, 0.5)
    assert np.array_equal(oracle.sgemm_f32(1.0, a, b, 0.5, c), oracle.cpu_gemm(1.0, 0.5, a, b, c))
    assert np.array_equal(oracle.sgemm_f32(1.0, a, b, 0.5, c, nthreads=1), oracle.sgemm_f32(1.0, a, b, 0.5, c, nthreads=3))


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 2, 2), (17, 13, 5), (33, 65, 129), (128, 256, 64)])
def test_fma_and_f32_gemm_within_north_star_tolerance(shape):
    M, N, K = shape
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    assert np.allclose(c64, a.astype(np.float64) @ b.astype(np.float64) + 0.5 * c.astype(np.float64), rtol=1e-12, atol=1e-12)
    assert oracle.gemm_error(oracle.sgemm_fma(1.0, a, b, 0.5, c), c64, den) <= 1e-5
    assert oracle.gemm_error(oracle.sgemm_f32(1.0, a, b, 0.5, c), c64, den) <= 1e-5


def test_known_answers():
    n = 8
    eye = np.eye(n, dtype=np.float32)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    z = np.zeros((n, n), np.float32)
    assert np.array_equal(oracle.sgemm_fma(1.0, eye, b, 0.0, z), b)
    ones = np.ones((n, n), np.float32)
    assert np.array_equal(oracle.sgemm_fma(1.0, ones, ones, 0.0, z), np.full((n, n), float(n), np.float32))
    onehot = np.zeros((n, n), np.float32)
    onehot[2, 5] = 3.0
    assert np.array_equal(oracle.sgemm_fma(1.0, onehot, b, 0.0, z)[2], 3.0 * b[5])
    # beta == 0 must not read C (NaN stays out)
    nan = np.full((n, n), np.nan, np.float32)
    assert np.isfinite(oracle.sgemm_fma(1.0, eye, b, 0.0, nan)).all()


def test_colmajor_nt_matches_row_major():
    M, N, K = 24, 40, 16
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)   # logical A
    b = oracle.fill_uniform(N * K, 2).reshape(N, K)   # logical B (N x K); C = A B^T
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    got = oracle.sgemm_colmajor_nt(M, N, K, 1.0, np.asfortranarray(a).ravel(order="F"), np.asfortranarray(b).ravel(order="F"),
                                   -1.5, np.asfortranarray(c).ravel(order="F"))
    want = oracle.sgemm_fma(1.0, a, np.ascontiguousarray(b.T), -1.5, c)
    assert np.array_equal(got.reshape(N, M).T, want)


@pytest.mark.parametrize("entry", GOLD["saxpy"], ids=lambda e: f"n{e['n']}")
def test_saxpy_golden(entry):
    n = entry["n"]
    x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
    got = oracle.saxpy(entry["alpha"], x, y)
    assert digest(got) == entry["sha256"]
    # alpha = 2 makes the product exact, so fused and unfused agree bit for bit
    assert np.array_equal(got, np.float32(2.0) * x + y)


@pytest.mark.parametrize("entry", GOLD["sdot"], ids=lambda e: f"n{e['n']}")
def test_sdot_golden(entry):
    n = entry["n"]
    x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
    s, sa = oracle.sdot(x, y, nthreads=1)
    assert s == entry["dot"] and sa == entry["abs"]
    s8, _ = oracle.sdot(x, y, nthreads=8)
    assert abs(s8 - s) <= 1e-12 * max(1.0, sa)


def test_sdot_empty():
    z = np.zeros(0, np.float32)
    assert oracle.sdot(z, z) == (0.0, 0.0)


def test_abft_checksum_algebra():
    """e^T(A_t B_t) and (A_t B_t)e equal the encoded (e^T A_t)B_t and A_t(B_t e)  (kernel/ft_sgemm/README.md:4-14)."""
    M, N, K = 256, 384, 96
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = a.astype(np.float64) @ b.astype(np.float64)
    for tm, tn in ((0, 0), (1, 2)):
        r, col = oracle.abft_tile_checksums(a, b, tm, tn)
        t = c[tm * 128:(tm + 1) * 128, tn * 128:(tn + 1) * 128]
        assert np.allclose(r, t.sum(axis=1), rtol=0, atol=1e-9)
        assert np.allclose(col, t.sum(axis=0), rtol=0, atol=1e-9)


def test_abft_partial_tile_checksums():
    M, N, K = 130, 200, 40
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = a.astype(np.float64) @ b.astype(np.float64)
    r, col = oracle.abft_tile_checksums(a, b, 1, 1)
    assert np.allclose(r[:2], c[128:, 128:].sum(axis=1), atol=1e-9) and np.all(r[2:] == 0)
    assert np.allclose(col[:72], c[128:, 128:].sum(axis=0), atol=1e-9) and np.all(col[72:] == 0)


def test_fault_effect_golden_and_semantics():
    n = 256
    a = oracle.fill_uniform(n * n, 1).reshape(n, n)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    clean_c = oracle.sgemm_fma(1.0, a, b, 0.0, np.zeros((n, n), np.float32))
    for e in GOLD["fault"]:
        clean, bad, ok = oracle.fault_effect(a, b, e["fault"])
        assert ok == e["in_range"] and clean == e["clean"] and repr(bad) == e["faulty"]
        tm, tn, r, c = e["fault"][:4]
        assert clean == clean_c[tm * 128 + r, tn * 128 + c]
    # flipping after the last slab is a pure bit flip of the final value
    clean, bad, _ = oracle.fault_effect(a, b, (0, 0, 1, 1, 10 ** 6, 22))
    assert np.float32(bad).view(np.uint32) ^ np.float32(clean).view(np.uint32) == 1 << 22
    assert oracle.fault_effect(a, b, (5, 0, 0, 0, 0, 20))[2] is False


def test_fault_plan_generation():
    plan = oracle.make_fault_plan(1024, 1024, 1024, seed=6)
    assert plan.shape == (1, 6)
    plan = oracle.make_fault_plan(4096, 4096, 4096, seed=6)
    assert plan.shape == (16, 6)
    tiles = set((int(p[0]), int(p[1])) for p in plan)
    assert len(tiles) == 16                                    # at most one fault per tile
    assert ((plan[:, 5] >= 20) & (plan[:, 5] <= 30)).all()
    assert ((plan[:, 2] >= 0) & (plan[:, 2] < 128) & (plan[:, 3] >= 0) & (plan[:, 3] < 128)).all()
    assert (plan[:, 4] < 4096 // 32).all()
    assert np.array_equal(plan, oracle.make_fault_plan(4096, 4096, 4096, seed=6))
    edge = oracle.make_fault_plan(130, 129, 64, seed=3, tiles_per_fault=1)
    for tm, tn, r, c, ks, bit in edge:
        assert tm * 128 + r < 130 and tn * 128 + c < 129


def test_reference_verify_semantics():
    a = np.ones((4, 4), np.float32)
    b = a.copy()
    b[3, 3] += 0.009
    assert oracle.verify_matrix(a, b)
    b[3, 3] += 0.002
    assert not oracle.verify_matrix(a, b)

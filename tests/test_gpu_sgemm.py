"""GPU parity of the SGEMM kernels against the CPU oracle, through the C ABI.

FFMA path and every rung of the series: bit-exact against the fused oracle (one fmaf per k in
ascending k) and within the north-star tolerance max|C-C_ref|/(|A|.|B|) <= 1e-5 of the double
reference.  3xTF32 path: <= 2e-5."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL_FFMA = 1e-5     # north-star tolerance of the FP32 path
TOL_3XTF32 = 2e-5   # and of the split-precision path


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mats(M, N, K, beta=0.5):
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = np.zeros((M, N), np.float32) if beta == 0.0 else oracle.fill_uniform(M * N, 3).reshape(M, N)
    return a, b, c


def run_gpu(path, a, b, c, alpha, beta):
    import hpcdeepneuralnetworks_b200 as b2
    M, K = a.shape
    N = b.shape[1]
    dc = dev(c)
    b2.sgemm(M, N, K, alpha, dev(a), dev(b), beta, dc, path=path)
    b2.check_status()
    return dc.cpu().numpy()


def test_config1_256_against_reference_cpu_gemm(cuda):
    """Benchmark configuration 1: 256^3, alpha=1, beta=0, C zero-initialised, checked against the reference's
    CPU row-major GEMM arithmetic (utils/utils.cu:93-103) with the reference's own verify_matrix rule
    and with the north-star metric."""
    a, b, c = mats(256, 256, 256, beta=0.0)
    got = run_gpu(0, a, b, c, 1.0, 0.0)
    ref = oracle.cpu_gemm(1.0, 0.0, a, b, c)
    assert oracle.verify_matrix(ref, got)                       # |ref-got| <= 1e-2 everywhere
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.0, c)
    assert oracle.gemm_error(got, c64, den) <= TOL_FFMA
    assert np.array_equal(got, oracle.sgemm_fma(1.0, a, b, 0.0, c))


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("shape", [(128, 128, 32), (256, 384, 96), (512, 512, 512)])
def test_ffma_variants_bit_exact(cuda, variant, shape):
    import hpcdeepneuralnetworks_b200 as b2
    b2.set_ffma_variant(variant)
    try:
        a, b, c = mats(*shape)
        got = run_gpu(0, a, b, c, 1.0, 0.5)
        assert np.array_equal(got, oracle.sgemm_fma(1.0, a, b, 0.5, c))
    finally:
        b2.set_ffma_variant(1)


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 3, 4), (17, 13, 5), (127, 129, 31), (130, 260, 33), (64, 512, 1000),
                                   (300, 100, 700), (1, 1024, 64), (1024, 4, 64), (129, 132, 4)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (1.0, 0.5), (-1.5, 1.0), (0.5, -1.5)])
def test_ffma_odd_shapes(cuda, shape, alpha, beta):
    M, N, K = shape
    a, b, c = mats(M, N, K, beta=1.0)
    got = run_gpu(0, a, b, c, alpha, beta)
    assert np.array_equal(got, oracle.sgemm_fma(alpha, a, b, beta, c))
    c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
    assert oracle.gemm_error(got, c64, den) <= TOL_FFMA


def test_ffma_beta_zero_does_not_read_c(cuda):
    a, b, _ = mats(200, 136, 64)
    c = np.full((200, 136), np.nan, np.float32)
    got = run_gpu(0, a, b, c, 1.0, 0.0)
    assert np.array_equal(got, oracle.sgemm_fma(1.0, a, b, 0.0, np.zeros_like(c)))


def test_ffma_degenerate_k_and_alpha(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    c = oracle.fill_uniform(64 * 48, 3).reshape(64, 48)
    dc = dev(c)
    b2.sgemm(64, 48, 0, 1.0, None, None, 0.5, dc)           # K = 0: C = beta*C
    assert np.array_equal(dc.cpu().numpy(), np.float32(0.5) * c)
    a, b, _ = mats(64, 48, 32)
    dc = dev(c)
    b2.sgemm(64, 48, 32, 0.0, dev(a), dev(b), 0.0, dc)      # alpha = 0, beta = 0: zeros
    assert not dc.cpu().numpy().any()
    b2.sgemm(0, 48, 32, 1.0, dev(a), dev(b), 0.0, dc)       # empty: no-op


def test_ffma_leading_dimensions_and_guards(cuda):
    """Sub-matrix views (lda/ldb/ldc larger than the logical width); everything outside C's view is untouched."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K, lda, ldb, ldc = 150, 200, 70, 96, 256, 212
    A = oracle.fill_uniform(M * lda, 1).reshape(M, lda)
    B = oracle.fill_uniform(K * ldb, 2).reshape(K, ldb)
    Cb = oracle.fill_uniform((M + 2) * ldc, 3).reshape(M + 2, ldc)
    dC = dev(Cb)
    b2.sgemm(M, N, K, 1.0, dev(A), dev(B), 0.5, dC[1:], lda=lda, ldb=ldb, ldc=ldc)
    want = Cb.copy()
    want[1:M + 1, :N] = oracle.sgemm_fma(1.0, A[:, :K], B[:, :N], 0.5, Cb[1:M + 1, :N])
    assert np.array_equal(dC.cpu().numpy(), want)


def test_ffma_unaligned_falls_back_to_generic_kernel(cuda):
    """Leading dimensions that are not multiples of 4 floats and odd base offsets cannot be described to TMA."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 77, 91, 53
    a, b, c = mats(M, N, K)
    da = dev(np.concatenate([[0.0], a.ravel()]).astype(np.float32))[1:]      # 4-byte aligned only
    dc = dev(c)
    b2.sgemm(M, N, K, 1.0, da, dev(b), 0.5, dc)
    assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))


@pytest.mark.parametrize("kid,n,t", [(1, 96, 32), (1, 100, 16), (2, 128, 32), (2, 64, 16), (3, 128, 32), (4, 128, 32),
                                     (5, 128, 32), (5, 64, 16), (6, 128, 32), (7, 128, 32), (8, 192, 32), (9, 256, 32),
                                     (10, 256, 32), (11, 256, 32), (12, 384, 32), (13, 384, 32), (14, 384, 32)])
def test_series_rungs_bit_exact(cuda, kid, n, t):
    """sgemm_1 .. sgemm_14 with the reference's argument order (N, A, B, C, alpha, beta)."""
    import hpcdeepneuralnetworks_b200 as b2
    a, b, c = mats(n, n, n)
    dc = dev(c)
    b2.sgemm_series(kid, n, dev(a), dev(b), dc, 1.0, 0.5, threads_x=t)
    got = dc.cpu().numpy()
    assert np.array_equal(got, oracle.sgemm_fma(1.0, a, b, 0.5, c))
    assert oracle.verify_matrix(oracle.cpu_gemm(1.0, 0.5, a, b, c), got)


@pytest.mark.parametrize("shape", [(96, 200, 64), (33, 65, 40), (520, 130, 300)])
def test_tile_family_colmajor_and_rowmajor(cuda, shape):
    """Every generated tile on the row-major and on the column-major (transposed-A) entry points."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    af, bf, cf = oracle.fill_uniform(M * K, 1), oracle.fill_uniform(N * K, 2), oracle.fill_uniform(M * N, 3)
    want_cm = oracle.sgemm_colmajor_nt(M, N, K, 1.0, af, bf, -1.5, cf) if M % 4 == 0 and N % 4 == 0 else None
    try:
        for idx, name, bm, bn, threads in b2.ffma_tiles():
            b2.set_ffma_tile(idx)
            got = run_gpu(0, a, b, c, 1.0, 0.5)
            assert np.array_equal(got, oracle.sgemm_fma(1.0, a, b, 0.5, c)), name
            if want_cm is not None:
                dcf = dev(cf)
                b2.sgemm_colmajor_nt(M, N, K, dev(af), dev(bf), dcf, 1.0, -1.5)
                assert np.array_equal(dcf.cpu().numpy(), want_cm), name
    finally:
        b2.set_ffma_tile(-1)


def test_series_rejects_non_multiple(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    t = torch.zeros(200 * 200, device="cuda")
    with pytest.raises(b2.B2Error) as e:
        b2.sgemm_series(13, 200, t, t, t.clone(), 1.0, 0.0)
    assert e.value.status == -2


def test_reference_shaped_shims(cuda):
    from hpcdeepneuralnetworks_b200 import _lib
    import hpcdeepneuralnetworks_b200 as b2
    L = _lib.load()
    n = 256
    a, b, c = mats(n, n, n)
    da, db, dc = dev(a), dev(b), dev(c)
    torch.cuda.synchronize()
    p = lambda t: C.c_void_p(t.data_ptr())
    assert L.ref_sgemm_rowmajor(n, p(da), p(db), p(dc), 1.0, 0.5) == 0
    torch.cuda.synchronize()
    assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))
    dc = dev(c)
    torch.cuda.synchronize()
    assert L.sgemm(n, n, n, 1.0, p(da), p(db), 0.5, p(dc)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))
    # column-major NT of kernel/ft_sgemm: A MxK (lda=M), B NxK (ldb=N), C MxN (ldc=M), beta = -1.5 as in its driver
    for (M, N, K) in ((128, 128, 64), (200, 72, 96), (132, 260, 40)):
        af = oracle.fill_uniform(M * K, 1)
        bf = oracle.fill_uniform(N * K, 2)
        cf = oracle.fill_uniform(M * N, 3)
        dcf = dev(cf)
        b2.sgemm_colmajor_nt(M, N, K, dev(af), dev(bf), dcf, 1.0, -1.5)
        assert np.array_equal(dcf.cpu().numpy(), oracle.sgemm_colmajor_nt(M, N, K, 1.0, af, bf, -1.5, cf))


@pytest.mark.parametrize("shape", [(128, 256, 32), (128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (130, 300, 70),
                                   (17, 13, 5), (384, 128, 1000), (200, 520, 36)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.5), (-1.5, 0.0)])
def test_3xtf32_path(cuda, shape, alpha, beta):
    M, N, K = shape
    a, b, c = mats(M, N, K)
    got = run_gpu(1, a, b, c, alpha, beta)
    c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
    err = oracle.gemm_error(got, c64, den)
    assert err <= TOL_3XTF32, f"3xTF32 error {err:.3e}"


@pytest.mark.parametrize("slab_k", [32, 16])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_3xtf32_both_tile_widths(cuda, tile_n, slab_k):
    import hpcdeepneuralnetworks_b200 as b2
    b2.set_tf32_tile_n(tile_n)
    b2.set_tf32_slab_k(slab_k)
    try:
        for shape in ((256, 512, 96), (130, 300, 70), (640, 384, 200)):
            a, b, c = mats(*shape)
            got = run_gpu(1, a, b, c, 1.0, 0.5)
            c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
            assert oracle.gemm_error(got, c64, den) <= TOL_3XTF32
    finally:
        b2.set_tf32_tile_n(0)
        b2.set_tf32_slab_k(32)


@pytest.mark.parametrize("shape", [(256, 256, 32), (128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (130, 300, 70),
                                   (17, 13, 5), (384, 128, 1000), (200, 520, 36), (257, 255, 33), (1, 1, 1)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.5), (-1.5, 0.0)])
@pytest.mark.parametrize("persistent", [1, 0])
def test_3xtf32_cta_pair_kernel_matches_single_cta(cuda, shape, alpha, beta, persistent):
    """The cta_group::2 kernel (256 x 256 tiles on two CTAs) accumulates every output in the same order as the
    single-CTA kernel, so the two agree bit for bit; both meet the tolerance against the double reference."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    try:
        b2.set_tf32_pair(2)
        b2.set_tf32_persistent(persistent)     # persistent clusters with a double-buffered accumulator, or one cluster per tile
        pair = run_gpu(1, a, b, c, alpha, beta)
        b2.set_tf32_pair(0)
        single = run_gpu(1, a, b, c, alpha, beta)
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_persistent(1)
    assert np.array_equal(pair, single)
    c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
    assert oracle.gemm_error(pair, c64, den) <= TOL_3XTF32


def test_3xtf32_persistent_many_tiles_per_cluster(cuda):
    """More tiles than resident clusters (13 x 9 = 117 pair tiles on 74 slots, partial tiles on both edges, K not a
    multiple of the slab): every cluster walks two tiles through both accumulator buffers."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 3200, 2200, 330
    A = b2.fill_uniform(torch.empty((M, K), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((K, N), device="cuda"), 2)
    C0 = b2.fill_uniform(torch.empty((M, N), device="cuda"), 3)
    out = {}
    try:
        b2.set_tf32_pair(2)
        for pers in (1, 0):
            b2.set_tf32_persistent(pers)
            Cm = C0.clone()
            b2.sgemm(M, N, K, 1.5, A, B, 0.5, Cm, path=1)
            b2.check_status()
            out[pers] = Cm
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_persistent(1)
    assert torch.equal(out[1], out[0])
    rows = np.array([0, 127, 128, 1599, 3199])
    c64, den = oracle.sgemm_f64(1.5, A.cpu().numpy()[rows], B.cpu().numpy(), 0.5, C0.cpu().numpy()[rows])
    assert oracle.gemm_error(out[1].cpu().numpy()[rows], c64, den) <= TOL_3XTF32


def test_3xtf32_cta_pair_large_and_strided(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    n = 2304
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    C0 = b2.fill_uniform(torch.empty((n, n + 12), device="cuda"), 3)
    out = {}
    try:
        for mode in (2, 0):
            b2.set_tf32_pair(mode)
            Cm = C0.clone()
            b2.sgemm(n - 3, n - 5, n - 8, 0.75, A, B, -0.25, Cm, path=1, lda=n, ldb=n, ldc=n + 12)
            b2.check_status()
            out[mode] = Cm
    finally:
        b2.set_tf32_pair(1)
    assert torch.equal(out[2], out[0])
    assert torch.equal(out[2][:, n - 5:], C0[:, n - 5:]) and torch.equal(out[2][n - 3:], C0[n - 3:])


def test_3xtf32_leading_dimensions(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K, lda, ldb, ldc = 150, 200, 70, 96, 256, 212
    A = oracle.fill_uniform(M * lda, 1).reshape(M, lda)
    B = oracle.fill_uniform(K * ldb, 2).reshape(K, ldb)
    Cb = oracle.fill_uniform((M + 2) * ldc, 3).reshape(M + 2, ldc)
    dC = dev(Cb)
    b2.sgemm(M, N, K, 1.0, dev(A), dev(B), 0.5, dC[1:], path=1, lda=lda, ldb=ldb, ldc=ldc)
    b2.check_status()
    got = dC.cpu().numpy()
    c64, den = oracle.sgemm_f64(1.0, A[:, :K], B[:, :N], 0.5, Cb[1:M + 1, :N])
    assert oracle.gemm_error(np.ascontiguousarray(got[1:M + 1, :N]), c64, den) <= TOL_3XTF32
    mask = np.ones_like(Cb, dtype=bool)
    mask[1:M + 1, :N] = False
    assert np.array_equal(got[mask], Cb[mask])          # nothing outside the view was touched


# ---- the hi/lo split inside the GEMM kernel (very small products) -----------------------------------------
@pytest.mark.parametrize("shape", [(128, 128, 32), (256, 256, 256), (384, 256, 320), (130, 300, 70), (17, 13, 5), (1, 1, 1),
                                   (200, 520, 36), (257, 255, 33), (512, 768, 1000), (640, 640, 4096)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.5), (-1.5, 0.0)])
def test_3xtf32_split_inside_the_kernel_is_identical_to_the_pre_pass(cuda, shape, alpha, beta):
    """The kernel that converts the raw tiles of A and B in shared memory (one launch, no workspace) does the same
    split arithmetic and issues the same MMAs in the same order as the 128 x 128 single-CTA kernel behind the two
    split kernels: bit-identical results on whole and partial tiles, K not a multiple of the slab, padded rows."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    lda, ldb, ldc = (K + 3) // 4 * 4 + 4, (N + 3) // 4 * 4, (N + 3) // 4 * 4 + 8
    A = oracle.fill_uniform(M * lda, 1).reshape(M, lda)
    B = oracle.fill_uniform(K * ldb, 2).reshape(K, ldb)
    Cb = oracle.fill_uniform(M * ldc, 3).reshape(M, ldc)
    out = {}
    try:
        for mode, tile_n in ((0, 128), (2, 0)):
            b2.set_tf32_fused_split(mode)
            b2.set_tf32_tile_n(tile_n)
            dC = dev(Cb)
            b2.sgemm(M, N, K, alpha, dev(A), dev(B), beta, dC, path=1, lda=lda, ldb=ldb, ldc=ldc)
            b2.check_status()
            out[mode] = dC.cpu().numpy()
    finally:
        b2.set_tf32_fused_split(1)
        b2.set_tf32_tile_n(0)
    assert np.array_equal(out[2], out[0])
    assert np.array_equal(out[2][:, N:], Cb[:, N:])
    c64, den = oracle.sgemm_f64(alpha, A[:, :K], B[:, :N], beta, Cb[:, :N])
    assert oracle.gemm_error(np.ascontiguousarray(out[2][:, :N]), c64, den) <= TOL_3XTF32


def test_3xtf32_split_inside_the_kernel_needs_aligned_operands_and_falls_back(cuda):
    """Operands that TMA cannot address (not 16-byte aligned, or a leading dimension that is not a multiple of 4) go
    through the pre-pass as before, whatever the knob says."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 96, 160, 200
    a, b, c = mats(M, N, K)
    big_a = np.zeros((M, K + 1), np.float32)
    big_a[:, 1:] = a
    dA = dev(big_a)
    try:
        b2.set_tf32_fused_split(2)
        dC = dev(c)
        b2.sgemm(M, N, K, 1.0, dA[:, 1:], dev(b), 0.5, dC, path=1, lda=K + 1)     # A starts 4 bytes into its allocation, odd pitch
        b2.check_status()
    finally:
        b2.set_tf32_fused_split(1)
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    assert oracle.gemm_error(dC.cpu().numpy(), c64, den) <= TOL_3XTF32


# ---- chunked accumulation of the 3xTF32 path (K beyond two chunks of 16 K-slabs) --------------------------
@pytest.mark.parametrize("shape", [(300, 1000, 2100), (256, 256, 1056), (1, 5, 1100), (513, 260, 4096), (130, 36, 1500),
                                   (2048, 2048, 2048), (3200, 2200, 1100)])     # the last: 117 pair tiles on 74 clusters
@pytest.mark.parametrize("alpha,beta", [(1.25, 0.5), (-1.5, 0.0)])
@pytest.mark.parametrize("chunk", [16, 3])
def test_3xtf32_chunked_forms_agree_bit_for_bit(cuda, shape, alpha, beta, chunk):
    """Chunked accumulation: the persistent CTA-pair kernel and the single-CTA 128 x 128 kernel cut K at the same
    slabs and add the chunks in the same order, so they agree bit for bit (partial tiles on every edge, K not a
    multiple of the slab, chunks that do not divide the slab count); both meet the tolerance."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    try:
        b2.set_tf32_chunk(chunk)
        b2.set_tf32_tail_split(0)      # every tile on one cluster: one chain of chunk sums per output in both forms
        b2.set_tf32_pair(2)
        pair = run_gpu(1, a, b, c, alpha, beta)
        b2.set_tf32_pair(0)
        single = run_gpu(1, a, b, c, alpha, beta)
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_chunk(-1)
        b2.set_tf32_tail_split(1)
    assert np.array_equal(pair, single)
    c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
    assert oracle.gemm_error(pair, c64, den) <= 0.25 * TOL_3XTF32


@pytest.mark.parametrize("shape", [(1024, 1024, 8192), (2304, 2304, 2304), (256, 300, 4100), (3328, 3300, 2047), (513, 260, 4096),
                                   (4096, 4096, 1200)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.5), (-1.5, 0.0)])
def test_3xtf32_last_round_cut_along_k(cuda, shape, alpha, beta):
    """When the tiles do not fill the last round of clusters, each tile of that round is cut along K into runs of
    whole chunks on different clusters, whose sums go through the workspace and are added in K order.  Same result as
    tile by tile up to the order of a few FP32 additions (identical when every run is one chunk), and the same twice."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    out = {}
    try:
        b2.set_tf32_pair(2)
        for tail in (1, 0, 1):
            b2.set_tf32_tail_split(tail)
            out.setdefault(tail, []).append(run_gpu(1, a, b, c, alpha, beta))
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_tail_split(1)
    assert np.array_equal(out[1][0], out[1][1])                 # deterministic
    c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
    assert oracle.gemm_error(out[1][0], c64, den) <= 0.25 * TOL_3XTF32
    assert float(np.max(np.abs(out[1][0].astype(np.float64) - out[0][0]) / den)) <= 2e-7
    if shape == (2304, 2304, 2304):                             # five runs of one chunk each: the same chain of additions
        assert np.array_equal(out[1][0], out[0][0])


@pytest.mark.parametrize("pair", [2, 0])
@pytest.mark.parametrize("col_offset", [4, 1])
@pytest.mark.parametrize("N", [300, 301, 303, 3])
def test_3xtf32_chunked_strided_c(cuda, pair, col_offset, N):
    """C as a view inside a larger array: 16-byte aligned (the blocks travel by TMA, clipped at the view's edges; the
    columns after the last whole group of four go element by element) and not aligned (everything element by
    element from the registers).  Nothing outside the view moves."""
    import hpcdeepneuralnetworks_b200 as b2
    M, K, ldc = 200, 1200, 312
    a, b, _ = mats(M, N, K)
    Cb = oracle.fill_uniform((M + 3) * ldc, 3).reshape(M + 3, ldc)
    dC = dev(Cb)
    try:
        b2.set_tf32_pair(pair)
        b2.sgemm(M, N, K, 1.0, dev(a), dev(b), 0.5, dC[2:, col_offset:], path=1, ldc=ldc)
        b2.check_status()
    finally:
        b2.set_tf32_pair(1)
    got = dC.cpu().numpy()
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, Cb[2:M + 2, col_offset:col_offset + N])
    assert oracle.gemm_error(np.ascontiguousarray(got[2:M + 2, col_offset:col_offset + N]), c64, den) <= 0.25 * TOL_3XTF32
    mask = np.ones_like(Cb, dtype=bool)
    mask[2:M + 2, col_offset:col_offset + N] = False
    assert np.array_equal(got[mask], Cb[mask])


@pytest.mark.parametrize("pair", [2, 0])
def test_3xtf32_chunks_bound_the_loss_for_operands_of_one_sign(cuda, pair):
    """Operands of one sign make the tensor cores' truncating accumulation lose coherently: over all of K = 8192 in
    one go the error passes the path's tolerance; in chunks of 16 slabs it stays below a third of it, and signed
    operands come out ten times closer than without chunks."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = 512, 512, 8192
    A = b2.fill_uniform(torch.empty((M, K), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((K, N), device="cuda"), 2)
    err = {}
    try:
        b2.set_tf32_pair(pair)
        for name, (X, Y) in {"signed": (A, B), "positive": (A.abs().contiguous(), B.abs().contiguous())}.items():
            ref = X.double() @ Y.double()
            den = X.double().abs() @ Y.double().abs()
            for chunk in (0, -1):
                b2.set_tf32_chunk(chunk)
                Cm = torch.zeros((M, N), device="cuda")
                b2.sgemm(M, N, K, 1.0, X, Y, 0.0, Cm, path=1)
                b2.check_status()
                err[name, chunk] = float(((Cm.double() - ref).abs() / den).max().item())
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_chunk(-1)
    assert err["positive", 0] > TOL_3XTF32, err          # the loss the chunks are there for
    assert err["positive", -1] <= 7e-6, err
    assert err["signed", -1] <= 1e-6 and err["signed", -1] < 0.2 * err["signed", 0], err


@pytest.mark.parametrize("shape", [(2816, 2816, 96), (3840, 3840, 40), (3584, 1920, 70), (5000, 3000, 33)])
def test_ffma_row_split_is_bit_identical(cuda, shape):
    """A product that the time model runs as two launches on different tiles (b2_ffma_row_split_plan) gives the bits of
    the single launch and of the fused oracle: every output is one FMA chain over all of K on any tile."""
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import _lib
    M, N, K = shape
    a, b, c = mats(M, N, K)
    out = {}
    try:
        for on in (1, 0):
            b2.set_ffma_row_split(on)
            out[on] = run_gpu(0, a, b, c, 1.0, 0.5)
    finally:
        b2.set_ffma_row_split(1)
    assert np.array_equal(out[1], out[0])
    assert np.array_equal(out[1], oracle.sgemm_fma(1.0, a, b, 0.5, c))
    if shape[:2] in ((2816, 2816), (3840, 3840)):
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        assert sms != 148 or _lib.load().b2_ffma_row_split_plan(M, N, sms, None, None, None) == 1     # the split did happen


def test_random_shapes_through_the_dispatchers(cuda):
    """Forty seeded random shapes (M, N up to 700, K up to 2600, leading dimensions with slack, alpha and beta drawn
    from {0, 1, -1.5, 0.5, 2}) through both dispatchers as a caller would use them - whatever tile, kernel form, split,
    chunking or cut of the last round they choose: FFMA bit-exact against the fused oracle, 3xTF32 within its tolerance,
    nothing outside the M x N view touched."""
    import hpcdeepneuralnetworks_b200 as b2
    rng = np.random.default_rng(20240607)
    for case in range(40):
        M, N = int(rng.integers(1, 700)), int(rng.integers(1, 700))
        K = int(rng.integers(1, 2600)) if case % 3 else int(rng.integers(1, 200))
        pad = lambda x: (x + 3) // 4 * 4 + 4 * int(rng.integers(0, 3))
        lda, ldb, ldc = pad(K), pad(N), pad(N)
        alpha, beta = float(rng.choice([1.0, -1.5, 0.5, 2.0])), float(rng.choice([0.0, 1.0, -1.5, 0.5]))
        A = oracle.fill_uniform(M * lda, 100 + case).reshape(M, lda)
        B = oracle.fill_uniform(K * ldb, 200 + case).reshape(K, ldb)
        Cb = oracle.fill_uniform(M * ldc, 300 + case).reshape(M, ldc)
        a, b, c = np.ascontiguousarray(A[:, :K]), np.ascontiguousarray(B[:, :N]), np.ascontiguousarray(Cb[:, :N])
        c64, den = oracle.sgemm_f64(alpha, a, b, beta, c)
        want = oracle.sgemm_fma(alpha, a, b, beta, c)
        for path, tol in ((0, TOL_FFMA), (1, TOL_3XTF32)):
            dC = dev(Cb)
            b2.sgemm(M, N, K, alpha, dev(A), dev(B), beta, dC, path=path, lda=lda, ldb=ldb, ldc=ldc)
            b2.check_status()
            got = dC.cpu().numpy()
            tag = (case, path, M, N, K, lda, ldb, ldc, alpha, beta)
            assert np.array_equal(got[:, N:], Cb[:, N:]), tag
            if path == 0:
                assert np.array_equal(got[:, :N], want), tag
            assert oracle.gemm_error(np.ascontiguousarray(got[:, :N]), c64, den) <= tol, tag


def test_sweep_sizes_both_paths(cuda):
    """Benchmark configuration 2 (alpha=1, beta=0.5) at a few sweep sizes, inputs generated on the device; checked on
    sampled rows against the double reference."""
    import hpcdeepneuralnetworks_b200 as b2
    for n in (768, 2048):
        A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
        B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
        C0 = b2.fill_uniform(torch.empty((n, n), device="cuda"), 3)
        rows = np.array([0, 1, n // 2 - 1, n // 2, n - 1])
        a, b, c0 = A.cpu().numpy(), B.cpu().numpy(), C0.cpu().numpy()
        c64, den = oracle.sgemm_f64(1.0, a[rows], b, 0.5, c0[rows])
        for path, tol in ((0, TOL_FFMA), (1, TOL_3XTF32)):
            Cm = C0.clone()
            b2.sgemm(n, n, n, 1.0, A, B, 0.5, Cm, path=path)
            b2.check_status()
            got = Cm.cpu().numpy()[rows]
            assert oracle.gemm_error(got, c64, den) <= tol
            if path == 0:
                assert np.array_equal(got, oracle.sgemm_fma(1.0, a[rows], b, 0.5, c0[rows]))


def test_full_size_6144_properties(cuda):
    """6144^3 (the metric's size): linearity in alpha and agreement of the two math paths, plus sampled rows."""
    import hpcdeepneuralnetworks_b200 as b2
    n = 6144
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    C1 = torch.zeros((n, n), device="cuda")
    C2 = torch.zeros((n, n), device="cuda")
    b2.sgemm(n, n, n, 1.0, A, B, 0.0, C1)
    b2.sgemm(n, n, n, 2.0, A, B, 0.0, C2)
    assert torch.equal(C2, 2.0 * C1)                          # scaling by 2 is exact
    C3 = torch.zeros((n, n), device="cuda")
    b2.sgemm(n, n, n, 1.0, A, B, 0.0, C3, path=1)
    b2.check_status()
    scale = n / 4.0                                           # E[(|A|.|B|)_ij] for uniform[-1,1]
    assert float((C3 - C1).abs().max().item()) <= 3e-5 * scale
    rows = np.array([5, 3071, 6143])
    a, b = A[rows].cpu().numpy(), B.cpu().numpy()
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.0, np.zeros((3, n), np.float32))
    assert oracle.gemm_error(C1[rows].cpu().numpy(), c64, den) <= TOL_FFMA
    assert oracle.gemm_error(C3[rows].cpu().numpy(), c64, den) <= TOL_3XTF32


@pytest.mark.parametrize("shape,panel,panel_k", [((300, 260, 128), 1024, 1024), ((700, 260, 512), 256, 128), ((64, 40, 32), 1024, 1024),
                                                 ((520, 384, 300), 128, 1024)])
@pytest.mark.parametrize("beta", [0.5, 0.0])
def test_host_buffer_api(cuda, shape, panel, panel_k, beta):
    """Host arrays in, host array out, through the pipelined three-stream path.  One K panel: bit-identical to one
    device call; several K panels: bit-identical to the same panel schedule on the CPU, and within the tolerance."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    hs = b2.HostSgemm(M, N, K, panel_rows=panel, panel_k=panel_k)
    hs.hA.copy_(torch.from_numpy(a)); hs.hB.copy_(torch.from_numpy(b)); hs.hC.copy_(torch.from_numpy(c))
    out = hs.run(1.0, beta).numpy().copy()
    want = c.copy()
    for i, k0 in enumerate(range(0, K, hs.pk)):
        k1 = min(K, k0 + hs.pk)
        want = oracle.sgemm_fma(1.0, np.ascontiguousarray(a[:, k0:k1]), np.ascontiguousarray(b[k0:k1]), beta if i == 0 else 1.0, want)
    assert np.array_equal(out, want)
    c64, den = oracle.sgemm_f64(1.0, a, b, beta, c)
    assert oracle.gemm_error(out, c64, den) <= TOL_FFMA
    hs.hC.copy_(torch.from_numpy(c))
    out2 = hs.run(1.0, beta, ft=(M >= 128)).numpy()          # second run on the same buffers, ABFT kernel
    assert np.array_equal(out2, out)


@pytest.mark.parametrize("shape,panel,panel_cols", [((300, 520, 96), 128, 128), ((1600, 700, 64), 512, 256), ((130, 2100, 40), 128, 1024),
                                                    ((256, 300, 72), 1536, 1536)])
@pytest.mark.parametrize("beta", [0.5, 0.0])
@pytest.mark.parametrize("path", [0, 1])
def test_host_buffer_api_column_panels(cuda, shape, panel, panel_cols, beta, path):
    """The default schedule of the host-buffer pipeline: the first row panel is computed in column tiles behind the
    pitched copies of B's column panels, the others full width.  Every output still sums all of K in one call, so the
    FFMA result is bit-identical to the oracle's single call whatever the panel sizes."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K)
    hs = b2.HostSgemm(M, N, K, path=path, panel_rows=panel, panel_cols=panel_cols)
    hs.hA.copy_(torch.from_numpy(a)); hs.hB.copy_(torch.from_numpy(b)); hs.hC.copy_(torch.from_numpy(c))
    out = hs.run(-1.5, beta).numpy().copy()
    c64, den = oracle.sgemm_f64(-1.5, a, b, beta, c)
    if path == 0:
        assert np.array_equal(out, oracle.sgemm_fma(-1.5, a, b, beta, c))
        assert oracle.gemm_error(out, c64, den) <= TOL_FFMA
    else:
        assert oracle.gemm_error(out, c64, den) <= TOL_3XTF32
    hs.hC.copy_(torch.from_numpy(c))
    out2 = hs.run(-1.5, beta).numpy()                                 # the buffers are reusable
    assert np.array_equal(out2, out)


def test_bounded_wait_times_out_and_context_survives(cuda):
    """A device-side wait that nothing satisfies gives up after its limit, the host reads B2_ERR_TIMEOUT, and the
    next launches run normally (no trap, no hang, no lost context)."""
    import time
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    h = b2.default_handle()
    t0 = time.time()
    assert L.b2_selftest_wait_timeout(h.raw, 2000, None) == 0          # 2 ms limit
    with pytest.raises(b2.B2Error) as e:
        b2.check_status()
    assert e.value.status == -4 and time.time() - t0 < 5.0
    b2.check_status()                                                   # the status word was cleared
    a, b, c = mats(128, 128, 64)
    assert np.array_equal(run_gpu(0, a, b, c, 1.0, 0.5), oracle.sgemm_fma(1.0, a, b, 0.5, c))
    assert L.b2_selftest_wait_timeout(h.raw, 0, None) == -1


def test_unchecked_timeout_does_not_stop_later_launches(cuda):
    """A timeout that nobody has read yet (the status word is sticky until b2_check_status) must not turn later SGEMMs
    into no-ops: every kernel form still computes, and the recorded status is still there to be read afterwards."""
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    h = b2.default_handle()
    assert L.b2_selftest_wait_timeout(h.raw, 2000, None) == 0
    torch.cuda.synchronize()
    a, b, c = mats(256, 512, 96)
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)

    def run(path):                       # run_gpu without its status check
        dc = dev(c)
        b2.sgemm(256, 512, 96, 1.0, dev(a), dev(b), 0.5, dc, path=path)
        return dc.cpu().numpy()
    assert np.array_equal(run(0), oracle.sgemm_fma(1.0, a, b, 0.5, c))
    try:
        for pair, persistent in ((0, 0), (2, 0), (2, 1)):
            b2.set_tf32_pair(pair)
            b2.set_tf32_persistent(persistent)
            assert oracle.gemm_error(run(1), c64, den) <= TOL_3XTF32
            da, db, dc = dev(a), dev(b), dev(c)
            b2.ft_sgemm(256, 512, 96, 1.0, da, db, 0.5, dc, path=1)
            assert oracle.gemm_error(dc.cpu().numpy(), c64, den) <= TOL_3XTF32
    finally:
        b2.set_tf32_pair(1)
        b2.set_tf32_persistent(1)
    with pytest.raises(b2.B2Error) as e:
        b2.check_status()
    assert e.value.status == -4
    b2.check_status()


@pytest.mark.parametrize("shape", [(128, 2048, 32), (130, 2052, 70), (257, 2304, 129), (1024, 3072, 512)])
def test_ffma_transposed_a_route_is_bit_identical(cuda, shape):
    """With scratch available the FFMA path first transposes a row-major A (K-major A tiles are faster); every output
    still sums its k in the same order, so the result is bit-identical to the direct route and to the oracle."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    assert b2.sgemm_workspace_bytes(0, M, N, K) > 0
    a, b, c = mats(M, N, K)
    out = {}
    try:
        for mode in (1, 0):
            b2.set_ffma_transpose_a(mode)
            out[mode] = run_gpu(0, a, b, c, -1.5, 0.5)
    finally:
        b2.set_ffma_transpose_a(1)
    assert np.array_equal(out[1], out[0])
    if M * N * K <= 130 * 2052 * 70:
        assert np.array_equal(out[1], oracle.sgemm_fma(-1.5, a, b, 0.5, c))


def test_ffma_transposed_a_route_needs_no_workspace(cuda):
    """A caller-supplied workspace that is too small is not an error for the FFMA path: the direct kernel runs."""
    import ctypes as C
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    M, N, K = 256, 2048, 64
    a, b, c = mats(M, N, K)
    h = C.c_void_p()
    assert L.b2_create(C.byref(h)) == 0
    small = torch.empty(4096, dtype=torch.uint8, device="cuda")
    base = (small.data_ptr() + 1023) & ~1023
    try:
        assert L.b2_set_workspace(h, C.c_void_p(base), 1024) == 0
        da, db, dc = dev(a), dev(b), dev(c)
        torch.cuda.synchronize()
        st = L.b2_sgemm(h, 0, M, N, K, 1.0, C.c_void_p(da.data_ptr()), K, C.c_void_p(db.data_ptr()), N, 0.5,
                        C.c_void_p(dc.data_ptr()), N, None)
        assert st == 0, L.b2_last_error()
        torch.cuda.synchronize()
        assert np.array_equal(dc.cpu().numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))
    finally:
        L.b2_set_workspace(h, None, 0)
        L.b2_destroy(h)


@pytest.mark.parametrize("n", [128, 256, 640])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (1.0, 0.5), (2.0, 0.25)])
def test_bit_identical_to_the_reference_gpu_kernel(cuda, tmp_path, n, alpha, beta):
    """The reference's own sgemm_11 kernel (kernel/sgemm/include/kernel_11.cuh:15), compiled unmodified from the
    reference tree into oracle/_ref/ref_kernel_dump, run here on the same seeded inputs: the FFMA path, the series
    rung that restates that kernel and the CPU oracle all reproduce its output bit for bit.  (alpha and beta are
    powers of two, so that alpha*t + beta*c rounds once whichever product the compiler fuses.)"""
    import subprocess
    import hpcdeepneuralnetworks_b200 as b2
    exe = os.path.join(os.path.dirname(oracle.__file__), "_ref", "ref_kernel_dump")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/ref_kernel_dump was not built (no reference tree at build time)")
    out = tmp_path / "c.bin"
    r = subprocess.run([exe, str(n), repr(alpha), repr(beta), str(out)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = np.fromfile(out, dtype=np.float32).reshape(n, n)
    a, b, c = mats(n, n, n)
    assert np.array_equal(run_gpu(0, a, b, c, alpha, beta), ref)
    assert np.array_equal(oracle.sgemm_fma(alpha, a, b, beta, c), ref)
    dc = dev(c)
    b2.sgemm_series(11, n, dev(a), dev(b), dc, alpha, beta)
    assert np.array_equal(dc.cpu().numpy(), ref)


@pytest.mark.parametrize("shape", [(128, 128, 8), (256, 128, 64), (384, 256, 200)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (1.0, 0.5), (-2.0, 0.25)])
def test_colmajor_nt_bit_identical_to_the_reference_generated_kernel(cuda, tmp_path, shape, alpha, beta):
    """The reference's generated column-major kernel sgemm_huge (kernel/ft_sgemm/include_code_gen/sgemm_huge.cuh:11),
    compiled unmodified and run on the same seeded inputs (its A and B allocated one K-slab larger, because it
    prefetches one slab past the end): ref_sgemm_colmajor_nt and the CPU oracle reproduce its C bit for bit."""
    import subprocess
    import hpcdeepneuralnetworks_b200 as b2
    exe = os.path.join(os.path.dirname(oracle.__file__), "_ref", "ref_kernel_dump")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/ref_kernel_dump was not built (no reference tree at build time)")
    M, N, K = shape
    out = tmp_path / "c.bin"
    r = subprocess.run([exe, "nt", str(M), str(N), str(K), repr(alpha), repr(beta), str(out)], capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = np.fromfile(out, dtype=np.float32)
    af = oracle.fill_uniform(M * K, 1)
    bf = oracle.fill_uniform(N * K, 2)
    cf = oracle.fill_uniform(M * N, 3)
    dcf = dev(cf)
    b2.sgemm_colmajor_nt(M, N, K, dev(af), dev(bf), dcf, alpha, beta)
    assert np.array_equal(dcf.cpu().numpy().ravel(), ref)
    assert np.array_equal(np.asarray(oracle.sgemm_colmajor_nt(M, N, K, alpha, af, bf, beta, cf)).ravel(), ref)


def test_two_devices_in_one_process(cuda):
    """One process that drives two GPUs: the kernels' shared-memory opt-in and the resident-pair count are per
    device, and a handle is refused while another device than its own is current."""
    import hpcdeepneuralnetworks_b200 as b2
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    a, b, c = mats(512, 768, 256)
    c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
    want = oracle.sgemm_fma(1.0, a, b, 0.5, c)
    try:
        for d in (0, 1, 0):
            with torch.cuda.device(d):
                da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
                dc = torch.from_numpy(c).cuda()
                b2.sgemm(512, 768, 256, 1.0, da, db, 0.5, dc, path=0)
                assert np.array_equal(dc.cpu().numpy(), want)
                for pair in (0, 2):
                    b2.set_tf32_pair(pair)
                    dc = torch.from_numpy(c).cuda()
                    b2.sgemm(512, 768, 256, 1.0, da, db, 0.5, dc, path=1)
                    assert oracle.gemm_error(dc.cpu().numpy(), c64, den) <= TOL_3XTF32
                    dc = torch.from_numpy(c).cuda()
                    b2.ft_sgemm(512, 768, 256, 1.0, da, db, 0.5, dc, path=1)
                    assert oracle.gemm_error(dc.cpu().numpy(), c64, den) <= TOL_3XTF32
                b2.check_status()
        with torch.cuda.device(0):
            h0 = b2.Handle()
        with torch.cuda.device(1):
            da, db, dc = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(c).cuda()
            with pytest.raises(b2.B2Error) as e:
                b2.sgemm(512, 768, 256, 1.0, da, db, 0.5, dc, handle=h0)
            assert e.value.status == -1 and "device" in str(e.value)
        with torch.cuda.device(0):
            h0.close()
    finally:
        b2.set_tf32_pair(1)
        torch.cuda.set_device(0)


def test_two_host_threads_one_handle_each(cuda):
    """Two host threads on one GPU, each with its own handle and stream, launching both math paths at the same time:
    every result is the oracle's (the library keeps no per-call state outside the handle)."""
    import threading
    import hpcdeepneuralnetworks_b200 as b2
    shapes = [(384, 512, 160), (256, 2304, 96)]
    cases = []
    for M, N, K in shapes:
        a, b, c = mats(M, N, K)
        cases.append((M, N, K, a, b, c, oracle.sgemm_fma(1.0, a, b, 0.5, c), oracle.sgemm_f64(1.0, a, b, 0.5, c)))
    errors = []

    def work(i):
        try:
            torch.cuda.set_device(0)
            h = b2.Handle()
            stream = torch.cuda.Stream()
            M, N, K, a, b, c, want, (c64, den) = cases[i]
            with torch.cuda.stream(stream):
                da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
                for it in range(20):
                    dc = torch.from_numpy(c).cuda()
                    b2.sgemm(M, N, K, 1.0, da, db, 0.5, dc, path=0, handle=h)
                    stream.synchronize()
                    if not np.array_equal(dc.cpu().numpy(), want):
                        errors.append(f"thread {i} iteration {it}: FFMA result differs")
                    dc = torch.from_numpy(c).cuda()
                    b2.sgemm(M, N, K, 1.0, da, db, 0.5, dc, path=1, handle=h)
                    stream.synchronize()
                    if oracle.gemm_error(dc.cpu().numpy(), c64, den) > TOL_3XTF32:
                        errors.append(f"thread {i} iteration {it}: 3xTF32 result out of tolerance")
                b2.check_status(h)
            h.close()
        except Exception as e:       # a failed assertion in a thread would otherwise be lost
            errors.append(f"thread {i}: {type(e).__name__}: {e}")

    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert errors == []


@pytest.mark.parametrize("shape,ways", [((256, 256, 256), 4), ((300, 260, 1000), 3), ((64, 64, 2048), 8), ((130, 70, 96), 2),
                                        ((512, 384, 640), -1)])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_split_k_is_deterministic_exactly_modelled_and_within_tolerance(cuda, shape, ways, beta):
    """The opt-in split-K form of the FFMA path: each output is the sum, in ascending order, of `ways` FMA chains over
    consecutive shares of K.  Deterministic run to run, bit-identical to that model (alpha = 1, beta = 0, where the
    epilogue adds no rounding of its own), inside the path's tolerance; off again, the default is the single chain."""
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K = shape
    a, b, c = mats(M, N, K, beta)
    c64, den = oracle.sgemm_f64(1.0, a, b, beta, c)
    try:
        b2.set_ffma_split_k(ways)
        out1 = run_gpu(0, a, b, c, 1.0, beta)
        out2 = run_gpu(0, a, b, c, 1.0, beta)
        assert np.array_equal(out1, out2)
        assert oracle.gemm_error(out1, c64, den) <= TOL_FFMA
        if beta == 0.0 and ways > 1:
            slabs = (K + 31) // 32
            w = min(ways, 8, slabs // 2)
            per = (slabs + w - 1) // w * 32
            total = None
            for k0 in range(0, per * w, per):
                k1 = min(K, k0 + per)
                part = (np.zeros((M, N), np.float32) if k0 >= K else
                        oracle.sgemm_fma(1.0, np.ascontiguousarray(a[:, k0:k1]), np.ascontiguousarray(b[k0:k1]), 0.0, np.zeros((M, N), np.float32)))
                total = part if total is None else (total + part).astype(np.float32)
            assert np.array_equal(out1, total)
    finally:
        b2.set_ffma_split_k(0)
    assert np.array_equal(run_gpu(0, a, b, c, 1.0, beta), oracle.sgemm_fma(1.0, a, b, beta, c))

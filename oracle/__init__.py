"""CPU oracle for the FP32 BLAS hot path -- TEST INFRASTRUCTURE ONLY.

Python binding (ctypes) of ``oracle.c`` and, when it has been built, of the reference's
own ``utils/utils.cu`` (``oracle/_ref/libref_utils.so``).  Only ``tests/``, the smoke
check and the benchmark's CPU-baseline leg import this package; the product package
never does.

Parity pinning: the reference holds no golden vectors for this path.  ``cpu_gemm`` here
is pinned bit-for-bit against the reference's compiled ``cpu_gemm`` (``ref_cpu_gemm``)
and by the committed fixtures under ``tests/golden``; SAXPY/SDOT/ABFT are restatements
of kernel arithmetic (kernel/saxpy/saxpy.cu:44-47, kernel/sdot/sdot.cu:15-19,
kernel/ft_sgemm/README.md:4-14) and are pinned by fixtures generated from them only.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


class Fault(C.Structure):
    """Mirror of ``b2_fault`` (include/b2blas.h)."""

    _fields_ = [("tile_m", C.c_int32), ("tile_n", C.c_int32), ("row", C.c_int32),
                ("col", C.c_int32), ("k_step", C.c_int32), ("bit", C.c_int32)]


def reference_tree():
    """The reference project's source tree, or None: the directory named by B2_REFERENCE_TREE, else a directory
    called ``reference`` beside this repository.  It exists where the checker is built, not where the GPU tests run
    (they use the prebuilt files under oracle/_ref)."""
    cand = os.environ.get("B2_REFERENCE_TREE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "utils", "utils.cu")) else None


def build(force: bool = False) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "--no-print-directory", os.path.join(_HERE, "liboracle.so")],
                              stdout=subprocess.DEVNULL)
    ref = reference_tree()
    if ref and (force or not os.path.exists(os.path.join(_HERE, "_ref", "libref_utils.so"))):
        subprocess.call(["make", "-C", _HERE, "--no-print-directory", "ref", "REFERENCE=" + ref], stdout=subprocess.DEVNULL,
                        stderr=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        build()
        L = C.CDLL(os.path.join(_HERE, "liboracle.so"))
        L.o_uniform_at.restype = C.c_float
        L.o_uniform_at.argtypes = [C.c_uint64, C.c_uint64]
        L.o_fill_uniform.argtypes = [_f32p, C.c_int64, C.c_uint64]
        L.o_cpu_gemm.argtypes = [C.c_float, C.c_float, _f32p, _f32p, C.c_int, _f32p]
        for name in ("o_sgemm_f32", "o_sgemm_fma"):
            getattr(L, name).argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _f32p, C.c_int, _f32p, C.c_int,
                                         C.c_float, _f32p, C.c_int, C.c_int]
        L.o_sgemm_f64.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _f32p, C.c_int, _f32p, C.c_int, C.c_float,
                                  _f32p, C.c_int, _f64p, _f64p, C.c_int]
        L.o_gemm_error.restype = C.c_double
        L.o_gemm_error.argtypes = [C.c_int, C.c_int, _f32p, C.c_int, _f64p, _f64p]
        L.o_sgemm_colmajor_nt.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _f32p, _f32p, C.c_float, _f32p]
        L.o_saxpy.argtypes = [C.c_int64, C.c_float, _f32p, _f32p]
        L.o_sdot.restype = C.c_double
        L.o_sdot.argtypes = [C.c_int64, _f32p, _f32p, C.POINTER(C.c_double), C.c_int]
        L.o_ft_fault_effect.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.POINTER(Fault),
                                        C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_int)]
        L.o_abft_tile_checksums.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.c_int,
                                            C.c_int, _f64p, _f64p]
        L.o_verify_matrix.argtypes = [_f32p, _f32p, C.c_int]
        L.o_verify_vector.argtypes = [_f32p, _f32p, C.c_int]
        _LIB = L
    return _LIB


def ref_lib():
    """The reference's own utils/utils.cu compiled as a shared object, or None."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libref_utils.so")
        if not os.path.exists(path):
            build()
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        # cpu_gemm(float alpha, float beta, float*, float*, int n, float*)  utils/utils.cu:93
        R._Z8cpu_gemmffPfS_iS_.argtypes = [C.c_float, C.c_float, _f32p, _f32p, C.c_int, _f32p]
        R._Z8cpu_gemmffPfS_iS_.restype = None
        # bool verify_matrix(float*, float*, int)  utils/utils.cu:75
        R._Z13verify_matrixPfS_i.argtypes = [_f32p, _f32p, C.c_int]
        R._Z13verify_matrixPfS_i.restype = C.c_bool
        # void generate_random_matrix(float*, int)  utils/utils.cu:36
        R._Z22generate_random_matrixPfi.argtypes = [_f32p, C.c_int]
        R._Z22generate_random_matrixPfi.restype = None
        _REF = R
    return _REF


def threads() -> int:
    return max(1, os.cpu_count() or 1)


# ---- inputs -------------------------------------------------------------------------
_M1 = np.uint64(0x9E3779B97F4A7C15)
_M2 = np.uint64(0xBF58476D1CE4E5B9)
_M3 = np.uint64(0x94D049BB133111EB)
_M4 = np.uint64(0xD1342543DE82EF95)


def _mix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + _M1
        z = (z ^ (z >> np.uint64(30))) * _M2
        z = (z ^ (z >> np.uint64(27))) * _M3
        return z ^ (z >> np.uint64(31))


def fill_uniform(n: int, seed: int, offset: int = 0) -> np.ndarray:
    """uniform[-1,1) stream `seed`, elements offset..offset+n (numpy, vectorised; same bits as
    ``o_fill_uniform`` and as the device fill kernel)."""
    with np.errstate(over="ignore"):
        i = np.arange(offset, offset + n, dtype=np.uint64)
        s = _mix64(np.array([seed], dtype=np.uint64))[0]
        h = _mix64(s ^ (i * _M4))
    u = (h >> np.uint64(40)).astype(np.float32)
    return u * np.float32(1.0 / 8388608.0) - np.float32(1.0)


def fill_uniform_c(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().o_fill_uniform(out, n, seed)
    return out


# ---- GEMM ---------------------------------------------------------------------------
def cpu_gemm(alpha: float, beta: float, a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """utils/utils.cu:93-103 restated; square n x n, returns the updated copy of c."""
    n = a.shape[0]
    out = np.ascontiguousarray(c, dtype=np.float32).copy()
    lib().o_cpu_gemm(alpha, beta, np.ascontiguousarray(a), np.ascontiguousarray(b), n, out)
    return out


def ref_cpu_gemm(alpha: float, beta: float, a: np.ndarray, b: np.ndarray, c: np.ndarray):
    """The reference's compiled cpu_gemm itself (None when oracle/_ref is not built)."""
    R = ref_lib()
    if R is None:
        return None
    out = np.ascontiguousarray(c, dtype=np.float32).copy()
    R._Z8cpu_gemmffPfS_iS_(alpha, beta, np.ascontiguousarray(a).copy(), np.ascontiguousarray(b).copy(), a.shape[0], out)
    return out


def _gemm(fn, alpha, a, b, beta, c, nthreads):
    M, K = a.shape
    N = b.shape[1]
    out = np.ascontiguousarray(c, dtype=np.float32).copy()
    fn(M, N, K, alpha, np.ascontiguousarray(a), K, np.ascontiguousarray(b), N, beta, out, N,
       nthreads or threads())
    return out


def sgemm_f32(alpha, a, b, beta, c, nthreads=None):
    """cpu_gemm arithmetic (separate multiply and add) for any MxNxK."""
    return _gemm(lib().o_sgemm_f32, alpha, a, b, beta, c, nthreads)


def sgemm_fma(alpha, a, b, beta, c, nthreads=None):
    """fmaf in ascending k, epilogue fmaf(alpha, acc, beta*c): bit-exact model of the FFMA path."""
    return _gemm(lib().o_sgemm_fma, alpha, a, b, beta, c, nthreads)


def sgemm_f64(alpha, a, b, beta, c, nthreads=None):
    """(C_ref in double, sum_k |a||b| denominators), both dense MxN."""
    M, K = a.shape
    N = b.shape[1]
    c64 = np.empty((M, N), dtype=np.float64)
    den = np.empty((M, N), dtype=np.float64)
    lib().o_sgemm_f64(M, N, K, alpha, np.ascontiguousarray(a), K, np.ascontiguousarray(b), N, beta,
                      np.ascontiguousarray(c, dtype=np.float32), N, c64, den, nthreads or threads())
    return c64, den


def gemm_error(got: np.ndarray, c64: np.ndarray, den: np.ndarray) -> float:
    """North-star metric max|C - C_ref| / (|A|.|B|)."""
    M, N = c64.shape
    g = np.ascontiguousarray(got, dtype=np.float32)
    return float(lib().o_gemm_error(M, N, g, N, c64, den))


def sgemm_colmajor_nt(M, N, K, alpha, a, b, beta, c):
    """kernel/ft_sgemm layout: a (flat, MxK col-major), b (flat, NxK col-major), c (flat MxN col-major)."""
    out = np.ascontiguousarray(c, dtype=np.float32).copy()
    lib().o_sgemm_colmajor_nt(M, N, K, alpha, np.ascontiguousarray(a), np.ascontiguousarray(b), beta, out)
    return out


# ---- vectors ------------------------------------------------------------------------
def saxpy(alpha: float, x: np.ndarray, y: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(y, dtype=np.float32).copy()
    lib().o_saxpy(out.size, alpha, np.ascontiguousarray(x), out)
    return out


def sdot(x: np.ndarray, y: np.ndarray, nthreads=None):
    """(sum x*y in double, sum |x*y| in double)."""
    ab = C.c_double(0.0)
    s = lib().o_sdot(x.size, np.ascontiguousarray(x), np.ascontiguousarray(y), C.byref(ab), nthreads or threads())
    return float(s), float(ab.value)


# ---- ABFT ---------------------------------------------------------------------------
def fault_effect(a: np.ndarray, b: np.ndarray, fault) -> tuple:
    """(clean accumulator, faulty accumulator, in_range) for one planned fault; `fault` is a
    (tile_m, tile_n, row, col, k_step, bit) tuple."""
    M, K = a.shape
    N = b.shape[1]
    f = Fault(*[int(v) for v in fault])
    clean, bad, ok = C.c_float(), C.c_float(), C.c_int()
    lib().o_ft_fault_effect(M, N, K, np.ascontiguousarray(a), K, np.ascontiguousarray(b), N, C.byref(f),
                            C.byref(clean), C.byref(bad), C.byref(ok))
    return clean.value, bad.value, bool(ok.value)


def abft_tile_checksums(a: np.ndarray, b: np.ndarray, tile_m: int, tile_n: int):
    M, K = a.shape
    N = b.shape[1]
    r = np.zeros(128, dtype=np.float64)
    c = np.zeros(128, dtype=np.float64)
    lib().o_abft_tile_checksums(M, N, K, np.ascontiguousarray(a), K, np.ascontiguousarray(b), N, tile_m, tile_n, r, c)
    return r, c


def make_fault_plan(M: int, N: int, K: int, seed: int, tiles_per_fault: int = 64, bit_lo: int = 20, bit_hi: int = 30):
    """Seeded plan of benchmark configuration 3: one bit flip (random bit bit_lo..bit_hi of a random
    accumulator, random K-slab) per `tiles_per_fault` output tiles of 128x128, at most one per tile.
    Returns an int32 array of shape (n, 6): tile_m, tile_n, row, col, k_step, bit."""
    tm, tn = (M + 127) // 128, (N + 127) // 128
    ntiles = tm * tn
    nf = max(1, ntiles // tiles_per_fault)
    rng = np.random.Generator(np.random.PCG64(seed))
    tiles = rng.choice(ntiles, size=nf, replace=False)
    plan = np.zeros((nf, 6), dtype=np.int32)
    nslab = max(1, (K + 31) // 32)
    for q, t in enumerate(sorted(int(v) for v in tiles)):
        i, j = divmod(t, tn)
        rows = min(128, M - i * 128)
        cols = min(128, N - j * 128)
        plan[q] = (i, j, rng.integers(0, rows), rng.integers(0, cols), rng.integers(0, nslab),
                   rng.integers(bit_lo, bit_hi + 1))
    return plan


def verify_matrix(m1: np.ndarray, m2: np.ndarray) -> bool:
    n = m1.shape[0]
    return bool(lib().o_verify_matrix(np.ascontiguousarray(m1, dtype=np.float32),
                                      np.ascontiguousarray(m2, dtype=np.float32), n))

"""Host-side mirror of the reference's kernel interface, calling the CUDA library through
its C ABI.  Names, argument order and meaning follow the reference:

* ``sgemm(M, N, K, alpha, A, B, beta, C)``  -- the north-star row-major launcher
  (kernel/sgemm/sgemm.cu:135-141 generalised), ``sgemm_series(kernel_id, N, A, B, C, alpha, beta)``
  -- the kernels ``sgemm_1..sgemm_14`` (kernel/sgemm/include/kernel_*.cuh).
* ``ft_sgemm(...)`` -- ABFT SGEMM (kernel/ft_sgemm/include/ft_sgemm_huge.cuh:21).
* ``saxpy(n, alpha, x, y)`` / ``sdot(n, x, y, out)`` (kernel/saxpy/saxpy.cu:38, kernel/sdot/sdot.cu:9).

Tensors are torch CUDA float32 tensors used only as device memory; all arithmetic happens in
libb2blas.so.  Errors surface as ``B2Error`` (the reference printf+exit()s).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import B2Error, Fault, FtReport, check

PATH_FFMA = 0
PATH_3XTF32 = 1


def _ptr(t):
    if t is None:
        return None
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise TypeError("expected a CUDA tensor")
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Handle:
    """Owner of per-device scratch (``b2_handle``).  The large workspace (3xTF32 planes) is a
    torch allocation handed to the library, so the library itself never calls cudaMalloc for it."""

    def __init__(self):
        self._L = _lib.load()
        self._h = C.c_void_p()
        check(self._L.b2_create(C.byref(self._h)))
        self._ws = None

    def close(self):
        if self._h:
            torch.cuda.synchronize()
            self._L.b2_destroy(self._h)
            self._h = C.c_void_p()
            self._ws = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reserve(self, nbytes: int):
        if nbytes <= 0:
            return
        if self._ws is None or self._ws.numel() < nbytes + 1024:
            torch.cuda.synchronize()
            self._ws = None
            self._ws = torch.empty(nbytes + 2048, dtype=torch.uint8, device="cuda")
            base = (self._ws.data_ptr() + 1023) & ~1023
            check(self._L.b2_set_workspace(self._h, C.c_void_p(base), self._ws.numel() - (base - self._ws.data_ptr())))

    @property
    def raw(self):
        return self._h


_default = {}


def default_handle() -> Handle:
    dev = torch.cuda.current_device()
    if dev not in _default:
        _default[dev] = Handle()
    return _default[dev]


def check_status(handle: Handle | None = None) -> None:
    """Synchronise and raise if a kernel's bounded wait ran out."""
    h = handle or default_handle()
    st = _lib.load().b2_check_status(h.raw, _stream())
    if st != 0:
        check(st if st < 0 else -3)


def sgemm(M, N, K, alpha, A, B, beta, Cm, *, path=PATH_FFMA, lda=None, ldb=None, ldc=None, handle=None):
    """Row-major C = alpha*A*B + beta*C on device tensors (in place on ``Cm``)."""
    L = _lib.load()
    h = handle or default_handle()
    h.reserve(L.b2_sgemm_workspace_bytes(path, M, N, K))   # required by the 3xTF32 path, optional speed-up for FFMA
    check(L.b2_sgemm(h.raw, path, M, N, K, alpha, _ptr(A), lda or K, _ptr(B), ldb or N, beta, _ptr(Cm), ldc or N,
                     _stream()))
    return Cm


def sgemm_series(kernel_id, N, A, B, Cm, alpha, beta, threads_x=32):
    """``sgemm_<kernel_id>(N, A, B, C, alpha, beta)`` of the reference series."""
    check(_lib.load().b2_sgemm_series(kernel_id, threads_x, N, _ptr(A), _ptr(B), _ptr(Cm), alpha, beta, _stream()))
    return Cm


def sgemm_colmajor_nt(M, N, K, A, B, Cm, alpha, beta):
    """kernel/ft_sgemm layout: column-major A (MxK), B stored NxK, C (MxN); C = alpha*A*B^T + beta*C.
    Runs on the default stream like the reference driver (kernel/ft_sgemm/sgemm.cu:114-157)."""
    torch.cuda.current_stream().synchronize()
    check(_lib.load().ref_sgemm_colmajor_nt(M, N, K, _ptr(A), _ptr(B), _ptr(Cm), alpha, beta))
    torch.cuda.synchronize()
    return Cm


def make_plan(plan) -> torch.Tensor | None:
    """(n,6) int array of (tile_m, tile_n, row, col, k_step, bit) -> device tensor of b2_fault."""
    if plan is None:
        return None
    arr = np.ascontiguousarray(np.asarray(plan, dtype=np.int32).reshape(-1, 6))
    return torch.from_numpy(arr).cuda()


def seeded_fault_plan(M, N, K, seed, tiles_per_fault=64, bit_lo=20, bit_hi=30) -> np.ndarray:
    """The injection plan of benchmark configuration 3: one bit flip (a random bit bit_lo..bit_hi of a random
    accumulator, after a random K-slab) per ``tiles_per_fault`` output tiles of 128 x 128, at most one per tile, drawn
    from ``seed``.  Returns an int32 array (n, 6) of (tile_m, tile_n, row, col, k_step, bit) for ``make_plan``."""
    tm, tn = (M + 127) // 128, (N + 127) // 128
    rng = np.random.Generator(np.random.PCG64(seed))
    struck = np.sort(rng.choice(tm * tn, size=max(1, (tm * tn) // tiles_per_fault), replace=False))
    slabs = max(1, (K + 31) // 32)
    plan = np.zeros((len(struck), 6), dtype=np.int32)
    for q, t in enumerate(struck):
        i, j = divmod(int(t), tn)
        plan[q] = (i, j, rng.integers(0, min(128, M - i * 128)), rng.integers(0, min(128, N - j * 128)),
                   rng.integers(0, slabs), rng.integers(bit_lo, bit_hi + 1))
    return plan


def ft_sgemm(M, N, K, alpha, A, B, beta, Cm, *, path=PATH_FFMA, plan=None, tau=0.0, report=None, lda=None, ldb=None,
             ldc=None, handle=None):
    """ABFT SGEMM.  ``plan``: device int32 tensor (n,6) from ``make_plan`` or None.  ``report``: device
    int32 tensor of 8 words that the call adds to (see ``FtReport``) or None.  ``tau``: > 0 absolute threshold,
    0 the default for operands of unit scale, < 0 that default scaled by 3*rms(A)*rms(B).  Returns ``Cm``."""
    L = _lib.load()
    h = handle or default_handle()
    h.reserve(L.b2_ft_sgemm_workspace_bytes(path, M, N, K))
    nf = 0 if plan is None else int(plan.shape[0])
    check(L.b2_ft_sgemm(h.raw, path, M, N, K, alpha, _ptr(A), lda or K, _ptr(B), ldb or N, beta, _ptr(Cm), ldc or N,
                        _ptr(plan), nf, tau, _ptr(report), _stream()))
    return Cm


def ft_sgemm_colmajor_nt(M, N, K, A, B, Cm, alpha, beta, *, plan=None, tau=0.0, report=None, handle=None):
    """ABFT SGEMM in the kernel/ft_sgemm layout (column-major A MxK, B NxK, C MxN; C = alpha*A*B^T + beta*C).
    A planned fault's (row, col) address C^T."""
    h = handle or default_handle()
    h.reserve(_lib.load().b2_ft_sgemm_workspace_bytes(PATH_FFMA, N, M, K))
    nf = 0 if plan is None else int(plan.shape[0])
    check(_lib.load().b2_ft_sgemm_colmajor_nt(h.raw, M, N, K, alpha, _ptr(A), _ptr(B), beta, _ptr(Cm), _ptr(plan), nf, tau,
                                              _ptr(report), _stream()))
    return Cm


def new_report() -> torch.Tensor:
    return torch.zeros(8, dtype=torch.int32, device="cuda")


def read_report(report: torch.Tensor) -> dict:
    v = report.cpu().tolist()
    import struct
    return {"tiles": v[0], "injected": v[1], "detected": v[2], "corrected": v[3], "uncorrectable": v[4],
            "false_alarms": v[5], "max_residual": struct.unpack("f", struct.pack("i", v[6]))[0]}


def saxpy(n, alpha, x, y, handle=None):
    """y <- alpha*x + y."""
    h = handle or default_handle()
    check(_lib.load().b2_saxpy(h.raw, n, alpha, _ptr(x), _ptr(y), _stream()))
    return y


def sdot(n, x, y, out=None, handle=None):
    """out[0] <- x . y (overwrites).  Returns the 1-element device tensor."""
    h = handle or default_handle()
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    check(_lib.load().b2_sdot(h.raw, n, _ptr(x), _ptr(y), _ptr(out), _stream()))
    return out


def sdot_fused(n, x, y, mailboxes, rank, world, seq, out=None, sum64=None, handle=None):
    """x . y summed over all ranks inside the kernel (``b2_sdot_fused``).  ``mailboxes``: list of the ``world`` device
    addresses (ints) of the ranks' 512-byte mailboxes.  Returns (float32 result tensor, float64 sum tensor)."""
    h = handle or default_handle()
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    if sum64 is None:
        sum64 = torch.empty(1, dtype=torch.float64, device=x.device)
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in mailboxes])
    check(_lib.load().b2_sdot_fused(h.raw, n, _ptr(x), _ptr(y), _ptr(out), _ptr(sum64), arr, rank, world, seq, _stream()))
    return out, sum64


def sdot_static(n, x, y, out):
    """out[0] <- x . y through the entry point that allocates nothing (``b2_sdot_static``): no handle, scratch in
    the library's own static device array, n <= 2**30.  ``out`` must be an existing 1-element device tensor."""
    check(_lib.load().b2_sdot_static(n, _ptr(x), _ptr(y), _ptr(out), _stream()))
    return out


def sdot_partial(n, x, y, out, partial64, handle=None):
    h = handle or default_handle()
    check(_lib.load().b2_sdot_partial(h.raw, n, _ptr(x), _ptr(y), _ptr(out), _ptr(partial64), _stream()))
    return out


# ---- host-buffer forms: what a caller holding host arrays (the reference drivers' situation
# before their cudaMemcpy calls, kernel/sgemm/sgemm.cu:50-58) would use -------------------------
class HostSgemm:
    """Row-major SGEMM on HOST arrays through ``b2_sgemm_host``: pinned host buffers ``hA``, ``hB``, ``hC`` (torch
    tensors used as page-locked memory) and a host plan of the library that owns the device copies, three streams
    and the pipeline schedule.

    Default schedule (one K panel, bit-identical to a single device call): the first ``first_panel_rows`` rows of C
    (default: half) are computed in column tiles of ``panel_cols`` behind the pitched copies of B's column panels, the
    other rows in panels of ``panel_rows`` as one full-width GEMM each as their rows land, and each row panel of C
    travels back as soon as it is done.  With ``panel_k > 0`` the second cut is along K instead and block (p, q) accumulates
    into C_p with beta on the first K panel and 1 afterwards (same tolerance, different rounding)."""

    def __init__(self, M, N, K, path=PATH_FFMA, panel_rows=0, panel_k=0, panel_cols=0, first_panel_rows=0, handle=None):
        self.M, self.N, self.K, self.path = M, N, K, path
        self._L = _lib.load()
        self._handle = handle or default_handle()
        def _round(want, extent, floor_at):
            return extent if extent < floor_at else max(128, (min(want, extent) + 127) // 128 * 128)
        self.pr0 = _round(first_panel_rows or (M + 1) // 2, M, 128)      # the library's own defaults and rounding
        self.pr = _round(panel_rows or min(1536, max(128, 128 * (296 // max(1, (N + 127) // 128)))), M, 128)
        self.pc = _round(panel_cols or 768, N, 256)
        self.pk = K if (K < 128 or panel_k <= 0) else _round(panel_k, K, 128)
        self.hA = torch.empty((M, K), dtype=torch.float32).pin_memory()
        self.hB = torch.empty((K, N), dtype=torch.float32).pin_memory()
        self.hC = torch.empty((M, N), dtype=torch.float32).pin_memory()
        # scratch for the largest panel product, handed to the library before the plan is made
        rows_max, k_max = min(max(self.pr, self.pr0), M), min(self.pk, K)
        if M > 0 and N > 0 and K > 0:
            self._handle.reserve(max(self._L.b2_ft_sgemm_workspace_bytes(path, rows_max, N, k_max),
                                     self._L.b2_ft_sgemm_workspace_bytes(path, rows_max, min(self.pc, N), k_max)))
        self._plan = C.c_void_p()
        check(self._L.b2_host_plan_create(C.byref(self._plan), self._handle.raw, path, M, N, K, first_panel_rows, panel_rows,
                                          panel_cols, max(panel_k, 0)))

    def h2d_bytes(self):
        return 4 * (self.M * self.K + self.K * self.N + self.M * self.N)

    def d2h_bytes(self):
        return 4 * self.M * self.N

    def run(self, alpha, beta, ft=False):
        """hC <- alpha*hA*hB + beta*hC through the device; returns hC (pinned) after everything has landed."""
        torch.cuda.current_stream().synchronize()      # earlier work of the caller on the handle's scratch
        check(self._L.b2_sgemm_host(self._plan, alpha, C.c_void_p(self.hA.data_ptr()), self.K, C.c_void_p(self.hB.data_ptr()),
                                    self.N, beta, C.c_void_p(self.hC.data_ptr()), self.N, 1 if ft else 0, None))
        return self.hC

    def close(self):
        if self._plan:
            self._L.b2_host_plan_destroy(self._plan)
            self._plan = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- harness ---------------------------------------------------------------------------------
def fill_uniform(t: torch.Tensor, seed: int):
    check(_lib.load().b2_fill_uniform(_ptr(t), t.numel(), seed, _stream()))
    return t


def fill_const(t: torch.Tensor, value: float):
    check(_lib.load().b2_fill_const(_ptr(t), t.numel(), value, _stream()))
    return t


def verify_matrix(ref: torch.Tensor, got: torch.Tensor, abs_tol: float = 1e-2):
    """verify_matrix of utils/utils.cu:75-91 on the device: (passed, max_abs_diff)."""
    rows, cols = ref.shape
    mx = C.c_float(0.0)
    r = check(_lib.load().b2_verify_matrix(_ptr(ref), _ptr(got), rows, cols, ref.stride(0), abs_tol, C.byref(mx), _stream()))
    return r == 0, mx.value


class EventTimer:
    """CUDA-event timer on the current stream (replaces the host-clock saxpy_timer, utils/utils.cuh:56-77)."""

    def __init__(self):
        self._L = _lib.load()
        self._t = C.c_void_p()
        check(self._L.b2_timer_create(C.byref(self._t)))

    def start(self):
        check(self._L.b2_timer_start(self._t, _stream()))

    def stop(self):
        check(self._L.b2_timer_stop(self._t, _stream()))

    def elapsed_ms(self) -> float:
        ms = C.c_float(0.0)
        check(self._L.b2_timer_elapsed_ms(self._t, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            self._L.b2_timer_destroy(self._t)
        except Exception:
            pass


def ffma_peak_tflops(launches: int = 3, ffma_per_thread: int = 1 << 20, packed: bool = False) -> float:
    """Measured FP32 SIMT peak of the current device (register-only FMA stream), TFLOP/s."""
    L = _lib.load()
    probe = L.b2_ffma2_peak_probe if packed else L.b2_ffma_peak_probe
    flops = C.c_double(0.0)
    check(probe(1, ffma_per_thread, C.byref(flops), _stream()))  # warm-up
    torch.cuda.synchronize()
    t = EventTimer()
    t.start()
    check(probe(launches, ffma_per_thread, C.byref(flops), _stream()))
    t.stop()
    return flops.value / (t.elapsed_ms() * 1e-3) / 1e12


def device_info() -> dict:
    sm, khz, mem = C.c_int(), C.c_int(), C.c_size_t()
    check(_lib.load().b2_device_info(C.byref(sm), C.byref(khz), C.byref(mem)))
    return {"sm_count": sm.value, "sm_clock_khz": khz.value, "global_mem_bytes": mem.value}


def set_ffma_row_split(on: int):
    """1 (default): the plain FFMA SGEMM may run as two launches on different tiles (rows split) when the time model
    favours it; results are bit-identical.  0: one launch."""
    check(_lib.load().b2_set_ffma_row_split(on))


def set_ffma_variant(v: int):
    check(_lib.load().b2_set_ffma_variant(v))


def ffma_tiles() -> list:
    """The generated FFMA tile family: [(index, name, bm, bn, threads)]."""
    L = _lib.load()
    out = []
    for i in range(L.b2_ffma_tile_count()):
        bm, bn, th, name = C.c_int(), C.c_int(), C.c_int(), C.c_char_p()
        check(L.b2_ffma_tile_info(i, C.byref(bm), C.byref(bn), C.byref(th), C.byref(name)))
        out.append((i, name.value.decode(), bm.value, bn.value, th.value))
    return out


def set_ffma_tile(index: int):
    """Pin the FFMA tile (index into ``ffma_tiles()``); -1 restores the automatic choice."""
    check(_lib.load().b2_set_ffma_tile(index))




def set_ffma_split_k(ways: int):
    """Split-K of the plain FFMA SGEMM: 0 never (default), 2..8 that many ways, -1 automatic."""
    check(_lib.load().b2_set_ffma_split_k(ways))


def set_tf32_tile_n(n: int):
    """Pin the 3xTF32 tile width (128 or 256; 0 = automatic)."""
    check(_lib.load().b2_set_tf32_tile_n(n))


def sgemm_workspace_bytes(path: int, M: int, N: int, K: int) -> int:
    """Bytes of workspace an M x N x K SGEMM uses on ``path`` (required for 3xTF32, optional for FFMA)."""
    return int(_lib.load().b2_sgemm_workspace_bytes(path, M, N, K))


def set_ft_level(level: int):
    """ABFT encode granularity of the FFMA path: 1 block-level (default), 2 thread-level (128 x 128 tile)."""
    check(_lib.load().b2_set_ft_level(level))


def set_ffma_transpose_a(on: int):
    """1 (default): the FFMA path may transpose a row-major A into the workspace first; 0: never."""
    check(_lib.load().b2_set_ffma_transpose_a(on))


def set_tf32_pair(on: int):
    """3xTF32 on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2): 0 never, 1 automatic (default), 2 always."""
    check(_lib.load().b2_set_tf32_pair(on))


def set_tf32_persistent(on: int):
    """1 (default): the plain CTA-pair 3xTF32 kernel is persistent; 0: one cluster per tile."""
    check(_lib.load().b2_set_tf32_persistent(on))


def set_tf32_chunk(slabs: int):
    """Plain 3xTF32 SGEMM: K-slabs (of 32) accumulated in tensor memory before they are added to FP32 sums in
    registers (default 16; applies when K spans more than two chunks); 0: one accumulation over all of K; negative:
    the default."""
    check(_lib.load().b2_set_tf32_chunk(slabs))


def set_tf32_fused_split(mode: int):
    """The 3xTF32 hi/lo split inside the GEMM kernel: 0 never, 1 for very small plain products (default), 2 whenever
    the operands' alignment allows."""
    check(_lib.load().b2_set_tf32_fused_split(mode))


def set_tf32_tail_split(on: int):
    """1 (default): the last, partial round of tiles of a chunked CTA-pair 3xTF32 call is shared out in chunks over all
    clusters; 0: every tile on one cluster."""
    check(_lib.load().b2_set_tf32_tail_split(on))


def set_tf32_abft_bias(bias: float):
    """Loss per K-slab that the 3xTF32 ABFT check expects of an accumulator (fraction of its value; < 0: built-in)."""
    check(_lib.load().b2_set_tf32_abft_bias(bias))


def set_tf32_slab_k(k: int):
    """K-slab depth of the 3xTF32 kernel (16 or 32)."""
    check(_lib.load().b2_set_tf32_slab_k(k))

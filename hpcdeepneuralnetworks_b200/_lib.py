"""ctypes binding of libb2blas.so (the C ABI declared in include/b2blas.h).

The library is the product: if it is missing or fails to load, importing the operators
raises -- there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libb2blas.so")
HEADER = os.path.join(PKG, "..", "include", "b2blas.h")

_lib = None


class B2Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b2blas status {status}: {message}")
        self.status = status


class Fault(C.Structure):
    """``b2_fault`` of include/b2blas.h."""

    _fields_ = [("tile_m", C.c_int32), ("tile_n", C.c_int32), ("row", C.c_int32),
                ("col", C.c_int32), ("k_step", C.c_int32), ("bit", C.c_int32)]


class FtReport(C.Structure):
    """``b2_ft_report`` of include/b2blas.h."""

    _fields_ = [("tiles", C.c_int32), ("injected", C.c_int32), ("detected", C.c_int32),
                ("corrected", C.c_int32), ("uncorrectable", C.c_int32), ("false_alarms", C.c_int32),
                ("max_residual_bits", C.c_int32), ("reserved", C.c_int32)]


def declared_symbols() -> list[str]:
    """Every function name include/b2blas.h declares."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:int|size_t|const char \*)\s*\*?\s*(\w+)\s*\(", text)
    return sorted(set(n for n in names if n not in ("defined",)))


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hpcdeepneuralnetworks_b200.build` "
            "(nvcc, sm_100a). There is no fallback path.")
    import torch  # noqa: F401  (loads libcudart.so.12 into the process before our library)

    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, i32, i64, f32, u64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64
    L.b2_status_string.restype = C.c_char_p
    L.b2_status_string.argtypes = [i32]
    L.b2_last_error.restype = C.c_char_p
    L.b2_version.restype = i32
    L.b2_create.argtypes = [C.POINTER(vp)]
    L.b2_destroy.argtypes = [vp]
    L.b2_set_workspace.argtypes = [vp, vp, C.c_size_t]
    L.b2_sgemm_workspace_bytes.restype = C.c_size_t
    L.b2_sgemm_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.b2_ft_sgemm_workspace_bytes.restype = C.c_size_t
    L.b2_ft_sgemm_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.sgemm.argtypes = [i32, i32, i32, f32, vp, vp, f32, vp]
    L.ft_sgemm.argtypes = [i32, i32, i32, f32, vp, vp, f32, vp]
    L.b2_sgemm.argtypes = [vp, i32, i32, i32, i32, f32, vp, i32, vp, i32, f32, vp, i32, vp]
    L.b2_sgemm_series.argtypes = [i32, i32, i32, vp, vp, vp, f32, f32, vp]
    L.ref_sgemm_rowmajor.argtypes = [i32, vp, vp, vp, f32, f32]
    L.ref_sgemm_colmajor_nt.argtypes = [i32, i32, i32, vp, vp, vp, f32, f32]
    L.b2_ft_sgemm.argtypes = [vp, i32, i32, i32, i32, f32, vp, i32, vp, i32, f32, vp, i32, vp, i32, f32, vp, vp]
    L.b2_ft_sgemm_colmajor_nt.argtypes = [vp, i32, i32, i32, f32, vp, vp, f32, vp, vp, i32, f32, vp, vp]
    L.ref_ft_sgemm_colmajor_nt.argtypes = [i32, i32, i32, vp, vp, vp, f32, f32]
    L.saxpy.argtypes = [i32, f32, vp, vp]
    L.b2_saxpy.argtypes = [vp, i64, f32, vp, vp, vp]
    L.sdot.argtypes = [i32, vp, vp, vp]
    L.b2_sdot.argtypes = [vp, i64, vp, vp, vp, vp]
    L.b2_sdot_partial.argtypes = [vp, i64, vp, vp, vp, vp, vp]
    L.b2_sdot_static.argtypes = [i64, vp, vp, vp, vp]
    L.b2_fill_uniform.argtypes = [vp, i64, u64, vp]
    L.b2_fill_uniform_host.argtypes = [vp, i64, u64]
    L.b2_fill_const.argtypes = [vp, i64, f32, vp]
    L.b2_sdot_fused.argtypes = [vp, i64, vp, vp, vp, vp, C.POINTER(vp), i32, i32, u64, vp]
    L.b2_copy_matrix_async.argtypes = [vp, i64, vp, i64, i64, i64, i32, vp]
    L.b2_verify_matrix.argtypes = [vp, vp, i64, i64, i64, f32, C.POINTER(f32), vp]
    L.b2_timer_create.argtypes = [C.POINTER(vp)]
    L.b2_timer_destroy.argtypes = [vp]
    L.b2_timer_start.argtypes = [vp, vp]
    L.b2_timer_stop.argtypes = [vp, vp]
    L.b2_timer_elapsed_ms.argtypes = [vp, C.POINTER(f32)]
    L.b2_ffma_peak_probe.argtypes = [i32, i64, C.POINTER(C.c_double), vp]
    L.b2_ffma2_peak_probe.argtypes = [i32, i64, C.POINTER(C.c_double), vp]
    L.b2_device_info.argtypes = [C.POINTER(i32), C.POINTER(i32), C.POINTER(C.c_size_t)]
    L.b2_check_status.argtypes = [vp, vp]
    L.b2_selftest_wait_timeout.argtypes = [vp, i32, vp]
    L.b2_set_ffma_variant.argtypes = [i32]
    L.b2_ffma_tile_info.argtypes = [i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(C.c_char_p)]
    L.b2_set_ffma_tile.argtypes = [i32]
    L.b2_set_ffma_split_k.argtypes = [i32]
    L.b2_set_tf32_tile_n.argtypes = [i32]
    L.b2_set_tf32_slab_k.argtypes = [i32]
    L.b2_set_tf32_pair.argtypes = [i32]
    L.b2_set_tf32_persistent.argtypes = [i32]
    L.b2_set_tf32_chunk.argtypes = [i32]
    L.b2_ffma_pick_tile.argtypes = [i32, i32, i32]
    L.b2_set_ffma_row_split.argtypes = [i32]
    L.b2_ffma_row_split_plan.argtypes = [i32, i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    L.b2_set_tf32_fused_split.argtypes = [i32]
    L.b2_set_tf32_tail_split.argtypes = [i32]
    L.b2_tf32_tail_plan.argtypes = [i32, i32, i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    L.b2_set_ft_level.argtypes = [i32]
    L.b2_set_ffma_transpose_a.argtypes = [i32]
    L.b2_set_tf32_abft_bias.argtypes = [f32]
    L.b2_host_plan_create.argtypes = [C.POINTER(vp), vp, i32, i32, i32, i32, i32, i32, i32, i32]
    L.b2_host_plan_destroy.argtypes = [vp]
    L.b2_sgemm_host.argtypes = [vp, f32, vp, i32, vp, i32, f32, vp, i32, i32, vp]
    L.b2_host_alloc.argtypes = [C.POINTER(vp), C.c_size_t]
    L.b2_host_free.argtypes = [vp]
    L.b2_mg_unique_id.argtypes = [vp]
    L.b2_mg_create.argtypes = [C.POINTER(vp), vp, i32, i32, vp]
    L.b2_mg_destroy.argtypes = [vp]
    L.b2_mg_row_block.argtypes = [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]
    L.b2_mg_k_panel.argtypes = [i32, i32, i32, C.POINTER(i32), C.POINTER(i32)]
    L.b2_mg_sgemm.argtypes = [vp, i32, i32, i32, i32, i32, f32, vp, i32, vp, i32, f32, vp, i32, i32, i32, vp, vp]
    L.b2_mg_sdot.argtypes = [vp, i64, vp, vp, vp, vp, vp]
    _lib = L
    return L


def check(status: int) -> int:
    if status < 0:
        L = load()
        msg = L.b2_last_error().decode() or L.b2_status_string(status).decode()
        raise B2Error(status, msg)
    return status

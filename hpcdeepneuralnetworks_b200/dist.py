"""Multi-GPU forms of the path: one process per GPU, ``torch.distributed`` for the plumbing.

* Sharded SGEMM (and ABFT-SGEMM): A and C are split by contiguous row blocks, one block per
  rank; B lives on ``src`` and is broadcast ONCE per GEMM in K-panels (contiguous row blocks of
  the row-major B) on a communication stream, while the compute stream consumes the panels that
  have already landed:  C_r = beta*C_r + alpha * sum_p A_r[:, panel p] * B[panel p, :].
  There is no result exchange -- C stays sharded -- so the only collective is the broadcast.
* Sharded SDOT: each rank reduces its slice to a double partial on the device, then one
  all-reduce(sum) of that scalar.

The reference is single-GPU (no NCCL/MPI call anywhere in it); this file has no counterpart
there.  On CUDA tensors both forms are one call into the library (``b2_mg_sgemm``, ``b2_mg_sdot``:
schedule, streams, events and NCCL calls live in C++ behind the C ABI); this module adds the
collective construction of the library's communicator over ``torch.distributed``.  ``gemm_fn`` /
``dot_fn`` exist so that the same partition (``b2_mg_row_block``, ``b2_mg_k_panel``) and panel
schedule can be exercised by CPU ranks over gloo in the tests.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def row_block(M: int, rank: int, world: int) -> Tuple[int, int]:
    """(first row, row count) of rank's block: contiguous, sizes differ by at most one row (``b2_mg_row_block``)."""
    import ctypes as C
    from . import _lib
    start, rows = C.c_int64(), C.c_int64()
    _lib.check(_lib.load().b2_mg_row_block(M, rank, world, C.byref(start), C.byref(rows)))
    return start.value, rows.value


def k_panels(K: int, panel: int) -> List[Tuple[int, int]]:
    """[(k0, width)] covering [0, K) in order; widths are `panel` except possibly the last (``b2_mg_k_panel``)."""
    import ctypes as C
    from . import _lib
    L = _lib.load()
    if K <= 0:
        return []
    out, k0, kw = [], C.c_int(), C.c_int()
    count = _lib.check(L.b2_mg_k_panel(K, panel, 0, C.byref(k0), C.byref(kw)))
    for i in range(count):
        L.b2_mg_k_panel(K, panel, i, C.byref(k0), C.byref(kw))
        out.append((k0.value, kw.value))
    return out


class MgHandle:
    """``b2_mg_handle``: this rank's membership of the library's own NCCL communicator.  Construction is collective:
    rank 0 draws the communicator id (``b2_mg_unique_id``) and ``torch.distributed`` carries it to the other ranks;
    with a world of one no communicator is made."""

    def __init__(self, group=None, handle=None):
        import ctypes as C
        from . import _lib, blas
        self._L = _lib.load()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._handle = handle or blas.default_handle()
        ident = None
        if self.world > 1:
            buf = (C.c_char * 128)()
            if self.rank == 0:
                _lib.check(self._L.b2_mg_unique_id(buf))
            box = [bytes(buf)]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            ident = C.create_string_buffer(box[0], 128)
        self._mg = C.c_void_p()
        _lib.check(self._L.b2_mg_create(C.byref(self._mg), self._handle.raw, self.rank, self.world, ident))

    @property
    def raw(self):
        return self._mg

    def close(self):
        if self._mg:
            torch.cuda.synchronize()
            self._L.b2_mg_destroy(self._mg)
            self._mg = type(self._mg)()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_mg_default = {}


def default_mg(group=None) -> MgHandle:
    """One ``MgHandle`` per process group and device, made on first use (collectively)."""
    key = (id(group), torch.cuda.current_device())
    if key not in _mg_default:
        _mg_default[key] = MgHandle(group)
    return _mg_default[key]


def _cuda_gemm(path: int, abft: bool, report):
    from . import blas

    def fn(M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc):
        if abft:
            blas.ft_sgemm(M, N, K, alpha, A, B, beta, Cm, path=path, lda=lda, ldb=ldb, ldc=ldc, report=report)
        else:
            blas.sgemm(M, N, K, alpha, A, B, beta, Cm, path=path, lda=lda, ldb=ldb, ldc=ldc)
    return fn


def sharded_sgemm(M: int, N: int, K: int, alpha: float, A_local: torch.Tensor, B: torch.Tensor, beta: float,
                  C_local: torch.Tensor, *, src: int = 0, panel: int = 4096, path: int = 0, abft: bool = False,
                  report=None, group=None, gemm_fn: Callable | None = None, mg: MgHandle | None = None) -> torch.Tensor:
    """Row-block-sharded row-major SGEMM.

    ``A_local`` (rows_r x K) and ``C_local`` (rows_r x N) are this rank's blocks (``row_block``);
    ``B`` is a K x N buffer on every rank whose contents are only valid on ``src`` at entry and on
    every rank at exit.  On CUDA tensors the whole schedule runs inside ``b2_mg_sgemm`` (the library's own NCCL
    communicator, ``mg`` or the default one of the group).  Returns ``C_local``.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    _, rows = row_block(M, rank, world)
    assert A_local.shape == (rows, K) and C_local.shape == (rows, N) and B.shape == (K, N)
    on_gpu = B.is_cuda
    fn = gemm_fn or _cuda_gemm(path, abft, report)
    panels = k_panels(K, panel)
    if not panels:
        if rows:
            fn(rows, N, 0, alpha, A_local, max(K, 1), B, N, beta, C_local, N)
        return C_local

    if not on_gpu or gemm_fn is not None:
        # CPU ranks (tests): the same schedule, ranks and panels as b2_mg_sgemm, arithmetic injected.
        for i, (k0, kw) in enumerate(panels):
            if world > 1:
                dist.broadcast(B[k0:k0 + kw], src=src, group=group)
            if rows:
                fn(rows, N, kw, alpha, A_local[:, k0:], K, B[k0:], N, beta if i == 0 else 1.0, C_local, N)
        return C_local

    import ctypes as C
    from . import _lib, blas
    mg = mg or default_mg(group)
    need = int(_lib.load().b2_ft_sgemm_workspace_bytes(path, rows, N, min(panel, K))) if rows else 0
    blas.default_handle().reserve(need)
    vp = lambda t: C.c_void_p(t.data_ptr())
    _lib.check(_lib.load().b2_mg_sgemm(mg.raw, path, 1 if abft else 0, M, N, K, alpha, vp(A_local), K, vp(B), N, beta, vp(C_local), N,
                                       src, panel, vp(report) if report is not None else None,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return C_local


def sharded_sdot(n_local: int, x_local: torch.Tensor, y_local: torch.Tensor, *, group=None,
                 dot_fn: Callable | None = None, mg: MgHandle | None = None) -> torch.Tensor:
    """Sum over ranks of x_local . y_local.  Returns a 1-element float64 tensor (same on every rank).  On CUDA tensors
    this is ``b2_mg_sdot``: the SDOT kernel's double partial, then one all-reduce of that scalar."""
    if dot_fn is None:
        import ctypes as C
        from . import _lib
        mg = mg or default_mg(group)
        part = torch.zeros(1, dtype=torch.float64, device=x_local.device)
        _lib.check(_lib.load().b2_mg_sdot(mg.raw, n_local, C.c_void_p(x_local.data_ptr()), C.c_void_p(y_local.data_ptr()), None,
                                          C.c_void_p(part.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return part
    part = dot_fn(n_local, x_local, y_local)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group)
    return part


class FusedSdot:
    """Sharded SDOT whose cross-GPU sum happens inside the kernel: the last block of every rank's SDOT kernel stores its
    partial into all ranks' mailboxes (peer stores over NVLink) and adds the others' in rank order after a bounded
    wait -- no collective call.  The mailboxes live in torch's symmetric memory (one 512-byte buffer per rank mapped
    into every process); construction is collective and raises if symmetric memory cannot be set up, in which case
    ``sharded_sdot`` (NCCL all-reduce of the double partials) is the way."""

    def __init__(self, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 16:
            raise RuntimeError("FusedSdot supports at most 16 ranks")
        self.buf = symm.empty(64, dtype=torch.float64, device=device)      # 512 bytes
        self.buf.zero_()
        try:
            self.hdl = symm.rendezvous(self.buf, self.group)
        except TypeError:
            self.hdl = symm.rendezvous(self.buf, self.group.group_name)
        self.mailboxes = [int(p) for p in self.hdl.buffer_ptrs]
        if len(self.mailboxes) != self.world or any(p % 256 for p in self.mailboxes):
            raise RuntimeError("symmetric memory gave unusable mailbox addresses")
        torch.cuda.synchronize(device)
        dist.barrier(self.group)        # every mailbox is zeroed before anyone's first call
        self.seq = 0
        self.out = torch.empty(1, dtype=torch.float32, device=device)
        self.sum64 = torch.empty(1, dtype=torch.float64, device=device)

    def __call__(self, n_local: int, x_local: torch.Tensor, y_local: torch.Tensor) -> torch.Tensor:
        """Sum over ranks of x_local . y_local as a 1-element float64 device tensor (same bits on every rank)."""
        from . import blas
        self.seq += 1
        blas.sdot_fused(n_local, x_local, y_local, self.mailboxes, self.rank, self.world, self.seq, out=self.out,
                        sum64=self.sum64)
        return self.sum64

"""Multi-GPU forms of the path: one process per GPU, ``torch.distributed`` for the plumbing.

* Sharded SGEMM (and ABFT-SGEMM): A and C are split by contiguous row blocks, one block per
  rank; B lives on ``src`` and is broadcast ONCE per GEMM in K-panels (contiguous row blocks of
  the row-major B) on a communication stream, while the compute stream consumes the panels that
  have already landed:  C_r = beta*C_r + alpha * sum_p A_r[:, panel p] * B[panel p, :].
  There is no result exchange -- C stays sharded -- so the only collective is the broadcast.
* Sharded SDOT: each rank reduces its slice to a double partial on the device, then one
  all-reduce(sum) of that scalar.

The reference is single-GPU (no NCCL/MPI call anywhere in it); this file has no counterpart
there.  The arithmetic is always the CUDA library's; ``gemm_fn``/``dot_fn`` exist so that the
host-side orchestration (partitioning, panel schedule, collectives) can be exercised by CPU
ranks over gloo in the tests.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def row_block(M: int, rank: int, world: int) -> Tuple[int, int]:
    """(first row, row count) of rank's block: contiguous, sizes differ by at most one row."""
    base, rem = divmod(M, world)
    rows = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, rows


def k_panels(K: int, panel: int) -> List[Tuple[int, int]]:
    """[(k0, width)] covering [0, K) in order; widths are `panel` except possibly the last."""
    if K <= 0:
        return []
    panel = max(1, panel)
    return [(k0, min(panel, K - k0)) for k0 in range(0, K, panel)]


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
                  report=None, group=None, gemm_fn: Callable | None = None, comm_stream=None) -> torch.Tensor:
    """Row-block-sharded row-major SGEMM.

    ``A_local`` (rows_r x K) and ``C_local`` (rows_r x N) are this rank's blocks (``row_block``);
    ``B`` is a K x N buffer on every rank whose contents are only valid on ``src`` at entry and on
    every rank at exit.  Returns ``C_local``.
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

    if world == 1 or not on_gpu:
        # CPU ranks (tests) and the single-GPU case: same schedule, no stream overlap.
        for i, (k0, kw) in enumerate(panels):
            if world > 1:
                dist.broadcast(B[k0:k0 + kw], src=src, group=group)
            if rows:
                fn(rows, N, kw, alpha, A_local[:, k0:], K, B[k0:], N, beta if i == 0 else 1.0, C_local, N)
        return C_local

    compute = torch.cuda.current_stream()
    comm = comm_stream or torch.cuda.Stream()
    comm.wait_stream(compute)            # B may still be being written by earlier work
    works = []
    with torch.cuda.stream(comm):
        for (k0, kw) in panels:
            works.append(dist.broadcast(B[k0:k0 + kw], src=src, group=group, async_op=True))
    for i, (k0, kw) in enumerate(panels):
        works[i].wait()                  # the compute stream waits for panel i only
        if rows:
            fn(rows, N, kw, alpha, A_local[:, k0:], K, B[k0:], N, beta if i == 0 else 1.0, C_local, N)
    return C_local


def sharded_sdot(n_local: int, x_local: torch.Tensor, y_local: torch.Tensor, *, group=None,
                 dot_fn: Callable | None = None) -> torch.Tensor:
    """Sum over ranks of x_local . y_local.  Returns a 1-element float64 tensor (same on every rank)."""
    if dot_fn is None:
        from . import blas
        out = torch.empty(1, dtype=torch.float32, device=x_local.device)
        part = torch.zeros(1, dtype=torch.float64, device=x_local.device)
        blas.sdot_partial(n_local, x_local, y_local, out, part)
    else:
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

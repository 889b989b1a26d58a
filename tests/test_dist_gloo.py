"""CPU tests of the multi-GPU orchestration: row-block partition, K-panel schedule, the per-panel broadcast and
the scalar all-reduce, run as world_size-2 (and 3) gloo ranks.  The arithmetic of each rank is injected from the
oracle here -- the product path always uses the CUDA library."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from hpcdeepneuralnetworks_b200 import dist as b2dist


def test_row_block_partition():
    for M in (1, 7, 128, 1000, 32768):
        for world in (1, 2, 3, 4, 8):
            blocks = [b2dist.row_block(M, r, world) for r in range(world)]
            assert blocks[0][0] == 0
            assert sum(b[1] for b in blocks) == M
            for (s0, n0), (s1, n1) in zip(blocks, blocks[1:]):
                assert s1 == s0 + n0 and 0 <= n0 - n1 <= 1
    assert b2dist.row_block(32768, 3, 8) == (12288, 4096)


def test_k_panels():
    assert b2dist.k_panels(0, 4096) == []
    assert b2dist.k_panels(10, 4) == [(0, 4), (4, 4), (8, 2)]
    assert b2dist.k_panels(32768, 4096) == [(k, 4096) for k in range(0, 32768, 4096)]
    assert b2dist.k_panels(5, 0) == [(k, 1) for k in range(5)]


def _oracle_gemm(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc):
    a = A.numpy()[:M, :K]
    b = B.numpy()[:K, :N]
    C.copy_(torch.from_numpy(oracle.sgemm_fma(alpha, np.ascontiguousarray(a), np.ascontiguousarray(b), beta, C.numpy())))


def _oracle_dot(n, x, y):
    s, _ = oracle.sdot(x.numpy()[:n], y.numpy()[:n], nthreads=1)
    return torch.tensor([s], dtype=torch.float64)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, panel, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a = oracle.fill_uniform(M * K, 1).reshape(M, K)
        b = oracle.fill_uniform(K * N, 2).reshape(K, N)
        c = oracle.fill_uniform(M * N, 3).reshape(M, N)
        start, rows = b2dist.row_block(M, rank, world)
        A_loc = torch.from_numpy(a[start:start + rows].copy())
        C_loc = torch.from_numpy(c[start:start + rows].copy())
        B = torch.from_numpy(b.copy()) if rank == 0 else torch.full((K, N), float("nan"))   # only the source holds B
        b2dist.sharded_sgemm(M, N, K, 1.0, A_loc, B, 0.5, C_loc, src=0, panel=panel, gemm_fn=_oracle_gemm)
        assert np.array_equal(B.numpy(), b)                      # every rank now holds B
        # expected: the panelled accumulation of the same oracle (beta on the first panel, 1 afterwards)
        want = c[start:start + rows].copy()
        for i, (k0, kw) in enumerate(b2dist.k_panels(K, panel)):
            want = oracle.sgemm_fma(1.0, np.ascontiguousarray(a[start:start + rows, k0:k0 + kw]),
                                    np.ascontiguousarray(b[k0:k0 + kw]), 0.5 if i == 0 else 1.0, want)
        assert np.array_equal(C_loc.numpy(), want)
        c64, den = oracle.sgemm_f64(1.0, a[start:start + rows], b, 0.5, c[start:start + rows])
        assert rows == 0 or oracle.gemm_error(C_loc.numpy(), c64, den) <= 1e-5
        # sharded dot: slices of one vector pair
        n = 100003
        x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
        s0, cnt = b2dist.row_block(n, rank, world)
        tot = b2dist.sharded_sdot(cnt, torch.from_numpy(x[s0:s0 + cnt].copy()), torch.from_numpy(y[s0:s0 + cnt].copy()),
                                  dot_fn=_oracle_dot)
        full, scale = oracle.sdot(x, y, nthreads=1)
        assert abs(float(tot.item()) - full) <= 1e-12 * scale
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape,panel", [(2, (96, 80, 64), 16), (2, (33, 17, 50), 64), (3, (10, 24, 40), 7)])
def test_sharded_paths_over_gloo(tmp_path, world, shape, panel):
    M, N, K = shape
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, panel, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]


def test_single_process_schedule_matches_one_call():
    """world = 1: the panel loop alone; one panel reproduces a single call bit for bit."""
    M, N, K = 40, 24, 64
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    C1 = torch.from_numpy(c.copy())
    b2dist.sharded_sgemm(M, N, K, 1.0, torch.from_numpy(a.copy()), torch.from_numpy(b.copy()), 0.5, C1, panel=K,
                         gemm_fn=_oracle_gemm)
    assert np.array_equal(C1.numpy(), oracle.sgemm_fma(1.0, a, b, 0.5, c))

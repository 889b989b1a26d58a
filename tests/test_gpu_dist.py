"""GPU tests of the sharded forms: the panel schedule on one GPU (world = 1) and, where two GPUs are
visible, two NCCL ranks launched the way the benchmark is launched."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_panelled_sgemm_single_gpu(cuda):
    from hpcdeepneuralnetworks_b200 import dist as b2dist
    import hpcdeepneuralnetworks_b200 as b2
    M, N, K, panel = 300, 260, 512, 128
    a = oracle.fill_uniform(M * K, 1).reshape(M, K)
    b = oracle.fill_uniform(K * N, 2).reshape(K, N)
    c = oracle.fill_uniform(M * N, 3).reshape(M, N)
    for path, tol in ((0, 1e-5), (1, 2e-5)):
        C1 = torch.from_numpy(c.copy()).cuda()
        b2dist.sharded_sgemm(M, N, K, 1.0, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), 0.5, C1, panel=panel, path=path)
        b2.check_status()
        got = C1.cpu().numpy()
        c64, den = oracle.sgemm_f64(1.0, a, b, 0.5, c)
        assert oracle.gemm_error(got, c64, den) <= tol
        if path == 0:   # bit-exact against the same panel schedule on the CPU
            want = c.copy()
            for i, (k0, kw) in enumerate(b2dist.k_panels(K, panel)):
                want = oracle.sgemm_fma(1.0, np.ascontiguousarray(a[:, k0:k0 + kw]), np.ascontiguousarray(b[k0:k0 + kw]),
                                        0.5 if i == 0 else 1.0, want)
            assert np.array_equal(got, want)


def test_sharded_sdot_single_gpu(cuda):
    from hpcdeepneuralnetworks_b200 import dist as b2dist
    n = (1 << 20) + 9
    x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
    tot = b2dist.sharded_sdot(n, torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda())
    want, scale = oracle.sdot(x, y)
    assert abs(float(tot.item()) - want) <= 1e-6 * scale


def test_fused_sdot_exchange_with_itself(cuda):
    """World of one: the kernel's exchange runs against its own mailbox (flag, bounded wait, slot sum) and must give
    b2_sdot's bits, call after call (the two epochs of the mailbox alternate)."""
    import hpcdeepneuralnetworks_b200 as b2
    n = (1 << 20) + 5
    x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    box = torch.zeros(64 + 32, dtype=torch.float64, device="cuda")
    addr = (box.data_ptr() + 255) & ~255
    want = b2.sdot(n, dx, dy).item()
    for seq in range(1, 6):
        out, s64 = b2.sdot_fused(n, dx, dy, [addr], 0, 1, seq)
        b2.check_status()
        assert out.item() == want
    ref, scale = oracle.sdot(x, y)
    assert abs(float(s64.item()) - ref) <= 1e-6 * scale


def test_fused_sdot_missing_peer_times_out(cuda):
    """A peer that never writes its flag: the bounded wait gives up after a second, the status word says TIMEOUT, the
    local sum is returned and the context stays usable (the second mailbox is plain local memory nobody writes)."""
    import hpcdeepneuralnetworks_b200 as b2
    n = 1 << 16
    x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    box = torch.zeros(2 * 64 + 32, dtype=torch.float64, device="cuda")
    a0 = (box.data_ptr() + 255) & ~255
    out, _ = b2.sdot_fused(n, dx, dy, [a0, a0 + 512], 0, 2, 1)
    with pytest.raises(b2.B2Error) as e:
        b2.check_status()
    assert e.value.status == -4
    assert out.item() == b2.sdot(n, dx, dy).item()
    b2.check_status()


_RANK_SCRIPT = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["B2_ROOT"])
import oracle
import hpcdeepneuralnetworks_b200 as b2
from hpcdeepneuralnetworks_b200 import dist as b2dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
M, N, K, panel = 520, 384, 768, 256
a = oracle.fill_uniform(M * K, 1).reshape(M, K); b = oracle.fill_uniform(K * N, 2).reshape(K, N); c = oracle.fill_uniform(M * N, 3).reshape(M, N)
s, rows = b2dist.row_block(M, rank, world)
A = torch.from_numpy(a[s:s + rows].copy()).cuda(); C = torch.from_numpy(c[s:s + rows].copy()).cuda()
B = torch.from_numpy(b.copy()).cuda() if rank == 0 else torch.full((K, N), float("nan"), device="cuda")
b2dist.sharded_sgemm(M, N, K, 1.0, A, B, 0.5, C, src=0, panel=panel, path=0)
b2.check_status()
want = c[s:s + rows].copy()
for i, (k0, kw) in enumerate(b2dist.k_panels(K, panel)):
    want = oracle.sgemm_fma(1.0, np.ascontiguousarray(a[s:s + rows, k0:k0 + kw]), np.ascontiguousarray(b[k0:k0 + kw]), 0.5 if i == 0 else 1.0, want)
assert np.array_equal(C.cpu().numpy(), want), "sharded SGEMM differs from the oracle"
assert np.array_equal(B.cpu().numpy(), b), "B was not broadcast"
n = 1 << 20
x, y = oracle.fill_uniform(n, 4), oracle.fill_uniform(n, 5)
s0, cnt = b2dist.row_block(n, rank, world)
tot = b2dist.sharded_sdot(cnt, torch.from_numpy(x[s0:s0 + cnt].copy()).cuda(), torch.from_numpy(y[s0:s0 + cnt].copy()).cuda())
ref, scale = oracle.sdot(x, y)
assert abs(float(tot.item()) - ref) <= 1e-6 * scale
# the same sum formed inside the kernels over peer memory (no collective): same bits on both ranks, several calls
fused = b2dist.FusedSdot(torch.device("cuda", int(os.environ["LOCAL_RANK"])))
xs, ys = torch.from_numpy(x[s0:s0 + cnt].copy()).cuda(), torch.from_numpy(y[s0:s0 + cnt].copy()).cuda()
vals = []
for it in range(5):
    vals.append(float(fused(cnt, xs, ys).item()))
b2.check_status()
assert all(v == vals[0] for v in vals), vals
assert abs(vals[0] - ref) <= 1e-6 * scale
both = torch.tensor([vals[0]], dtype=torch.float64, device="cuda")
gathered = [torch.empty_like(both) for _ in range(world)]
dist.all_gather(gathered, both)
assert all(float(g.item()) == vals[0] for g in gathered), "ranks disagree on the fused sum"
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_ranks_nccl(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, B2_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29533", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout

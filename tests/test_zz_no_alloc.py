"""GPU test of the allocation-free SDOT entry point (``b2_sdot_static``).

Some callers of this library cannot allocate device memory when they need a dot product -- a plugin inside a
framework that owns all device memory, a latency-critical callback that must not hit cudaMalloc's implicit
synchronisation, a process with a fixed memory budget.  For them the library keeps the SDOT scratch in a static
device array.  This test calls that entry point through the C ABI, twice in a row on the same scratch, and checks
it against the regular entry point (``b2_sdot``), within the SDOT tolerance used elsewhere in the suite
(1e-5 relative to sum |x_i*y_i|).  It lives in a file that pytest collects last, and it must pass both alone in a
fresh process and after every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _call_static(L, n, x, y, out):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return L.b2_sdot_static(n, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(out.data_ptr()), stream)


def test_static_sdot_matches_regular_entry_point_twice(cuda):
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    n = (1 << 22) + 5
    x = oracle.fill_uniform(n, 4)
    y = oracle.fill_uniform(n, 5)
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    _, scale = oracle.sdot(x, y)
    want = float(b2.sdot(n, dx, dy).item())                    # the existing entry point
    out = torch.full((1,), -7.0, device="cuda")                 # allocated before the calls under test
    for attempt in range(2):                                    # second call re-uses the scratch the first one left
        out.fill_(-7.0)
        assert _call_static(L, n, dx, dy, out) == 0
        got = float(out.item())
        assert abs(got - want) <= TOL * scale, (attempt, got, want)
    # a different problem on the same scratch right afterwards
    m = 100003
    assert _call_static(L, m, dx[3:], dy[1:], out) == 0
    want_m, scale_m = oracle.sdot(x[3:3 + m], y[1:1 + m])
    assert abs(float(out.item()) - want_m) <= TOL * scale_m
    # empty input gives exactly zero
    assert _call_static(L, 0, dx, dy, out) == 0
    assert float(out.item()) == 0.0


def test_static_sdot_rejects_sizes_beyond_its_limit(cuda):
    from hpcdeepneuralnetworks_b200 import _lib
    L = _lib.load()
    t = torch.zeros(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert _call_static(L, (1 << 30) + 1, t, t, out) == -2      # B2_ERR_UNSUPPORTED, nothing launched
    assert b"exceeds the limit" in L.b2_last_error()
    assert _call_static(L, -1, t, t, out) == -1


_FRESH = r"""
import ctypes as C, os, sys
sys.path.insert(0, os.environ["B2_ROOT"])
import torch
from hpcdeepneuralnetworks_b200 import _lib
L = _lib.load()
torch.cuda.set_device(0)
n = (1 << 20) + 3
x = torch.rand(n, device="cuda") - 0.5
y = torch.rand(n, device="cuda") - 0.5
out = torch.zeros(1, device="cuda")
torch.cuda.synchronize()
def call():
    st = L.b2_sdot_static(n, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(out.data_ptr()), None)
    assert st == 0, st
    torch.cuda.synchronize()
call()                                   # first call on the device: looks up the scratch symbol's address
free0, _ = torch.cuda.mem_get_info()
for _ in range(50):
    call()
free1, _ = torch.cuda.mem_get_info()
want = float((x.double() * y.double()).sum().item())
scale = float((x.double() * y.double()).abs().sum().item())
assert abs(float(out.item()) - want) <= 1e-5 * scale
assert free1 == free0, (free0, free1)
print("free bytes unchanged over 50 calls:", free0)
"""


def test_static_sdot_allocates_nothing_in_a_fresh_process(cuda, tmp_path):
    """The point of the entry point: in a process that never creates a library handle, the free device memory the
    driver reports does not move across fifty calls (any cudaMalloc inside would show, whole pages at a time)."""
    import os
    import subprocess
    import sys
    script = tmp_path / "fresh.py"
    script.write_text(_FRESH)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, str(script)], env=dict(os.environ, B2_ROOT=root), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "free bytes unchanged" in r.stdout

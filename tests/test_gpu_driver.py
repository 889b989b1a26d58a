"""GPU test of the C++ command-line driver (reference-shaped main() over the C ABI): every sub-command verifies
its own results and must exit 0."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("argv", [["sgemm", "14", "256", "768"], ["sgemm", "13", "256", "512"], ["sgemm", "2", "256", "256", "16"],
                                  ["ft_sgemm", "512", "1024", "512"], ["saxpy"], ["sdot"],
                                  ["small"], ["tiles", "1024"], ["sgemm_host", "1536"], ["sgemm_host", "1024", "1"], ["mg", "0", "1", "unused", "1024", "256"]])
def test_driver_subcommands(cuda, built_lib, argv):
    from hpcdeepneuralnetworks_b200 import build
    exe = build.build_driver()
    r = subprocess.run([exe] + argv, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert ("GFLOPS" in r.stdout) or ("GB/s" in r.stdout) or ("tflops" in r.stdout)


def test_driver_reports_unsupported_size(cuda, built_lib):
    from hpcdeepneuralnetworks_b200 import build
    exe = build.build_driver()
    r = subprocess.run([exe, "sgemm", "9", "200", "200"], capture_output=True, text=True, timeout=120)   # 200 % 128 != 0
    assert r.returncode == 3 and "multiple of 128" in r.stderr


def test_driver_two_processes_two_gpus(cuda, built_lib, tmp_path):
    """The multi-GPU entry points from plain C++: two driver processes, one per GPU, that find each other through the
    communicator id rank 0 writes to a file; each checks its block of the sharded SGEMM bit for bit and the SDOT sum."""
    import os
    import torch
    from hpcdeepneuralnetworks_b200 import build
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = build.build_driver()
    idf = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([exe, "mg", str(r), "2", idf, "2048", "512"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("bit-identical" in o for o in outs)

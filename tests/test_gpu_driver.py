"""GPU test of the C++ command-line driver (reference-shaped main() over the C ABI): every sub-command verifies
its own results and must exit 0."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("argv", [["sgemm", "14", "256", "768"], ["sgemm", "13", "256", "512"], ["sgemm", "2", "256", "256", "16"],
                                  ["ft_sgemm", "512", "1024", "512"], ["saxpy"], ["sdot"]])
def test_driver_subcommands(cuda, built_lib, argv):
    from hpcdeepneuralnetworks_b200 import build
    exe = build.build_driver()
    r = subprocess.run([exe] + argv, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert ("GFLOPS" in r.stdout) or ("GB/s" in r.stdout)


def test_driver_reports_unsupported_size(cuda, built_lib):
    from hpcdeepneuralnetworks_b200 import build
    exe = build.build_driver()
    r = subprocess.run([exe, "sgemm", "9", "200", "200"], capture_output=True, text=True, timeout=120)   # 200 % 128 != 0
    assert r.returncode == 3 and "multiple of 128" in r.stderr

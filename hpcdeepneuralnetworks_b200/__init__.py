"""B200-native (sm_100a) FP32 BLAS-kernel library: row-major SGEMM (FFMA and 3xTF32 paths),
ABFT fault-tolerant SGEMM, SAXPY and SDOT behind the reference project's launcher signatures.

The arithmetic lives in ``libb2blas.so`` (hand-written CUDA, C ABI in ``include/b2blas.h``);
this package is the host-side mirror of the reference interface and uses PyTorch only for
device memory, streams and ``torch.distributed``.
"""
from ._lib import B2Error, Fault, FtReport, LIB_PATH  # noqa: F401


def __getattr__(name):
    # Operators are resolved lazily so that importing the package (and building the library)
    # works on a machine without a GPU; using an operator without the built library raises.
    import importlib
    if name in ("blas", "build", "dist", "gen_ft_sgemm", "_lib"):
        return importlib.import_module(f"{__name__}.{name}")
    blas = importlib.import_module(f"{__name__}.blas")
    if hasattr(blas, name):
        return getattr(blas, name)
    raise AttributeError(name)

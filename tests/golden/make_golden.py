"""Generates tests/golden/golden.json.

Run in the build container, where the reference tree is mounted:  python tests/golden/make_golden.py
GEMM entries come from the REFERENCE's own cpu_gemm (utils/utils.cu:93-103) compiled by
oracle/Makefile into oracle/_ref/libref_utils.so; the reference has no CPU SAXPY/SDOT/ABFT code,
so those entries come from the restated loops in oracle/oracle.c and pin them against change.
Inputs are the seeded uniform[-1,1) streams (seed 1 = A, 2 = B, 3 = C, 4 = x, 5 = y).
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
import oracle  # noqa: E402


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    out = {"generator": "tests/golden/make_golden.py", "rng": {}, "cpu_gemm": [], "saxpy": [], "sdot": [], "fault": []}
    for seed in (1, 2, 5):
        v = oracle.fill_uniform(8, seed)
        out["rng"][str(seed)] = [float(x) for x in v]
    out["rng_sha_seed1_1M"] = digest(oracle.fill_uniform(1 << 20, 1))
    if oracle.ref_lib() is None:
        raise SystemExit("oracle/_ref is not built (reference tree missing): cannot pin cpu_gemm")
    for n, alpha, beta in ((8, 1.0, 0.0), (64, 1.0, 0.5), (256, 1.0, 0.0), (256, -1.5, 0.5)):
        a = oracle.fill_uniform(n * n, 1).reshape(n, n)
        b = oracle.fill_uniform(n * n, 2).reshape(n, n)
        c = np.zeros((n, n), np.float32) if beta == 0.0 else oracle.fill_uniform(n * n, 3).reshape(n, n)
        ref = oracle.ref_cpu_gemm(alpha, beta, a, b, c)
        entry = {"n": n, "alpha": alpha, "beta": beta, "sha256": digest(ref),
                 "first_row": [float(x) for x in ref[0, :8]], "source": "reference cpu_gemm (oracle/_ref)"}
        if n == 8:
            entry["full"] = [float(x) for x in ref.ravel()]
        out["cpu_gemm"].append(entry)
    for n in (1, 7, 1024, (1 << 20) + 3):
        x = oracle.fill_uniform(n, 4)
        y = oracle.fill_uniform(n, 5)
        out["saxpy"].append({"n": n, "alpha": 2.0, "sha256": digest(oracle.saxpy(2.0, x, y))})
        s, sa = oracle.sdot(x, y, nthreads=1)
        out["sdot"].append({"n": n, "dot": s, "abs": sa})
    n = 256
    a = oracle.fill_uniform(n * n, 1).reshape(n, n)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    for f in ((0, 0, 3, 5, 2, 20), (1, 1, 127, 0, 7, 30), (0, 1, 64, 64, 0, 25)):
        clean, bad, ok = oracle.fault_effect(a, b, f)
        out["fault"].append({"fault": list(f), "clean": clean, "faulty": repr(bad), "in_range": ok})
    with open(os.path.join(HERE, "golden.json"), "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote golden.json")


if __name__ == "__main__":
    main()

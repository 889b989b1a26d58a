#!/usr/bin/env python
"""Benchmark of the FP32 BLAS hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--path ffma|3xtf32]

One JSON line on stdout (rank 0).  A "step" is one SGEMM of the workload:
  N = 1  : row-major SGEMM M=N=K=6144, alpha=1, beta=0.5 (the largest point of benchmark configuration 2, the
           size the metric "SGEMM TFLOPS @6144^3 fp32" is quoted on); inputs resident in HBM.
  N > 1  : SGEMM M=N=K=32768, alpha=1, beta=0 (benchmark configuration 5), A and C split by row blocks over
           the ranks, B broadcast once per GEMM from rank 0 with NCCL in K-panels overlapped with
           the compute -- strong scaling; the broadcast is inside the timed step.
`value` is whole-job TFLOP/s (2*M*N*K per step) on the device clock (CUDA events, max over ranks).
`e2e` is the same metric through the host-buffer API with the host<->device copies timed.
The extra objects carry the other parts of the metric (3xTF32 path, ABFT overhead, SAXPY/SDOT
GB/s), each with its own roofline.  `--impl reference` times the reference's own CPU GEMM
(utils/utils.cu:93-103, compiled from the reference tree into oracle/_ref) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "SGEMM TFLOPS @6144^3 fp32"
N1 = 6144
NMULTI = 32768
CPU_SAMPLE_N = 1152          # reference CPU GEMM sample: 1152^3 = (3/16 * 6144)^3, about 1/152 of the flop


def ncu_traffic(key):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the table of ncu captures
    kept in profiles/dram_traffic.md (one row per kernel and size: | key | read bytes | write bytes | capture |);
    None when no capture of that kernel at that size has been recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    try:
        for line in open(path):
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 3 and cells[0] == key:
                return float(cells[1]) + float(cells[2])
    except (OSError, ValueError):
        pass
    return None


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: through NVML (read-only, every few
    milliseconds) when the bindings are there, else with nvidia-smi (about ten samples a second)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop_flag, self.thread, self.label = index, [], False, None, None

    def _nvml_handle(self):
        """NVML handle of this process's CUDA device `index` (by PCI bus id, so that CUDA_VISIBLE_DEVICES does not
        matter), or None when NVML cannot be used.  NVML is only read here, never written."""
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            pr = torch.cuda.get_device_properties(self.index)
            try:
                bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
                return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)
        except Exception:
            return None, None

    def _run(self):
        nv, h = self._nvml_handle()
        if h is not None:
            # a few milliseconds per sample: a timed region of tens of milliseconds still gets several
            bits = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))
            try:
                mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
                while not self.stop_flag:
                    mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                    try:
                        rs = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    self.samples.append([str(mhz), str(mx)] + [("Active" if rs & b else "Not Active") for _, b in bits] + [self.label])
                    time.sleep(0.004)
                return
            except Exception:
                pass
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([v.strip() for v in out.split(",")][:6] + [self.label])
            except Exception:
                pass
            time.sleep(0.1)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        self.thread.join(timeout=10)

    def summary(self, label=None):
        """All samples, or those taken while `label` was set (the interleaved legs)."""
        mhz, mx, reasons = [], 0, set()
        for s in self.samples:
            if label is not None and (len(s) < 7 or s[6] != label):
                continue
            try:
                mhz.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def timed(fn, steps, warmup, dist_barrier=None):
    """ms per step: `warmup` untimed calls, then exactly `steps` calls between CUDA events on the current stream."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_barrier:
        dist_barrier()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    beg.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if dist_barrier:
        dist_barrier()
    return beg.elapsed_time(end) / steps


def timed_interleaved(legs, rounds=8, reps=5, clk=None):
    """Times several alternatives under the same conditions: A, B, A, B, ... for `rounds` rounds, each turn a block of
    `reps` back-to-back calls between its own event pair, followed by a synchronize.  `clk` (a running ClockSampler)
    is told which leg is on, so that every leg gets its own clock record.  Returns {leg: {"ms": median over the
    blocks, "ms_min", "ms_all", "clocks": {...}, "ms_x_ghz": median ms times median SM GHz}}."""
    import torch
    for fn in legs.values():
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    out = {k: [] for k in legs}
    for _ in range(rounds):
        for k, fn in legs.items():
            if clk is not None:
                clk.label = k
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            if clk is not None:
                clk.label = None
            out[k].append(e0.elapsed_time(e1) / reps)
    res = {}
    for k, v in out.items():
        sv = sorted(v)
        med = sv[len(sv) // 2]
        c = clk.summary(k) if clk is not None else None
        res[k] = {"ms": med, "ms_min": sv[0], "ms_all": v, "clocks": c,
                  "ms_x_ghz": (med * c["sm_mhz"] / 1e3) if c and c.get("sm_mhz") else None}
    return res


def sampled_rows_error(torch, A_rows, B, C_rows, chunk=4096):
    """max |C - C_ref| / (|A| |B|) over a few rows of a product C = A B (alpha = 1, beta = 0): the reference rows are
    double-precision dot products formed on the device in column chunks (checker only; nothing of the library runs)."""
    worst = 0.0
    a64 = A_rows.double()
    for c0 in range(0, B.shape[1], chunk):
        b64 = B[:, c0:c0 + chunk].double()
        ref = a64 @ b64
        den = a64.abs() @ b64.abs()
        err = ((C_rows[:, c0:c0 + chunk].double() - ref).abs() / den.clamp_min(1e-30)).max().item()
        worst = max(worst, float(err))
        del b64, ref, den
    return worst


def abft_fault_report(b2, torch, n, path):
    """Benchmark configuration 3 at one size and math path: a clean run (false alarms, output identical to the plain
    kernel) and the seeded plan of one bit flip (bit 20..30 of a random accumulator) per 64 output tiles."""
    tol = 1e-5 if path == 0 else 2e-5
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    plain = torch.zeros((n, n), device="cuda")
    if path == 1:
        # the ABFT kernel accumulates a tile over all of K in one go: compare with the plain kernel that does too, and
        # keep both from cutting the tiles of a partial last round along K (which changes the last bits of those tiles)
        b2.set_tf32_chunk(0)
        b2.set_tf32_tail_split(0)
    try:
        b2.sgemm(n, n, n, 1.0, A, B, 0.0, plain, path=path)
    finally:
        if path == 1:
            b2.set_tf32_chunk(-1)
    try:
        return _abft_fault_report_body(b2, torch, n, path, tol, A, B, plain)
    finally:
        if path == 1:
            b2.set_tf32_tail_split(1)


def _abft_fault_report_body(b2, torch, n, path, tol, A, B, plain):
    out = torch.zeros((n, n), device="cuda")
    rep = b2.new_report()
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=path, report=rep)
    clean = b2.read_report(rep)
    clean_same = bool(torch.equal(out, plain)) if path == 0 else bool(((out - plain).abs().max() == 0).item())
    plan = b2.seeded_fault_plan(n, n, n, seed=6)
    rep = b2.new_report()
    out.zero_()
    b2.ft_sgemm(n, n, n, 1.0, A, B, 0.0, out, path=path, plan=b2.make_plan(plan), report=rep)
    b2.check_status()
    r = b2.read_report(rep)
    left = (out != plain)
    n_left = int(left.sum().item())
    worst = 0.0
    if n_left:
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            idx = left.nonzero()
            rows = idx[:, 0].unique()
            den = (A[rows].abs() @ B.abs())
            dev = (out[rows] - plain[rows]).abs() / den
            worst = float(dev.max().item())
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old
    return {"n": n, "planned": int(len(plan)), "injected": r["injected"], "detected": r["detected"], "corrected": r["corrected"],
            "false_alarms": r["false_alarms"], "clean_run": {"false_alarms": clean["false_alarms"], "detected": clean["detected"],
                                                            "identical_to_plain_kernel": clean_same},
            "outputs_differing_from_plain_kernel": n_left,
            "largest_remaining_deviation_over_abs_a_abs_b": worst, "tolerance": tol,
            "every_fault_beyond_tolerance_corrected": bool(worst <= tol)}


def cpu_reference_gemm_tflops(n, reps):
    """The reference's own cpu_gemm (oracle/_ref) when built, else the oracle port; 1 thread (it is serial)."""
    import numpy as np
    import oracle
    a = oracle.fill_uniform(n * n, 1).reshape(n, n)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    c = oracle.fill_uniform(n * n, 3).reshape(n, n)
    use_ref = oracle.ref_lib() is not None
    fn = (lambda: oracle.ref_cpu_gemm(1.0, 0.5, a, b, c)) if use_ref else (lambda: oracle.cpu_gemm(1.0, 0.5, a, b, c))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return 2.0 * n ** 3 / (sum(times) / len(times)) / 1e12, ("reference" if use_ref else "port"), times


def reference_gpu_kernel_tflops(kernel_id=11, n=N1):
    """The reference's own kernel/sgemm driver, compiled unmodified for sm_100a (oracle/_ref/ref_sgemm), run on this
    GPU: its sgemm_<kernel_id> at one size.  Only kernels without the one-slab over-read (9, 11) are ever run.
    Returns TFLOP/s or None when the binary or a GPU is missing."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_sgemm")
    if kernel_id not in (9, 11) or not os.path.exists(exe):
        return None
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        r = subprocess.run([exe, str(kernel_id), str(n), str(n), "32"], capture_output=True, text=True, timeout=300)
        if r.returncode != 0:
            return None
        vals = [v for v in r.stdout.strip().splitlines()[-1].split(",") if v.strip()]
        return float(vals[-1]) / 1e3
    except Exception:
        return None


def run_reference(args):
    """--impl reference: the reference's CPU GEMM on the host cores, same metric and unit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np  # noqa: F401
    n = CPU_SAMPLE_N
    tf_w, kind, _ = cpu_reference_gemm_tflops(n, max(0, args.warmup)) if args.warmup > 0 else (0, None, None)
    tf, kind, times = cpu_reference_gemm_tflops(n, args.steps)
    import oracle
    # the same arithmetic with the row loop split over every host core (bit-identical results)
    a = oracle.fill_uniform(n * n, 1).reshape(n, n)
    b = oracle.fill_uniform(n * n, 2).reshape(n, n)
    c = oracle.fill_uniform(n * n, 3).reshape(n, n)
    t0 = time.perf_counter()
    oracle.sgemm_f32(1.0, a, b, 0.5, c)
    t_all = time.perf_counter() - t0
    sample = f"row-major SGEMM {n}^3 per step (alpha=1, beta=0.5, uniform[-1,1]); 6144^3 is {(N1 / n) ** 3:.0f}x the flop"
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"sgemm_rowmajor_{n}^3_cpu_sample_of_{N1}^3", "alpha": 1.0, "beta": 0.5,
                   "code": "utils/utils.cu:93-103 cpu_gemm compiled from the reference tree (oracle/_ref)" if kind == "reference"
                   else "oracle port of cpu_gemm"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": 1, "kind": kind, "sample": sample,
                         "all_cores_port": {"value": 2.0 * n ** 3 / t_all / 1e12, "cores": os.cpu_count()}},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        # context only: the reference's Turing kernel sgemm_11 recompiled for sm_100a on this GPU, 6144^3
        "reference_gpu_kernel": {"kernel": "sgemm_11 (kernel/sgemm/include/kernel_11.cuh:15), unmodified, -arch=sm_100a",
                                 "value": reference_gpu_kernel_tflops(11), "unit": "TFLOP/s"},
    }
    print(json.dumps(line))
    return 0


def bench_vectors(b2, torch, peaks, steps, warmup, log2n=28):
    """SAXPY / SDOT at n = 2^28 (1 GiB per vector, larger than L2): GB/s against the measured HBM copy peak."""
    out = {}
    n = 1 << log2n
    x = b2.fill_uniform(torch.empty(n, device="cuda"), 4)
    y = b2.fill_uniform(torch.empty(n, device="cuda"), 5)
    res = torch.zeros(1, device="cuda")
    ms = timed(lambda: b2.saxpy(n, 2.0, x, y), steps, warmup)
    gbs = 12.0 * n / (ms * 1e-3) / 1e9
    out["saxpy"] = {"n": n, "ms": ms, "value": gbs, "unit": "GB/s",
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / peaks["hbm_gbs"], "traffic": ncu_traffic("saxpy_2p28"),
                                 "algorithmic_bytes": 12 * n, "peak_source": peaks["source"], "frac_of_8TBs_spec": gbs / 8000.0}}
    ms = timed(lambda: b2.sdot(n, x, y, res), steps, warmup)
    gbs = 8.0 * n / (ms * 1e-3) / 1e9
    out["sdot"] = {"n": n, "ms": ms, "value": gbs, "unit": "GB/s",
                   "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": gbs / peaks["hbm_gbs"], "traffic": ncu_traffic("sdot_2p28"),
                                "algorithmic_bytes": 8 * n, "peak_source": peaks["source"], "frac_of_8TBs_spec": gbs / 8000.0}}
    return out


def cublas_abft_baseline_ms(torch, A, B, Cm, steps, warmup):
    """The reference's NON-fused ABFT baseline ("Ding et al." line of its plots), reproduced step for step with
    library calls (kernel/ft_sgemm/include/baseline_ft_sgemm.cuh:1-34): per 256-wide K panel one cuBLAS SGEMM,
    six SGEMVs (row/col sums of C, A, B and their products), two AXPYs and two DOTs, with a device
    synchronisation between the stages.  Comparison line only; nothing of the library runs here."""
    torch.backends.cuda.matmul.allow_tf32 = False
    n = A.shape[0]
    e = torch.ones(n, device="cuda")

    def one():
        for k0 in range(0, n, 256):
            a, b = A[:, k0:k0 + 256], B[k0:k0 + 256, :]
            torch.addmm(Cm, a, b, beta=0.5, alpha=1.0, out=Cm)
            torch.cuda.synchronize()
            c_row, c_col = torch.mv(Cm, e), torch.mv(Cm.t(), e)
            a_col, b_row = torch.mv(a.t(), e), torch.mv(b, e)
            torch.cuda.synchronize()
            ab_col, ba_row = torch.mv(b.t(), a_col), torch.mv(a, b_row)
            torch.cuda.synchronize()
            c_col.add_(ab_col, alpha=-1.0)
            torch.dot(c_col, e)
            torch.cuda.synchronize()
            c_row.add_(ba_row, alpha=-1.0)
            torch.dot(c_row, e)
    return timed(one, steps, warmup)


def run_vec_sweep(args):
    """Benchmark configuration 4: SAXPY and SDOT at n = 2^20, 2^24, 2^28, 2^30 (alpha = 2).  The two small sizes fit in the
    126 MB L2; they are timed twice: back to back on the same vectors (L2-resident) and rotating through enough
    distinct vector pairs to exceed L2 (the reference's own trick, kernel/saxpy/saxpy.cu:79-80,126)."""
    import torch
    import hpcdeepneuralnetworks_b200 as b2
    torch.cuda.set_device(0)
    peaks = load_peaks()
    rows = []
    res = torch.zeros(1, device="cuda")
    for log2n in (20, 24, 28, 30):
        n = 1 << log2n
        pairs = max(1, min(64, (512 * 2 ** 20) // (8 * n)))          # distinct (x, y) pairs: >= 512 MB in rotation
        xs = b2.fill_uniform(torch.empty(pairs * n, device="cuda"), 4)
        ys = b2.fill_uniform(torch.empty(pairs * n, device="cuda"), 5)
        state = {"i": 0}

        def rot(fn):
            def f():
                i = state["i"] = (state["i"] + 1) % pairs
                fn(xs[i * n:(i + 1) * n], ys[i * n:(i + 1) * n])
            return f
        reps = 200 if log2n <= 24 else 10
        row = {"n": n, "log2n": log2n, "pairs_in_rotation": pairs}
        for name, per_elt, fn in (("saxpy", 12.0, lambda x, y: b2.saxpy(n, 2.0, x, y)), ("sdot", 8.0, lambda x, y: b2.sdot(n, x, y, res))):
            ms = timed(rot(fn), reps, 5)
            row[name + "_gbs"] = per_elt * n / (ms * 1e-3) / 1e9
            row[name + "_frac_of_measured_hbm"] = row[name + "_gbs"] / peaks["hbm_gbs"]
            if pairs > 1:
                ms_hot = timed(lambda: fn(xs[:n], ys[:n]), reps, 5)
                row[name + "_gbs_l2_resident"] = per_elt * n / (ms_hot * 1e-3) / 1e9
        rows.append(row)
        del xs, ys
    print(json.dumps({"sweep": "saxpy_sdot_config4", "alpha": 2.0, "hbm_peak_gbs": peaks["hbm_gbs"], "rows": rows}))
    return 0


def run_series(args):
    """The reference's step-wise series sgemm_1 .. sgemm_14 (kernel/sgemm/include/kernel_*.cuh) at one size, GFLOPS per
    rung as in its README table and fig/ABFT_GEMM/bar_graph/fig9_plot_step_wise.py.  Prints one JSON object."""
    import torch
    import hpcdeepneuralnetworks_b200 as b2
    torch.cuda.set_device(0)
    n = args.size or 2048
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    Cm = b2.fill_uniform(torch.empty((n, n), device="cuda"), 3)
    flush = torch.empty(160 * 2 ** 20 // 4, device="cuda")
    ms_flush = timed(lambda: flush.zero_(), 10, 3)
    rows = []
    for kid in range(1, 15):
        def one():
            flush.zero_()
            b2.sgemm_series(kid, n, A, B, Cm, 1.0, 0.5)
        reps = 3 if kid <= 2 else 8
        ms = max(timed(one, reps, 2) - ms_flush, 1e-6)
        rows.append({"kernel": kid, "ms": ms, "gflops": 2.0 * n ** 3 / (ms * 1e-3) / 1e9})
    print(json.dumps({"series": "sgemm_1..14", "n": n, "alpha": 1.0, "beta": 0.5,
                      "l2": "160 MB flush between launches, flush time subtracted", "rows": rows}))
    return 0


def run_sweep(args):
    """Benchmark configuration 2: square row-major SGEMM, N = 256 .. 6144 step 256, alpha=1, beta=0.5, both math paths.
    Prints one JSON object with a row per size (not the headline line)."""
    import torch
    import hpcdeepneuralnetworks_b200 as b2
    torch.cuda.set_device(0)
    peaks = load_peaks()
    ffma_peak = b2.ffma_peak_tflops()
    nmax = args.size or N1
    A = b2.fill_uniform(torch.empty(nmax * nmax, device="cuda"), 1)
    B = b2.fill_uniform(torch.empty(nmax * nmax, device="cuda"), 2)
    Cm = b2.fill_uniform(torch.empty(nmax * nmax, device="cuda"), 3)
    flush = torch.empty(160 * 2 ** 20 // 4, device="cuda")       # > L2: written between timed launches of small sizes
    rows = []
    for n in range(256, nmax + 1, 256):
        a, b, c = A[:n * n].view(n, n), B[:n * n].view(n, n), Cm[:n * n].view(n, n)
        row = {"n": n}
        for path, key in ((0, "ffma"), (1, "3xtf32")):
            small = 3 * 4 * n * n < 2 * 126 * 2 ** 20               # operands could sit in L2: flush between launches
            def one():
                if small:
                    flush.zero_()
                b2.sgemm(n, n, n, 1.0, a, b, 0.5, c, path=path)
            reps = 20 if n <= 2048 else 8
            if small:
                # time the flush alone and subtract it
                ms_both = timed(one, reps, 3)
                ms_flush = timed(lambda: flush.zero_(), reps, 3)
                ms = max(ms_both - ms_flush, 1e-6)
            else:
                ms = timed(one, reps, 3)
            row[key + "_ms"] = ms
            row[key + "_tflops"] = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
        row["ffma_frac_of_fp32_peak"] = row["ffma_tflops"] / ffma_peak
        row["3xtf32_tensor_frac"] = 3 * row["3xtf32_tflops"] / (peaks["bf16_tflops"] / 2)
        rows.append(row)
    b2.check_status()
    print(json.dumps({"sweep": "sgemm_rowmajor_square", "alpha": 1.0, "beta": 0.5, "ffma_peak_tflops": ffma_peak,
                      "tf32_peak_tflops": peaks["bf16_tflops"] / 2, "l2": "sizes whose operands fit twice in L2 are timed with a 160 MB flush between launches, flush time subtracted",
                      "rows": rows}))
    return 0


def single_gpu_anchors(b2, torch, peaks, ffma_peak, n=NMULTI, panel=4096):
    """The workloads of the multi-GPU lines on ONE GPU, through the same entry points (b2_mg_sgemm with a world of one:
    the K-panel schedule without a broadcast; b2_mg_sdot), so that N-GPU values can be divided by a 1-GPU value of the
    same workload: SGEMM 32768^3 (alpha = 1, beta = 0) and SDOT over 2^30 elements."""
    from hpcdeepneuralnetworks_b200 import dist as b2dist
    out = {}
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1000)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    Cm = torch.zeros((n, n), device="cuda")
    ms = timed(lambda: b2dist.sharded_sgemm(n, n, n, 1.0, A, B, 0.0, Cm, panel=panel, path=0), 2, 1)
    b2.check_status()
    rows = torch.tensor([0, n // 2 + 77, n - 1], device="cuda")
    err = sampled_rows_error(torch, A[rows], B, Cm[rows])
    tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
    out["sgemm_32768_1gpu"] = {"n": n, "ms": ms, "value": tf, "unit": "TFLOP/s", "path": "ffma", "panel_k": panel, "steps": 2,
                               "frac_of_fp32_peak": tf / ffma_peak,
                               "checked": {"rows": [int(r) for r in rows.tolist()], "max_err_over_abs_a_abs_b": err, "tolerance": 1e-5,
                                           "ok": bool(err <= 1e-5)}}
    del A, B, Cm
    torch.cuda.empty_cache()
    m = 1 << 30
    x = b2.fill_uniform(torch.empty(m, device="cuda"), 4)
    y = b2.fill_uniform(torch.empty(m, device="cuda"), 5)
    ms = timed(lambda: b2dist.sharded_sdot(m, x, y), 5, 3)
    got = float(b2dist.sharded_sdot(m, x, y).item())
    ref, scale = 0.0, 0.0
    for c0 in range(0, m, 1 << 26):
        xd, yd = x[c0:c0 + (1 << 26)].double(), y[c0:c0 + (1 << 26)].double()
        ref += float((xd * yd).sum().item())
        scale += float((xd * yd).abs().sum().item())
    gbs = 8.0 * m / (ms * 1e-3) / 1e9
    out["sdot_2p30_1gpu"] = {"n": m, "ms": ms, "value": gbs, "unit": "GB/s", "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                             "checked": {"rel_err_over_sum_abs": abs(got - ref) / scale, "tolerance": 1e-5,
                                         "ok": bool(abs(got - ref) <= 1e-5 * scale)}}
    return out


def run_single(args):
    import torch
    import hpcdeepneuralnetworks_b200 as b2
    torch.cuda.set_device(0)
    peaks = load_peaks()
    if args.sweep:
        return run_sweep(args)
    if args.series:
        return run_series(args)
    if args.vec_sweep:
        return run_vec_sweep(args)
    if args.only == "vectors":   # small-case command for profiling the streaming kernels
        print(json.dumps(bench_vectors(b2, torch, peaks, args.steps, args.warmup, args.vec_log2n)))
        return 0
    n = args.size or N1
    flop = 2.0 * n ** 3
    path = 1 if args.path == "3xtf32" else 0
    A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
    B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
    Cm = b2.fill_uniform(torch.empty((n, n), device="cuda"), 3)
    sm_count = b2.device_info()["sm_count"]

    # FP32 SIMT peak, measured live with a register-only FMA stream (the roofline of the FFMA path)
    ffma_peak = b2.ffma_peak_tflops()

    def step(p=path):
        if args.abft:
            b2.ft_sgemm(n, n, n, 1.0, A, B, 0.5, Cm, path=p)
        else:
            b2.sgemm(n, n, n, 1.0, A, B, 0.5, Cm, path=p)

    with ClockSampler(0) as clk:
        ms = timed(step, args.steps, args.warmup)
    b2.check_status()
    clocks = clk.summary()
    tflops = flop / (ms * 1e-3) / 1e12

    def tf32_library_peak():
        """cuBLAS TF32 GEMM 8192^3 through torch, best of 5 (the same recipe as the pool's bf16 peak): context for
        the tensor-path fraction, since TF32 is not in MEASURED_PEAKS.json."""
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            m = 8192
            x = torch.rand(m, m, device="cuda")
            y = torch.rand(m, m, device="cuda")
            for _ in range(2):
                x @ y
            best = 1e30
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                x @ y
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            return 2.0 * m ** 3 / (best * 1e-3) / 1e12
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old

    tf32_lib = None if args.quick else tf32_library_peak()

    def roof(p, tf):
        if p == 0:
            return {"bound": "fp32_simt", "achieved": tf, "peak": ffma_peak, "unit": "TFLOP/s", "frac": tf / ffma_peak,
                    "traffic": ncu_traffic("sgemm_ffma_6144") if n == N1 else None, "peak_source": "register-only FFMA probe, same run",
                    "peak_spec": sm_count * 128 * 2 * 1.965e9 / 1e12, "algorithmic_flop": flop}
        tf32_peak = peaks["bf16_tflops"] / 2.0       # dense TF32 runs at half the bf16 rate
        return {"bound": "tensor", "achieved": 3.0 * tf, "peak": tf32_peak, "unit": "TFLOP/s", "frac": 3.0 * tf / tf32_peak,
                "traffic": ncu_traffic("sgemm_3xtf32_6144") if n == N1 else None, "peak_source": f"{peaks['source']} bf16 GEMM / 2",
                "useful_tflops": tf, "algorithmic_flop": 3.0 * flop,
                "cublas_tf32_gemm_tflops_same_run": tf32_lib, "frac_of_cublas_tf32": (3.0 * tf / tf32_lib) if tf32_lib else None}

    extras = {}
    if not args.quick:
        other = 1 - path
        ms_o = timed(lambda: step(other), max(3, args.steps // 2), 3)
        b2.check_status()
        tf_o = flop / (ms_o * 1e-3) / 1e12
        extras["sgemm_3xtf32" if other == 1 else "sgemm_ffma"] = {"ms": ms_o, "value": tf_o, "unit": "TFLOP/s",
                                                                  "roofline": roof(other, tf_o)}
        # ABFT overhead: plain and fault-tolerant kernels timed interleaved (A, B, A, B, ... blocks of 5 calls, 8 rounds
        # each), so that both legs see the same power and clock state; every leg carries its own clock record
        for key, pth in (("abft_ffma", 0), ("abft_3xtf32", 1)):
            try:
                with ClockSampler(0) as clk2:
                    legs = timed_interleaved({"plain": lambda: step(pth),
                                              "abft": lambda: b2.ft_sgemm(n, n, n, 1.0, A, B, 0.5, Cm, path=pth)}, clk=clk2)
                b2.check_status()
                ms_ft, ms_pl = legs["abft"]["ms"], legs["plain"]["ms"]
                extras[key] = {"ms": ms_ft, "value": flop / (ms_ft * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "plain_ms_interleaved": ms_pl, "overhead_pct": 100.0 * (ms_ft / ms_pl - 1.0),
                               "overhead_pct_at_equal_clock": (100.0 * (legs["abft"]["ms_x_ghz"] / legs["plain"]["ms_x_ghz"] - 1.0)
                                                               if legs["abft"]["ms_x_ghz"] and legs["plain"]["ms_x_ghz"] else None),
                               "method": "interleaved blocks of 5 calls, 8 rounds per leg, median block",
                               "clocks_plain": legs["plain"]["clocks"], "clocks_abft": legs["abft"]["clocks"],
                               "ms_blocks_plain": legs["plain"]["ms_all"], "ms_blocks_abft": legs["abft"]["ms_all"]}
            except Exception as e:  # reported, not hidden
                extras[key] = {"error": str(e)}
        # benchmark configuration 3: clean run and seeded single-bit faults at 1024, 4096, 8192 on both paths
        try:
            extras["abft_config3"] = {("ffma" if pth == 0 else "3xtf32"): [abft_fault_report(b2, torch, m, pth) for m in (1024, 4096, 8192)]
                                      for pth in (0, 1)}
        except Exception as e:
            extras["abft_config3"] = {"error": str(e)}
        try:
            ms_cb = cublas_abft_baseline_ms(torch, A, B, Cm, 3, 1)
            extras["abft_cublas_nonfused_baseline"] = {"ms": ms_cb, "value": flop / (ms_cb * 1e-3) / 1e12, "unit": "TFLOP/s",
                                                       "note": "cuBLAS gemm/gemv/axpy/dot per 256-K panel with syncs, as baseline_ft_sgemm.cuh"}
        except Exception as e:
            extras["abft_cublas_nonfused_baseline"] = {"error": str(e)}
        extras.update(bench_vectors(b2, torch, peaks, max(5, args.steps), 3))
        del A, B, Cm
        torch.cuda.empty_cache()
        try:
            extras.update(single_gpu_anchors(b2, torch, peaks, ffma_peak))
        except Exception as e:
            extras["sgemm_32768_1gpu"] = {"error": str(e)}
        A = b2.fill_uniform(torch.empty((n, n), device="cuda"), 1)
        B = b2.fill_uniform(torch.empty((n, n), device="cuda"), 2)
        Cm = b2.fill_uniform(torch.empty((n, n), device="cuda"), 3)

    # end to end through the host-buffer API: pinned host A, B, C -> device -> SGEMM -> host C
    hs = b2.HostSgemm(n, n, n, path=path)
    hs.hA.copy_(A)
    hs.hB.copy_(B)
    hs.hC.copy_(Cm)
    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e = timed(lambda: hs.run(1.0, 0.5), e2e_steps, 1)
    e2e = {"value": flop / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": hs.h2d_bytes(),
           "d2h_bytes_per_step": hs.d2h_bytes(), "ms_per_step": ms_e2e, "steps": e2e_steps}

    cpu = None
    if not args.no_cpu:
        reps = 1
        tf_cpu, kind, _ = cpu_reference_gemm_tflops(CPU_SAMPLE_N, reps)
        cpu = {"value": tf_cpu, "unit": "TFLOP/s", "cores": 1, "kind": kind,
               "sample": f"one row-major SGEMM {CPU_SAMPLE_N}^3 (alpha=1, beta=0.5), 1/{(N1 / CPU_SAMPLE_N) ** 3:.0f} of the flop of {N1}^3"}

    line = {
        "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"sgemm_rowmajor_{n}^3" + ("_abft" if args.abft else ""), "path": args.path, "alpha": 1.0, "beta": 0.5,
                   "inputs": "seeded uniform[-1,1) generated on the device", "l2": "A, B, C are 3 x %d MB, larger than the 126 MB L2" % (4 * n * n // 2 ** 20),
                   "parallelism": "1 GPU"},
        "roofline": roof(path, tflops), "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": args.steps * ((2 if b2.sgemm_workspace_bytes(0, n, n, n) > 0 else 1) if path == 0 else 3),
        "clocks": clocks, "extra": extras,
    }
    print(json.dumps(line))
    return 0


def run_multi(args):
    import torch
    import torch.distributed as dist
    import hpcdeepneuralnetworks_b200 as b2
    from hpcdeepneuralnetworks_b200 import dist as b2dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n = args.size or NMULTI
    path = 1 if args.path == "3xtf32" else 0
    tol = 1e-5 if path == 0 else 2e-5
    start, rows = b2dist.row_block(n, rank, world)
    A = torch.empty((rows, n), device="cuda")
    # every rank fills its own row block of A from its own seeded stream; B comes from rank 0 only
    b2.fill_uniform(A, 1000 + rank)
    B = torch.empty((n, n), device="cuda")
    if rank == 0:
        b2.fill_uniform(B, 2)
    else:
        B.fill_(float("nan"))        # a rank that computed before its panel landed would show
    Cm = torch.zeros((rows, n), device="cuda")
    mg = b2dist.default_mg()         # the library's own communicator (collective), made outside the timed region
    report = b2.new_report() if args.abft else None

    def step(abft=args.abft, rep=report):
        b2dist.sharded_sgemm(n, n, n, 1.0, A, B, 0.0, Cm, src=0, panel=args.panel, path=path, abft=abft, report=rep, mg=mg)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with ClockSampler(local) as clk:
        ms_local = timed(step, args.steps, args.warmup, dist_barrier=barrier)
    b2.check_status()
    ms = max_over_ranks(ms_local)
    flop = 2.0 * n ** 3
    tflops = flop / (ms * 1e-3) / 1e12

    # ---- the result is checked, outside the timed region: three rows of every rank's block of C against double dot
    # products of the same rows of A with the B this rank received
    checked = {}
    pick = torch.tensor(sorted({0, rows // 2, rows - 1}), device="cuda") if rows else torch.empty(0, dtype=torch.long, device="cuda")
    err = sampled_rows_error(torch, A[pick], B, Cm[pick]) if rows else 0.0
    err = max_over_ranks(err if err == err else float("inf"))
    checked["sgemm"] = {"rows_per_rank": int(pick.numel()), "max_err_over_abs_a_abs_b": err, "tolerance": tol, "ok": bool(err <= tol)}

    # ---- the same product with the fault-tolerant kernels: overhead, and the fault report summed over the ranks
    abft_extra = None
    if not args.abft:
        rep2 = b2.new_report()
        ms_ft = max_over_ranks(timed(lambda: step(True, rep2), max(1, min(args.steps, 2)), 1, dist_barrier=barrier))
        b2.check_status()
        rsum = rep2.clone().to(torch.int64)
        dist.all_reduce(rsum, op=dist.ReduceOp.SUM)
        v = rsum.cpu().tolist()
        err_ft = sampled_rows_error(torch, A[pick], B, Cm[pick]) if rows else 0.0
        err_ft = max_over_ranks(err_ft if err_ft == err_ft else float("inf"))
        abft_extra = {"ms": ms_ft, "value": flop / (ms_ft * 1e-3) / 1e12, "unit": "TFLOP/s", "overhead_pct": 100.0 * (ms_ft / ms - 1.0),
                      "report_summed_over_ranks": {"tiles": v[0], "injected": v[1], "detected": v[2], "corrected": v[3],
                                                   "uncorrectable": v[4], "false_alarms": v[5]},
                      "max_err_over_abs_a_abs_b": err_ft}
        checked["abft"] = {"false_alarms": v[5], "detected": v[2], "max_err_over_abs_a_abs_b": err_ft,
                           "ok": bool(v[5] == 0 and v[2] == 0 and err_ft <= tol)}

    # sharded SDOT: 2^30 elements in total, one scalar all-reduce (b2_mg_sdot)
    nloc = (1 << 30) // world
    x = b2.fill_uniform(torch.empty(nloc, device="cuda"), 4 + 10 * rank)
    y = b2.fill_uniform(torch.empty(nloc, device="cuda"), 5 + 10 * rank)
    ms_dot = max_over_ranks(timed(lambda: b2dist.sharded_sdot(nloc, x, y, mg=mg), max(5, args.steps), 3, dist_barrier=barrier))
    dot_nccl = b2dist.sharded_sdot(nloc, x, y, mg=mg).clone()
    # an independent sum for the check: double products summed by torch, all-reduced
    ind = torch.zeros(2, dtype=torch.float64, device="cuda")
    for c0 in range(0, nloc, 1 << 26):
        pr = x[c0:c0 + (1 << 26)].double() * y[c0:c0 + (1 << 26)].double()
        ind[0] += pr.sum()
        ind[1] += pr.abs().sum()
    dist.all_reduce(ind, op=dist.ReduceOp.SUM)
    ref, scale = float(ind[0].item()), float(ind[1].item())

    def same_bits_everywhere(t64):
        g = [torch.empty_like(t64) for _ in range(world)]
        dist.all_gather(g, t64.contiguous())
        return all(bool((gi.view(torch.int64) == t64.view(torch.int64)).all().item()) for gi in g)

    nccl_same = same_bits_everywhere(dot_nccl)
    checked["sdot"] = {"rel_err_over_sum_abs": abs(float(dot_nccl.item()) - ref) / scale, "tolerance": 1e-5,
                       "same_bits_on_every_rank": nccl_same,
                       "ok": bool(nccl_same and abs(float(dot_nccl.item()) - ref) <= 1e-5 * scale)}

    # the same with the cross-GPU sum inside the kernel (peer stores over NVLink, no collective call)
    ms_fused, fused_error = None, None
    fused = None
    try:
        fused = b2dist.FusedSdot(torch.device("cuda", local))
    except Exception as e:
        fused_error = f"{type(e).__name__}: {e}"
    agree = torch.tensor([1 if fused is not None else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)      # every rank runs the fused leg, or none does
    try:
        if int(agree.item()) == 0:
            raise RuntimeError(fused_error or "symmetric memory could not be set up on another rank")
        ms_fused = max_over_ranks(timed(lambda: fused(nloc, x, y), max(5, args.steps), 3, dist_barrier=barrier))
        dot_fused = fused(nloc, x, y).clone()
        b2.check_status()
        fused_same = same_bits_everywhere(dot_fused)
        gap = abs(float(dot_fused.item()) - float(dot_nccl.item()))
        checked["sdot_fused"] = {"rel_err_over_sum_abs": abs(float(dot_fused.item()) - ref) / scale, "tolerance": 1e-5,
                                 "same_bits_on_every_rank": fused_same,
                                 "gap_to_allreduce_form_over_sum_abs": gap / scale,
                                 "same_bits_as_allreduce_form": bool(gap == 0.0),
                                 "ok": bool(fused_same and abs(float(dot_fused.item()) - ref) <= 1e-5 * scale and gap <= 1e-12 * scale)}
    except Exception as e:   # reported below, never hidden
        fused_error = f"{type(e).__name__}: {e}"

    all_ok = all(c["ok"] for c in checked.values())
    if rank == 0:
        ffma_peak = b2.ffma_peak_tflops()
        peaks = load_peaks()
        per_gpu = tflops / world
        launches_per_panel = 2 if path == 0 else 3     # the GEMM kernel, plus the transpose of the A panel (FFMA) or the two split kernels
        line = {
            "metric": METRIC.replace("6144", str(n)), "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"sgemm_rowmajor_{n}^3_rowblock_sharded" + ("_abft" if args.abft else ""), "path": args.path, "alpha": 1.0, "beta": 0.0,
                       "parallelism": f"A,C row blocks over {world} GPUs; B broadcast from rank 0 per GEMM in K-panels of {args.panel} (NCCL) inside b2_mg_sgemm",
                       "l2": "operands are GBs per GPU, far larger than L2",
                       "one_gpu_value_of_this_workload": "extra.sgemm_32768_1gpu of the --gpus 1 line"},
            "roofline": {"bound": "fp32_simt" if path == 0 else "tensor", "achieved": per_gpu if path == 0 else 3 * per_gpu,
                         "peak": ffma_peak if path == 0 else peaks["bf16_tflops"] / 2, "unit": "TFLOP/s",
                         "frac": (per_gpu / ffma_peak) if path == 0 else (3 * per_gpu / (peaks["bf16_tflops"] / 2)),
                         "traffic": None, "note": "per-GPU average, broadcast included in the time"},
            "cpu_baseline": None,
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "operands of 32768^3 are generated on the device; no host copy is part of this workload"},
            "gpu_launches": args.steps * len(b2dist.k_panels(n, args.panel)) * launches_per_panel,
            "clocks": clk.summary(),
            "checked": dict(checked, all_ok=all_ok),
            "abft_report": (b2.read_report(report) if args.abft else None),
            "extra": {"abft": abft_extra,
                      "sdot_sharded": {"n_total": nloc * world, "ms": ms_dot, "value": 8.0 * nloc * world / (ms_dot * 1e-3) / 1e9,
                                       "unit": "GB/s", "per_gpu_frac_of_hbm_peak": 8.0 * nloc / (ms_dot * 1e-3) / 1e9 / peaks["hbm_gbs"]},
                      "sdot_sharded_fused": ({"n_total": nloc * world, "ms": ms_fused, "value": 8.0 * nloc * world / (ms_fused * 1e-3) / 1e9,
                                              "unit": "GB/s", "per_gpu_frac_of_hbm_peak": 8.0 * nloc / (ms_fused * 1e-3) / 1e9 / peaks["hbm_gbs"]}
                                             if ms_fused else {"error": fused_error})},
        }
        print(json.dumps(line))
    dist.barrier()
    mg.close()
    dist.destroy_process_group()
    return 0 if all_ok else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="ffma", choices=["ffma", "3xtf32"])
    ap.add_argument("--size", type=int, default=0, help="override the matrix size (profiling of small cases)")
    ap.add_argument("--panel", type=int, default=4096, help="K-panel of the B broadcast (multi-GPU)")
    ap.add_argument("--only", default="all", choices=["all", "vectors"], help="vectors: SAXPY/SDOT only (profiling)")
    ap.add_argument("--vec-log2n", type=int, default=28, help="log2 of the vector length of the SAXPY/SDOT leg")
    ap.add_argument("--vec-sweep", action="store_true", help="config 4: SAXPY/SDOT at n = 2^20, 2^24, 2^28, 2^30")
    ap.add_argument("--series", action="store_true", help="the reference's rungs sgemm_1..14 at --size (default 2048)")
    ap.add_argument("--sweep", action="store_true", help="config 2: N = 256..6144 step 256, both paths (prints a table object)")
    ap.add_argument("--abft", action="store_true", help="time the fault-tolerant SGEMM as the headline step (profiling)")
    ap.add_argument("--quick", action="store_true", help="headline kernel only (no extras); used for profiling")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.quick else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    from hpcdeepneuralnetworks_b200 import _lib
    _lib.load()   # raises if the CUDA library is missing: there is no fallback
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_multi(args)
    return run_single(args)


if __name__ == "__main__":
    sys.exit(main())

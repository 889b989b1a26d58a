"""Generator of the SGEMM tile families (the role of kernel/ft_sgemm/code_gen/main.py:4-19 and
code_gen/code_gen.py:4-30 in the reference).

The reference generator prints one CUDA kernel per parameter tuple ``(ms, ns, ks, mw, nw, mr, nr)`` and an
``if_abft`` flag.  Here each math path is one C++ template, and the generator turns a table of tuples into the
instantiation / launch tables the library compiles:

* ``csrc/ffma_tiles.inc`` -- FP32 FFMA path, ``sgemm_ffma_kernel<BM, NR, MR, STAGES, ...>`` (csrc/sgemm_ffma.cu): one
  ``B2_FFMA_TILE(name, BM, NR, MR, stages, efficiency, min_waves)`` row per tile, expanded into the plain and ABFT,
  row-major and K-major instantiations, the launch table and the automatic picker.
* ``csrc/tf32_tiles.inc`` -- 3xTF32 tensor-core path (csrc/sgemm_3xtf32.cu): one
  ``B2_TF32_TILE(name, form, TBN, TBK, cost)`` row per kernel form the dispatcher may choose by whole waves.

From each tuple (plus ``stages`` and, for 3xTF32, the kernel form) the generator derives what the reference derives
(code_gen.py:5-30: thread count, vector widths) and what sm_100a adds: warps, thread tile, bytes per ring stage,
shared memory per CTA, CTAs per SM, a register estimate and tensor-memory columns -- and refuses, with the reason, what
the hardware or the templates cannot run.  ``efficiency`` / ``cost`` come from ``tile_measurements.json`` (throughput of
every tile at 4096^3 and 8192^3 on a B200, from back-to-back launches through the C ABI with the tile pinned).

    python -m hpcdeepneuralnetworks_b200.gen_ft_sgemm            # rewrite both .inc files
    python -m hpcdeepneuralnetworks_b200.gen_ft_sgemm --check    # fail if a committed file is stale
    python -m hpcdeepneuralnetworks_b200.gen_ft_sgemm --describe # print the derived figures of every tile

Tuple meaning (as in the reference): ms x ns x ks = block tile, mw x nw = warp tile, mr x nr = thread tile.
"""
from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_FFMA = os.path.join(HERE, "csrc", "ffma_tiles.inc")
OUT_TF32 = os.path.join(HERE, "csrc", "tf32_tiles.inc")
MEASURED = os.path.join(HERE, "tile_measurements.json")

SMEM_PER_SM = 227 * 1024          # usable by CTAs; each resident CTA also takes 1 KB of system use
SMEM_PER_CTA = 227 * 1024
REGS_PER_SM = 65536
TMEM_COLUMNS = 512

# ---- FP32 FFMA path --------------------------------------------------------------------------------------------
# name: dict(param=(ms, ns, ks, mw, nw, mr, nr), stages=ring depth, min_waves=the picker considers the tile only for
# problems of at least that many waves of resident CTAs)
FFMA_TILES = {
    "huge":   dict(param=(128, 128, 32, 16, 128, 4, 16), stages=3, min_waves=0),   # reference: 128x128x8  (code_gen/main.py:13)
    "tall":   dict(param=(128, 64, 32, 16, 64, 4, 8), stages=3, min_waves=0),      # reference: 128x32x8   (code_gen/main.py:11)
    "wide":   dict(param=(32, 128, 32, 16, 128, 4, 16), stages=3, min_waves=0),    # reference: 32x128x8   (code_gen/main.py:12)
    "large":  dict(param=(64, 64, 32, 16, 64, 4, 8), stages=3, min_waves=0),       # reference: 64x64x8    (code_gen/main.py:10)
    "medium": dict(param=(32, 64, 32, 16, 64, 4, 8), stages=3, min_waves=0),       # reference: 32x32x8    (code_gen/main.py:9)
    "b200_64x128": dict(param=(64, 128, 32, 16, 128, 4, 16), stages=3, min_waves=0),
    # 8 x 16 outputs per thread: 6 shared loads per 64 packed FMAs instead of 5 per 32 (the shared-memory pipe, not the
    # FMA pipe, bounds the 4 x 16 tiles); 4 warps per CTA, so short problems, which run few CTAs per SM, do better on
    # "huge" (measured: 3072^3, 1.95 waves, 57.2 against 55.9; from 3328^3, 2.3 waves, on the 8 x 16 tile is ahead)
    "b200_8x16": dict(param=(128, 128, 32, 32, 128, 8, 16), stages=3, min_waves=2),
}
TILES = FFMA_TILES    # the name the tests use


def derive_ffma(name: str, param, stages: int = 3) -> dict:
    """Everything the template needs and the hardware limits, from one reference-style tuple; ValueError with the
    reason when the tile cannot exist on sm_100a."""
    ms, ns, ks, mw, nw, mr, nr = param
    problems = []
    if ks != 32:
        problems.append("ks must be 32: one K-slab is one 128-byte swizzled TMA row of A")
    if mr not in (4, 8):
        problems.append("mr must be 4 or 8 (packed FMAs pair columns; rows come in float4 loads)")
    if mw != 4 * mr or nw != ns:
        problems.append("the warp tile must be (4 mr) x ns: lanes are laid out 4 along M x 8 along N")
    if nr * 8 != ns or nr not in (8, 16):
        problems.append("the thread tile must be mr x ns/8 with ns in {64, 128}")
    if ms not in (32, 64, 128) or (mw and ms % mw):
        problems.append("ms must be 32, 64 or 128 and a multiple of mw")
    if not 2 <= stages <= 8:
        problems.append("2 to 8 ring stages")
    if problems:
        raise ValueError(f"tile '{name}' {param}: " + "; ".join(problems))
    warps = ms // mw
    threads = 32 * warps                                  # reference: (ms / mr) * (ns / nr), code_gen.py:8
    assert threads == (ms // mr) * (ns // nr)
    stage = ms * ks * 4 + ks * ns * 4                     # A tile + B tile
    stage_cs = warps * 128 + 1024                         # ABFT: band checksums of A + column-set checksums of B
    smem = 1024 + stages * stage + 128 + stages * stage_cs + 512
    regs = mr * nr + (mr + nr) + 34                       # accumulators, one set of operands, addressing and barriers
    by_warps = (16 if mr == 4 else 8) // warps
    by_smem = SMEM_PER_SM // (smem + 1024)
    ctas = max(1, min(by_warps, by_smem))
    if smem > SMEM_PER_CTA:
        raise ValueError(f"tile '{name}' {param} with {stages} stages: {smem} bytes of shared memory, {SMEM_PER_CTA} per CTA")
    if regs > 255:
        raise ValueError(f"tile '{name}' {param}: about {regs} registers per thread, 255 at most")
    if ctas < 1 or ctas * threads * ((regs + 7) // 8 * 8) > REGS_PER_SM:
        raise ValueError(f"tile '{name}' {param}: {ctas} CTAs of {threads} threads x {regs} registers exceed the register file")
    return dict(bm=ms, bn=ns, nr=nr, mr=mr, stages=stages, warps=warps, threads=threads, stage_bytes=stage, smem_bytes=smem,
                ctas_per_sm=ctas, regs_estimate=regs, launch_bounds=(threads, ctas),
                lds_per_ffma2=round((mr / 4 + nr / 4) / (mr * nr / 2), 4))


def validate(name: str, param, stages: int = 3):
    d = derive_ffma(name, param, stages)
    return d["bm"], d["nr"], d["mr"]


def measured() -> dict:
    try:
        return json.load(open(MEASURED))
    except OSError:
        return {}


def ffma_efficiency(name: str) -> float:
    """Throughput relative to "huge" at the size class the picker would use the tile for: 4096^3, or 8192^3 for a
    tile that is only considered for long problems (min_waves > 0)."""
    m = measured().get("ffma_tflops_8192" if FFMA_TILES[name]["min_waves"] > 0 else "ffma_tflops_4096", {})
    if name in m and "huge" in m:
        return m[name] / m["huge"]
    return 1.0


def render_ffma() -> str:
    lines = ["// Generated by hpcdeepneuralnetworks_b200/gen_ft_sgemm.py -- do not edit by hand.",
             "// B2_FFMA_TILE(name, BM, NR, MR, stages, efficiency, min_waves): block tile BM x (8*NR) x 32, BM/(4*MR) warps,",
             "// MR x NR outputs per thread, `stages` K-slabs in the TMA ring."]
    for name, t in FFMA_TILES.items():
        d = derive_ffma(name, t["param"], t["stages"])
        lines.append(f"// {name}: {d['threads']} threads, {d['smem_bytes']} B shared memory, {d['ctas_per_sm']} CTAs/SM, "
                     f"~{d['regs_estimate']} registers, {d['lds_per_ffma2']} shared loads per packed FMA")
        lines.append(f'B2_FFMA_TILE("{name}", {d["bm"]}, {d["nr"]}, {d["mr"]}, {d["stages"]}, {ffma_efficiency(name):.3f}f, {t["min_waves"]})')
    return "\n".join(lines) + "\n"


# ---- 3xTF32 tensor-core path -----------------------------------------------------------------------------------
# name: dict(param=(ms, ns, ks, ...), form).  ms x ns is the accumulator tile of one CTA (single) or of a CTA pair
# (pair: 256 x 256 over two SMs, tcgen05 cta_group::2); ks the K-slab (32 floats = one 128-byte swizzled row, 16 = one
# 64-byte row).  Each stage holds the hi and lo planes of both operands.
TF32_TILES = {
    "single_128x128": dict(param=(128, 128, 32), form="single"),
    "single_128x256": dict(param=(128, 256, 32), form="single"),
    "pair_256x256": dict(param=(256, 256, 32), form="pair"),
}
TF32_FORMS = {"single": 0, "pair": 1}


def derive_tf32(name: str, param, form: str) -> dict:
    ms, ns, ks = param
    problems = []
    if form not in TF32_FORMS:
        problems.append("form is 'single' or 'pair'")
    if ks not in (16, 32):
        problems.append("ks is 32 (128-byte swizzle) or 16 (64-byte swizzle)")
    if form == "single" and (ms != 128 or ns not in (128, 256)):
        problems.append("a single CTA accumulates 128 rows (the 128 lanes of tensor memory) x 128 or 256 columns")
    if form == "pair" and (ms, ns, ks) != (256, 256, 32):
        problems.append("a CTA pair accumulates 256 x 256 with ks = 32")
    if problems:
        raise ValueError(f"3xTF32 tile '{name}' {param}: " + "; ".join(problems))
    rows_per_cta = 128
    cols_staged = ns if form == "single" else ns // 2       # a pair's CTAs stage half of the B columns each
    stage = 2 * rows_per_cta * ks * 4 + 2 * cols_staged * ks * 4
    stages = (192 * 1024) // stage if form == "single" else 3
    tmem = ns * (2 if form == "pair" else 1)                # the persistent pair kernel double-buffers the accumulator
    smem = 1024 + stages * stage + 256
    if tmem > TMEM_COLUMNS:
        raise ValueError(f"3xTF32 tile '{name}': {tmem} tensor-memory columns, {TMEM_COLUMNS} per SM")
    if smem > SMEM_PER_CTA or stages < 2:
        raise ValueError(f"3xTF32 tile '{name}': {stages} stages of {stage} bytes do not fit {SMEM_PER_CTA} bytes of shared memory")
    return dict(tbn=ns, tbk=ks, form=form, stages=stages, stage_bytes=stage, smem_bytes=smem, tmem_columns=tmem,
                sms_per_tile=2 if form == "pair" else 1, bytes_per_flop=round(stage / (2.0 * 3 * rows_per_cta * ns * ks), 5))


def tf32_cost(name: str) -> float:
    """Time of one tile relative to a single-CTA 128 x 256 tile, per SM slot, from the measured throughputs."""
    m = measured().get("tf32_tile_cost", {})
    return float(m.get(name, {"single_128x128": 0.55, "single_128x256": 1.0, "pair_256x256": 0.9}[name]))


def render_tf32() -> str:
    lines = ["// Generated by hpcdeepneuralnetworks_b200/gen_ft_sgemm.py -- do not edit by hand.",
             "// B2_TF32_TILE(name, form, TBN, TBK, cost): form 0 = one tile per CTA, 1 = one 256 x 256 tile per CTA pair;",
             "// cost = time of one tile relative to a 128 x 256 single-CTA tile (the dispatcher counts whole waves)."]
    for name, t in TF32_TILES.items():
        d = derive_tf32(name, t["param"], t["form"])
        lines.append(f"// {name}: {d['stages']} stages of {d['stage_bytes']} B, {d['smem_bytes']} B shared memory, "
                     f"{d['tmem_columns']} tensor-memory columns, {d['bytes_per_flop']} staged bytes per flop")
        lines.append(f'B2_TF32_TILE("{name}", {TF32_FORMS[d["form"]]}, {d["tbn"]}, {d["tbk"]}, {tf32_cost(name):.3f})')
    return "\n".join(lines) + "\n"


def render() -> str:
    return render_ffma()


def main(argv) -> int:
    outputs = ((OUT_FFMA, render_ffma()), (OUT_TF32, render_tf32()))
    if "--describe" in argv:
        for name, t in FFMA_TILES.items():
            print("ffma", name, derive_ffma(name, t["param"], t["stages"]))
        for name, t in TF32_TILES.items():
            print("3xtf32", name, derive_tf32(name, t["param"], t["form"]))
        return 0
    if "--check" in argv:
        for path, text in outputs:
            if not os.path.exists(path) or open(path).read() != text:
                print(f"{os.path.relpath(path, HERE)} is stale: run python -m hpcdeepneuralnetworks_b200.gen_ft_sgemm", file=sys.stderr)
                return 1
        return 0
    for path, text in outputs:
        with open(path, "w") as fh:
            fh.write(text)
    print(f"wrote {OUT_FFMA} ({len(FFMA_TILES)} tiles) and {OUT_TF32} ({len(TF32_TILES)} tiles)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

"""CPU tests of the C-ABI boundary: the library builds, loads, exports every symbol that
include/b2blas.h declares, and validates arguments before touching the device."""
import ctypes as C

import pytest

from hpcdeepneuralnetworks_b200 import _lib


@pytest.fixture(scope="module")
def L(built_lib):
    return _lib.load()


def test_exports_every_declared_symbol(L):
    names = _lib.declared_symbols()
    assert len(names) >= 28
    for required in ("sgemm", "ft_sgemm", "saxpy", "sdot", "b2_sgemm", "b2_ft_sgemm", "b2_saxpy", "b2_sdot",
                     "b2_sgemm_series", "ref_sgemm_rowmajor", "ref_sgemm_colmajor_nt", "ref_ft_sgemm_colmajor_nt",
                     "b2_sdot_static"):
        assert required in names
    missing = [n for n in names if not hasattr(L, n)]
    assert missing == []


def test_status_strings(L):
    assert L.b2_status_string(0) == b"ok"
    for code in range(-6, 0):
        assert L.b2_status_string(code) not in (b"ok", b"unknown status")
    assert L.b2_status_string(-99) == b"unknown status"
    assert L.b2_version() >= 100


def test_argument_validation_needs_no_device(L):
    null = C.c_void_p(None)
    fake = C.c_void_p(0x1000)
    assert L.b2_sgemm(null, 0, -1, 4, 4, 1.0, fake, 4, fake, 4, 0.0, fake, 4, null) == -1
    assert b"negative" in L.b2_last_error()
    assert L.b2_sgemm(null, 7, 4, 4, 4, 1.0, fake, 4, fake, 4, 0.0, fake, 4, null) == -1
    assert L.b2_sgemm(null, 0, 4, 4, 4, 1.0, fake, 2, fake, 4, 0.0, fake, 4, null) == -1       # lda < K
    assert L.b2_sgemm(null, 0, 4, 4, 4, 1.0, fake, 4, fake, 4, 0.0, fake, 3, null) == -1       # ldc < N
    assert L.b2_sgemm(null, 0, 4, 4, 4, 1.0, null, 4, fake, 4, 0.0, fake, 4, null) == -1       # A NULL
    assert L.b2_sgemm(null, 0, 0, 4, 4, 1.0, null, 4, null, 4, 0.0, null, 4, null) == 0        # empty: no-op
    assert L.b2_saxpy(null, -5, 2.0, fake, fake, null) == -1
    assert L.b2_saxpy(null, 0, 2.0, null, null, null) == 0
    assert L.b2_saxpy(null, 4, 2.0, C.c_void_p(0x1001), fake, null) == -1                      # misaligned
    assert L.b2_sdot(null, 4, fake, fake, null, null) == -1                                    # result NULL
    assert L.b2_sgemm_series(0, 32, 256, fake, fake, fake, 1.0, 0.0, null) == -1
    assert L.b2_sgemm_series(15, 32, 256, fake, fake, fake, 1.0, 0.0, null) == -1
    assert L.b2_sgemm_series(9, 32, 200, fake, fake, fake, 1.0, 0.0, null) == -2               # 200 % 128 != 0
    assert b"multiple of 128" in L.b2_last_error()
    assert L.b2_set_ffma_variant(2) == -1
    assert L.b2_timer_start(null, null) == -1


def test_host_fill_matches_oracle(L):
    import numpy as np
    import oracle
    buf = np.empty(1000, np.float32)
    assert L.b2_fill_uniform_host(buf.ctypes.data_as(C.c_void_p), 1000, 42) == 0
    assert np.array_equal(buf, oracle.fill_uniform(1000, 42))


def test_generated_tile_table_is_current_and_exported(L):
    import ctypes as C
    from hpcdeepneuralnetworks_b200 import gen_ft_sgemm
    assert gen_ft_sgemm.main(["--check"]) == 0                       # csrc/ffma_tiles.inc matches the generator
    assert L.b2_ffma_tile_count() == len(gen_ft_sgemm.TILES)
    bm, bn, th, name = C.c_int(), C.c_int(), C.c_int(), C.c_char_p()
    for i, (tname, t) in enumerate(gen_ft_sgemm.FFMA_TILES.items()):
        param = t["param"]
        assert L.b2_ffma_tile_info(i, C.byref(bm), C.byref(bn), C.byref(th), C.byref(name)) == 0
        assert (name.value.decode(), bm.value, bn.value, th.value) == (tname, param[0], param[1], 8 * param[0] // param[5])
    assert L.b2_ffma_tile_info(99, None, None, None, None) == -1
    assert L.b2_set_ffma_tile(99) == -1 and L.b2_set_ffma_tile(-1) == 0
    import pytest as _pt
    with _pt.raises(ValueError, match="ks must be 32"):
        gen_ft_sgemm.validate("small", (16, 16, 16, 8, 16, 2, 2))    # the reference's 16x16x16 tile has no B200 form
    with _pt.raises(ValueError, match="shared memory"):
        gen_ft_sgemm.derive_ffma("too_deep", (128, 128, 32, 16, 128, 4, 16), stages=8)
    with _pt.raises(ValueError, match="tensor-memory|accumulates"):
        gen_ft_sgemm.derive_tf32("too_wide", (128, 512, 32), "single")
    d = gen_ft_sgemm.derive_ffma("b200_8x16", *[gen_ft_sgemm.FFMA_TILES["b200_8x16"][k] for k in ("param", "stages")])
    assert (d["threads"], d["ctas_per_sm"], d["mr"]) == (128, 2, 8) and d["smem_bytes"] <= 113 * 1024


def test_workspace_query(L):
    assert L.b2_sgemm_workspace_bytes(0, 1024, 1024, 1024) == 0
    need = L.b2_sgemm_workspace_bytes(1, 1024, 1024, 1024)
    assert need >= 4 * 1024 * 1024 * 4


def test_partition_helpers_need_no_device(L):
    """b2_mg_row_block / b2_mg_k_panel: contiguous row blocks whose sizes differ by at most one, K panels in order."""
    start, rows = C.c_int64(), C.c_int64()
    for M in (0, 1, 7, 128, 1000, 32768):
        for world in (1, 2, 3, 8):
            seen = 0
            sizes = []
            for r in range(world):
                assert L.b2_mg_row_block(M, r, world, C.byref(start), C.byref(rows)) == 0
                assert start.value == seen
                seen += rows.value
                sizes.append(rows.value)
            assert seen == M and max(sizes) - min(sizes) <= 1
    assert L.b2_mg_row_block(10, 2, 2, C.byref(start), C.byref(rows)) == -1          # rank out of range
    k0, kw = C.c_int(), C.c_int()
    assert L.b2_mg_k_panel(0, 4096, 0, C.byref(k0), C.byref(kw)) == 0
    assert L.b2_mg_k_panel(10, 4, 2, C.byref(k0), C.byref(kw)) == 3 and (k0.value, kw.value) == (8, 2)
    assert L.b2_mg_k_panel(32768, 4096, 7, C.byref(k0), C.byref(kw)) == 8 and (k0.value, kw.value) == (28672, 4096)
    assert L.b2_mg_k_panel(5, 0, 4, C.byref(k0), C.byref(kw)) == 5 and (k0.value, kw.value) == (4, 1)   # panel < 1 means 1


def test_ffma_picker_ranks_tiles_as_measured(L):
    """b2_ffma_pick_tile: the time model (CTAs of the busiest SM at the tile's measured efficiency, occupancy penalty,
    the 8 x 16 tile from two waves on) takes, on 148 SMs, the tile that `b2_driver tiles <n>` measured fastest or within
    1.5 % of it at these sizes."""
    name = C.c_char_p()
    def pick(m, n):
        i = L.b2_ffma_pick_tile(m, n, 148)
        assert i >= 0 and L.b2_ffma_tile_info(i, None, None, None, C.byref(name)) == 0
        return name.value.decode()
    assert pick(1024, 1024) in ("large", "tall")          # 36.2 / 36.4 TFLOP/s; 128 x 128 tiles fill 64 SMs only: 20.7
    assert pick(1280, 1280) == "large"                      # 41.8 against 33 for every other tile
    assert pick(1536, 1536) == "huge"                       # 144 tiles, one per SM: 48.5
    assert pick(1792, 1792) in ("b200_64x128", "tall", "large")   # 45.6 / 45.3 / 45.0; huge: 35.6
    assert pick(2048, 2048) == "large"                      # 50.7; huge 48.5
    assert pick(2816, 2816) == "b200_64x128"                # 52.2; huge 48.0
    assert pick(3072, 3072) == "huge"                       # 57.2; the 8 x 16 tile below two waves: 55.9
    for n in (3328, 4096, 5120, 6144, 8192):
        assert pick(n, n) == "b200_8x16"
    assert pick(768, 6144) == "huge" and pick(3072, 768) in ("huge", "b200_64x128")    # panels of the host-buffer pipeline
    assert L.b2_ffma_pick_tile(0, 5, 148) < 0 and L.b2_ffma_pick_tile(5, 5, 0) < 0


def test_ffma_row_split_plan(L):
    """b2_ffma_row_split_plan: on 148 SMs the model splits 3840^2 into 29 tile rows of the 8 x 16 tile (whole SM-rounds) and
    a remainder of 128 rows on small tiles, and leaves 4096^2, 6144^2 and small outputs in one launch; the first part is
    always whole tiles of its own tile shape and smaller than M."""
    rows1, t1, t2 = C.c_int(), C.c_int(), C.c_int()
    name = C.c_char_p()
    def tile(i):
        assert L.b2_ffma_tile_info(i, None, None, None, C.byref(name)) == 0
        return name.value.decode()
    assert L.b2_ffma_row_split_plan(3840, 3840, 148, C.byref(rows1), C.byref(t1), C.byref(t2)) == 1
    assert (rows1.value, tile(t1.value)) == (3712, "b200_8x16") and tile(t2.value) in ("large", "medium", "b200_64x128")
    for n in (256, 1024, 4096, 6144, 8192):
        assert L.b2_ffma_row_split_plan(n, n, 148, C.byref(rows1), C.byref(t1), C.byref(t2)) == 0 and rows1.value == 0
    bm = C.c_int()
    for M in range(1500, 6200, 173):
        for N in (1536, 2816, 4000, 6144):
            if L.b2_ffma_row_split_plan(M, N, 148, C.byref(rows1), C.byref(t1), C.byref(t2)) == 1:
                assert L.b2_ffma_tile_info(t1.value, C.byref(bm), None, None, None) == 0
                assert 0 < rows1.value < M and rows1.value % bm.value == 0 and 0 <= t2.value < L.b2_ffma_tile_count()
    assert L.b2_ffma_row_split_plan(0, 5, 148, None, None, None) < 0
    assert L.b2_set_ffma_row_split(2) == -1 and L.b2_set_ffma_row_split(1) == 0


def test_tail_plan_of_the_3xtf32_path(L):
    """b2_tf32_tail_plan: when the tiles of the last round leave at least half of the clusters idle, each of them is cut
    into `parts` non-empty runs of whole chunks that cover the K loop once, on parts * R distinct clusters."""
    first, parts, longest = C.c_int(), C.c_int(), C.c_int()
    ref = lambda: (first.value, parts.value, longest.value)
    cases = 0
    for clusters in (74, 66, 8):
        for tiles in list(range(1, 3 * clusters + 2)) + [576, 1024]:
            for K in (1100, 2304, 4096, 8192, 16384):
                for chunk in (16, 8, 3):
                    cut = L.b2_tf32_tail_plan(tiles, clusters, K, chunk, C.byref(first), C.byref(parts), C.byref(longest))
                    nkb = (K + 31) // 32
                    nch = (nkb + chunk - 1) // chunk
                    rem = tiles % clusters
                    if not cut:
                        assert ref() == (tiles, 0, 0)
                        want = min(clusters // rem, nch) if rem else 0
                        assert want < 2 or (nch - (nch + want - 1) // want) * chunk < 16
                        continue
                    cases += 1
                    f, p, lg = ref()
                    assert f == tiles - rem and f % clusters == 0 and 2 <= p <= nch and p * rem <= clusters
                    runs = [(r * nch // p, (r + 1) * nch // p) for r in range(p)]
                    assert runs[0][0] == 0 and runs[-1][1] == nch
                    assert all(b > a for a, b in runs) and all(runs[i][1] == runs[i + 1][0] for i in range(p - 1))
                    assert max(b - a for a, b in runs) == lg and (nch - lg) * chunk >= 16
    assert cases > 1000
    # the shapes quoted in the design notes, on the 74 clusters of a B200
    assert L.b2_tf32_tail_plan(81, 74, 2304, 16, C.byref(first), C.byref(parts), C.byref(longest)) == 1 and ref() == (74, 5, 1)
    assert L.b2_tf32_tail_plan(256, 74, 4096, 16, C.byref(first), C.byref(parts), C.byref(longest)) == 1 and ref() == (222, 2, 4)
    assert L.b2_tf32_tail_plan(576, 74, 6144, 16, C.byref(first), C.byref(parts), C.byref(longest)) == 0      # 58 of 74 busy
    assert L.b2_tf32_tail_plan(4, 74, 16384, 16, None, C.byref(parts), None) == 1 and parts.value == 18
    assert L.b2_tf32_tail_plan(0, 74, 4096, 16, None, None, None) == 0 and L.b2_tf32_tail_plan(5, 74, 0, 16, None, None, None) == 0


def test_new_entry_points_validate_before_touching_a_device(L):
    null = C.c_void_p(None)
    plan = C.c_void_p()
    assert L.b2_host_plan_create(None, null, 0, 4, 4, 4, 0, 0, 0, 0) == -1                 # out is NULL
    assert L.b2_host_plan_create(C.byref(plan), null, 9, 4, 4, 4, 0, 0, 0, 0) == -1        # unknown path
    assert L.b2_host_plan_create(C.byref(plan), null, 0, -4, 4, 4, 0, 0, 0, 0) == -1       # negative dimension
    assert L.b2_host_plan_create(C.byref(plan), null, 0, 4, 4, 4, -1, 0, 0, 0) == -1       # negative panel size
    assert L.b2_sgemm_host(null, 1.0, null, 4, null, 4, 0.0, null, 4, 0, null) == -1       # plan is NULL
    assert L.b2_host_plan_destroy(null) == 0 and L.b2_mg_destroy(null) == 0
    mg = C.c_void_p()
    assert L.b2_mg_create(C.byref(mg), null, 3, 2, null) == -1                             # rank 3 of 2
    assert L.b2_mg_create(C.byref(mg), null, 0, 2, null) == -1                             # two ranks need an id
    assert L.b2_mg_sgemm(null, 0, 0, 4, 4, 4, 1.0, null, 4, null, 4, 0.0, null, 4, 0, 0, null, null) == -1
    assert L.b2_mg_sdot(null, 4, null, null, null, null, null) == -1
    assert L.b2_ft_sgemm_workspace_bytes(0, 1024, 1024, 1024) > 0                          # the checksum tables
    assert L.b2_ft_sgemm_workspace_bytes(1, 1024, 1024, 1024) == L.b2_sgemm_workspace_bytes(1, 1024, 1024, 1024)
    assert L.b2_set_tf32_abft_bias(0.5) == -1
    assert L.b2_set_tf32_tail_split(2) == -1 and L.b2_set_tf32_tail_split(1) == 0
    assert L.b2_set_tf32_fused_split(3) == -1 and L.b2_set_tf32_fused_split(1) == 0
    assert L.b2_set_tf32_chunk(5000) == -1 and L.b2_set_tf32_chunk(8) == 0 and L.b2_set_tf32_chunk(-1) == 0   # -1: default

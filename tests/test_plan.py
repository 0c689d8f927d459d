"""Host logic of the fused kernels: the tile plan covers every element exactly once, the
fast division is exact where it is used, and the lookahead rule that makes the in-kernel
wait cycle-free holds.  Runs on CPU through the planner's diagnostic entry points."""
import ctypes

import numpy as np
import pytest

from anode_b200 import _lib

FIELDS = ["regime", "vec", "cb", "units", "rows_per_tile", "piece_len", "pieces", "sample_blocks",
          "tiles_per_unit", "total_tiles", "grid", "lookahead_steps", "div_mul", "ws_lo", "ws_hi"]


def plan(d0, c, n, aligned=True, resident=592, tile_floats=8192, slack=1):
    out = (ctypes.c_uint32 * len(FIELDS))()
    rc = _lib.load().anode_gpu_batch_norm_fused_plan(d0, c, n, int(aligned), resident, tile_floats, slack, out, len(FIELDS))
    assert rc == 0
    return dict(zip(FIELDS, list(out)))


def tile(d0, c, n, t, aligned=True, resident=592, tile_floats=8192):
    out = (ctypes.c_uint64 * 8)()
    rc = _lib.load().anode_gpu_batch_norm_fused_plan_tile(d0, c, n, int(aligned), resident, tile_floats, t, out)
    assert rc == 0
    return dict(zip(["unit", "c0", "cw", "n0", "rows", "col0", "len", "base"], list(out)))


SHAPES = [(784, 64, 32), (12544, 6, 8), (3136, 8, 16), (49, 96, 64), (49, 3, 5), (1, 2, 3), (1, 1, 1),
          (117, 5, 7), (15, 260, 33), (16, 8, 4), (40800, 3, 2), (288, 4, 2), (262144, 2, 1), (49, 2048, 16),
          (500, 4, 3), (65536, 1, 2), (255, 4, 9), (511, 8, 2)]


@pytest.mark.parametrize("d0,c,n", SHAPES)
@pytest.mark.parametrize("aligned", [True, False])
def test_tiles_cover_every_element_once(d0, c, n, aligned):
    p = plan(d0, c, n, aligned, resident=64, tile_floats=2048)
    cover = np.zeros(d0 * c * n, np.int32)
    for t in range(p["total_tiles"]):
        r = tile(d0, c, n, t, aligned, resident=64, tile_floats=2048)
        assert r["unit"] == t // p["tiles_per_unit"]
        assert r["rows"] * r["len"] <= 65532
        if p["vec"] == 4:
            assert r["len"] % 4 == 0 and r["base"] % 4 == 0 and (c * d0) % 4 == 0 or r["rows"] == 1
            assert r["len"] % 4 == 0 and r["base"] % 4 == 0
        for k in range(r["rows"]):
            lo = r["base"] + k * c * d0
            cover[lo:lo + r["len"]] += 1
            # the tile stays inside its unit's channels
            first_c = (lo // d0) % c
            last_c = ((lo + r["len"] - 1) // d0) % c
            assert r["c0"] <= first_c <= last_c < r["c0"] + r["cw"]
    assert (cover == 1).all()
    if p["vec"] == 4 and p["regime"] == 1:
        assert p["cb"] * d0 <= 2048 and p["cb"] <= 256
    # wait-freedom of the pipeline: a block reduces tile i + lookahead*grid before applying tile i
    assert p["lookahead_steps"] * p["grid"] >= p["tiles_per_unit"]
    assert p["grid"] <= 64 and p["grid"] <= p["total_tiles"]


def test_benchmark_shapes_pick_the_expected_regimes():
    assert plan(12544, 64, 256)["regime"] == 0 and plan(12544, 64, 256)["vec"] == 4      # config 2
    assert plan(3136, 256, 256)["vec"] == 4                                              # config 3 / 8 GPUs
    assert plan(262144, 32, 4)["pieces"] > 1                                             # config 4 / 8 GPUs
    p5 = plan(49, 2048, 128)                                                             # config 5 / 8 GPUs
    assert p5["regime"] == 1 and p5["cb"] % 4 == 0 and p5["cb"] * 49 > 0.9 * 2048
    assert plan(49, 3, 5)["vec"] == 1                                                    # nothing aligns: scalar


def test_division_by_one_is_special_cased():
    assert plan(1, 2, 3, aligned=False)["div_mul"] == 0
    assert plan(784, 64, 32)["div_mul"] == (1 << 32) // 196 + 1


def test_fast_division_is_exact_in_its_domain():
    # q = (n * mul) >> 32 with mul = floor(2^32/d) + 1 must equal n // d for every vector index of a
    # tile: n < rows*d <= 65532
    rng = np.random.default_rng(0)
    ds = np.unique(np.concatenate([np.arange(2, 300), rng.integers(300, 65532, 400), [16383, 32766, 65532]]))
    for d in ds:
        mul = (1 << 32) // int(d) + 1
        assert mul < (1 << 32)          # fits the plan's 32-bit field (d == 1 is special-cased)
        rows = 65532 // int(d)
        n = np.arange(0, rows * int(d), dtype=np.uint64)
        if n.size > 20000:
            n = np.unique(np.concatenate([n[:5000], n[-5000:], rng.choice(n, 5000)]))
        q = (n * np.uint64(mul)) >> np.uint64(32)
        assert (q == n // np.uint64(d)).all(), d


@pytest.mark.parametrize("d0,c,n", SHAPES)
def test_division_free_walk_equals_per_tile_ranges(d0, c, n):
    """The kernels step from tile to tile with an iterator that avoids divisions; it must give
    exactly the ranges of the direct formula, for strides below and above tiles_per_unit."""
    p = plan(d0, c, n, True, resident=64, tile_floats=2048)
    total = p["total_tiles"]
    for first, stride in ((0, 1), (3, 7), (1, 64), (0, max(1, p["tiles_per_unit"] * 2 + 1)), (5, 1000)):
        if first >= total:
            continue
        count = (total - first + stride - 1) // stride
        out = (ctypes.c_uint64 * (8 * count))()
        rc = _lib.load().anode_gpu_batch_norm_fused_plan_walk(d0, c, n, 1, 64, 2048, first, stride, count, out)
        assert rc == 0
        for i in range(0, count, max(1, count // 50)):
            want = tile(d0, c, n, first + i * stride, True, resident=64, tile_floats=2048)
            got = dict(zip(["unit", "c0", "cw", "n0", "rows", "col0", "len", "base"], list(out[8 * i:8 * i + 8])))
            assert got == want, (first, stride, i)


def test_cluster_kernel_geometry_invariants():
    """Geometry of the cluster kernel for short rows (no GPU needed): a unit's runs are 16-byte
    aligned, the cluster's blocks cover all samples, the slices fit the shared memory of a block."""
    import ctypes
    from anode_b200 import _lib
    lib = _lib.load()
    cases = [(49, 2048, 1024), (49, 2048, 128), (196, 1024, 256), (15, 260, 33), (16, 8, 4), (49, 96, 64), (1, 512, 64),
             (9, 12, 7), (25, 64, 4096), (225, 4, 2)]
    for d0, c, n in cases:
        for direction in (0, 1):
            out = (ctypes.c_uint32 * 6)()
            assert lib.anode_gpu_batch_norm_segres_geometry(d0, c, n, direction, out) == 0
            ok, cb, cluster, rows, units, smem = list(out)
            kind = lib.anode_gpu_batch_norm_fused_kernel_kind(d0, c, n, direction)
            if not ok:
                assert kind in (1, 4)       # ANODE_KERNEL_TILED, ANODE_KERNEL_PLAIN
                continue
            assert kind == 2                # ANODE_KERNEL_CLUSTER
            assert (cb * d0) % 4 == 0 or cb == c
            assert cb * d0 <= 1024 and 1 <= cb <= max(c, 1)
            assert units == -(-c // cb)
            assert cluster in (1, 2, 4, 8, 16) and rows * cluster >= n and rows * (cluster - 1) < n + rows
            assert smem <= 227 * 1024
            tensors = 2 if direction else 1
            assert smem >= tensors * rows * min(cb, c) * d0 * 4
    # long aligned rows belong to the tiled kernel, odd strides to the plain one
    assert lib.anode_gpu_batch_norm_fused_kernel_kind(3136, 256, 2048, 0) == 1
    assert lib.anode_gpu_batch_norm_fused_kernel_kind(117, 5, 3, 1) == 4
    # long aligned rows whose channel fits a few blocks' shared memory: the cluster kernel takes them
    assert lib.anode_gpu_batch_norm_fused_kernel_kind(784, 64, 32, 0) == 2
    assert lib.anode_gpu_batch_norm_fused_kernel_kind(784, 2048, 1024, 0) == 1


def test_host_step_block_count_and_staging_size():
    from anode_b200 import _lib
    lib = _lib.load()
    d0, c, n = 3136, 256, 2048
    assert lib.anode_gpu_batch_norm_host_step_blocks(d0, c, n, 0) == 32          # 8 channels of 25.7 MB per block
    assert lib.anode_gpu_batch_norm_host_step_blocks(d0, c, n, 100) == 3         # 100 + 100 + 56
    assert lib.anode_gpu_batch_norm_host_step_blocks(d0, c, n, 1000) == 1
    assert lib.anode_gpu_batch_norm_host_step_blocks(0, c, n, 0) == 0
    small = lib.anode_gpu_batch_norm_host_step_staging_bytes(d0, c, n, 4)
    big = lib.anode_gpu_batch_norm_host_step_staging_bytes(d0, c, n, 8)
    assert 0 < small < big
    # three buffers of three tensors of one block each, plus the workspace
    assert big >= 9 * 8 * d0 * n * 4
    rc = lib.anode_gpu_batch_norm_relu_fused_step_host_3d1_packed_f32(d0, c, n, 1e-5, 0.1, 1, None, None, None, None, None, None,
                                                                      None, None, None, None, None, None, None, 0, 0, None, None)
    assert rc == -1


def tiled_geometry(d0, c, n, direction):
    out = (ctypes.c_uint32 * 12)()
    assert _lib.load().anode_gpu_batch_norm_tiled_geometry(d0, c, n, direction, out) == 0
    keys = ["applies", "rows", "piece", "tiles_per_unit", "slots", "slot_bytes", "smem", "window_kib", "keep_permille",
            "grid", "lookahead", "tiles"]
    return dict(zip(keys, list(out)))


def test_tiled_kernel_geometry_follows_the_window():
    """Backward pass: three slots of larger tiles while the window between a tile's two visits stays within
    what L2 keeps (48 MiB), four slots of the standard tiles beyond; and only the part of a larger window that
    fits is loaded with the keep priority.  (148 SMs are assumed where no device can be asked.)"""
    small = tiled_geometry(3136, 256, 256, 1)        # one GPU's share of config 3 at eight GPUs
    mid = tiled_geometry(3136, 256, 512, 1)
    big = tiled_geometry(3136, 256, 1024, 1)
    full = tiled_geometry(3136, 256, 2048, 1)        # config 3 on one GPU
    assert (small["rows"], small["slots"]) == (3, 3) and (mid["rows"], mid["slots"]) == (3, 3)
    assert (big["rows"], big["slots"]) == (2, 4) and (full["rows"], full["slots"]) == (2, 4)
    for g in (small, mid, big):
        assert g["window_kib"] <= 48 * 1024 and g["keep_permille"] == 1000
    assert full["window_kib"] > 48 * 1024
    assert abs(full["keep_permille"] - 1000 * 48 * 1024 / full["window_kib"]) <= 1
    # the forward pass has one geometry; everything fits the 227 KB of shared memory; short rows are not this kernel's
    for n in (256, 512, 1024, 2048):
        f = tiled_geometry(3136, 256, n, 0)
        assert (f["rows"], f["slots"]) == (5, 3) and f["smem"] <= 227 * 1024
    for g in (small, mid, big, full):
        assert g["smem"] <= 227 * 1024 and g["slots"] * g["slot_bytes"] < g["smem"]
    assert tiled_geometry(49, 2048, 1024, 0)["applies"] == 0


def simulate_tiled_schedule(tiles, per_unit, grid, look):
    """Every block walks its visits in order (reduce tile b + s*G, apply tile b + (s - look)*G); an apply visit
    can only be served once every tile of its unit has been reduced.  Returns True when all blocks finish."""
    units = tiles // per_unit
    reduced = [0] * units
    seq = []
    for b in range(grid):
        mine = range(b, tiles, grid)
        n = len(mine)
        v = []
        for s in range(n + look):
            if s < n:
                v.append((0, b + s * grid))
            if s >= look:
                v.append((1, b + (s - look) * grid))
        seq.append(v)
    pos = [0] * grid
    progress = True
    while progress:
        progress = False
        for b in range(grid):
            v = seq[b]
            while pos[b] < len(v):
                kind, t = v[pos[b]]
                u = t // per_unit
                if kind == 0:
                    reduced[u] += 1
                elif reduced[u] < per_unit:
                    break
                pos[b] += 1
                progress = True
    return all(pos[b] == len(seq[b]) for b in range(grid))


def test_tiled_schedule_cannot_wait_in_a_cycle():
    """The fixed schedule of the tiled kernel with the planner's distance between a tile's two visits, on the
    geometries the planner picks for a spread of shapes (both backward tile choices among them): a block that
    waits for a unit's statistics never holds back a reduce visit of that unit.  One step less does deadlock."""
    shapes = [(3136, 8, 64), (3136, 16, 300), (3136, 4, 2048), (12544, 6, 40), (784, 12, 256), (1024, 5, 77),
              (65536, 3, 4), (3136, 2, 1)]
    seen = set()
    for d0, c, n in shapes:
        for direction in (0, 1):
            g = tiled_geometry(d0, c, n, direction)
            if not g["applies"]:
                continue
            seen.add((g["rows"], g["slots"]))
            assert g["tiles"] % g["tiles_per_unit"] == 0 and g["lookahead"] * g["grid"] >= g["tiles_per_unit"]
            assert simulate_tiled_schedule(g["tiles"], g["tiles_per_unit"], g["grid"], g["lookahead"]), (d0, c, n, direction)
    assert len(seen) >= 3
    # what the rule guards against: with too few steps in between, blocks wait for tiles that sit behind their own
    # apply visits (a step's reduce visit comes before its apply visit, so (look + 1) * grid >= tiles per unit is
    # the exact bound; the planner asks for one step more, and for the slack on top)
    assert not simulate_tiled_schedule(tiles=8 * 40, per_unit=40, grid=8, look=3)
    assert simulate_tiled_schedule(tiles=8 * 40, per_unit=40, grid=8, look=4)

"""The C-ABI library without a GPU: it builds, loads, exports every declared symbol,
and its host-only entry points (validate / plan / workspace) behave."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

from fuseml_b200 import _native as N

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "fuseml_sm100.h").read_text()
    return sorted(set(re.findall(r"\b(fuseml_sm100_[a-z_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native_lib):
    declared = _declared_symbols()
    assert len(declared) >= 9
    for sym in declared:
        assert hasattr(native_lib, sym), f"{sym} declared in the header but not exported"
    assert set(declared) == set(N.EXPORTS)


def test_abi_version_and_strerror(native_lib):
    assert native_lib.fuseml_sm100_abi_version() == N.ABI_VERSION == 3
    assert N.strerror(0) == "ok"
    for code in range(1, 13):
        assert N.strerror(code) and "unknown" not in N.strerror(code)
    assert "unknown" in N.strerror(999)


def _desc(M=8192, Nn=16384, K=4096, ab=N.BF16, kmajor=True):
    d = N.GemmDesc()
    d.M, d.N, d.K = M, Nn, K
    d.a, d.lda = 0x10000, K
    d.b = 0x20000
    if kmajor:
        d.b_stride_k, d.b_stride_n = 1, K
    else:
        d.b_stride_k, d.b_stride_n = Nn, 1
    d.ab_dtype, d.out_dtype = ab, ab
    d.d, d.ldd = 0x30000, Nn
    return d


def test_validate_accepts_the_benchmark_shapes(native_lib):
    for (M, Nn, K, km) in [(256, 16384, 4096, False), (8192, 4096, 4096, False), (8192, 16384, 4096, True),
                           (8192, 4096, 16384, True), (128, 2048, 512, True)]:
        assert native_lib.fuseml_sm100_validate(C.byref(_desc(M, Nn, K, kmajor=km))) == N.OK


def test_validate_rejections(native_lib):
    v = native_lib.fuseml_sm100_validate
    assert v(None) == N.E_NULL
    d = _desc(); d.a = None
    assert v(C.byref(d)) == N.E_NULL
    d = _desc(K=0)
    assert v(C.byref(d)) == N.E_SHAPE
    d = _desc(); d.ab_dtype = 7
    assert v(C.byref(d)) == N.E_DTYPE
    d = _desc(); d.a = 0x10002           # not 16-byte aligned
    assert v(C.byref(d)) == N.E_LAYOUT
    d = _desc(K=100); d.lda = 100; d.b_stride_n = 100   # 200-byte rows: not a multiple of 16
    assert v(C.byref(d)) == N.E_LAYOUT
    d = _desc(); d.b_stride_k, d.b_stride_n = 3, 5      # no unit stride
    assert v(C.byref(d)) == N.E_LAYOUT
    d = _desc(); d.n_ops = 17
    assert v(C.byref(d)) == N.E_EPILOGUE
    d = _desc(); d.n_ops = 1; d.ops[0].opcode = 99
    assert v(C.byref(d)) == N.E_EPILOGUE
    d = _desc(); d.n_ops = 1; d.ops[0].opcode = N.OP_ADD_T; d.ops[0].slot = 0   # slot without operand
    assert v(C.byref(d)) == N.E_EPILOGUE
    d = _desc(); d.d = None               # nothing to produce
    assert v(C.byref(d)) == N.E_NULL
    d = _desc(); d.reduce.kinds = N.RED_SUM; d.reduce.axis = N.AXIS_N     # missing output pointer
    assert v(C.byref(d)) == N.E_NULL
    d = _desc(); d.reduce.kinds = 64
    assert v(C.byref(d)) == N.E_REDUCTION


def test_fp32_operands_have_no_tma_layout_rule(native_lib):
    d = _desc(M=128, Nn=2048, K=510, ab=N.F32)
    d.lda = 510
    d.b_stride_n = 510
    assert native_lib.fuseml_sm100_validate(C.byref(d)) == N.OK


def _plan(native_lib, d, props=None):
    p = N.Plan()
    rc = native_lib.fuseml_sm100_plan(C.byref(d), C.byref(props) if props is not None else None, C.byref(p))
    return rc, p


def test_plan_budgets_and_bounds(native_lib):
    # compute-bound MLP GEMM: tensor-bound, CTA pairs on 256 x 256 tiles, 6 stages of 32 KB per
    # CTA, both TMEM buffers
    rc, p = _plan(native_lib, _desc(8192, 16384, 4096))
    assert rc == N.OK and p.fuse == 1
    assert (p.tile_m, p.tile_n, p.tile_k, p.cluster) == (128, 256, 64, 2)
    assert p.stages == 6 and p.tmem_cols == 512 and p.acc_stages == 2
    assert p.smem_bytes <= 232448
    assert p.grid == 148 and p.bound == 1
    assert p.flops == 2.0 * 8192 * 16384 * 4096
    assert p.t_tensor_us > p.t_hbm_us
    # weight-streaming shape: HBM-bound
    rc, p = _plan(native_lib, _desc(256, 16384, 4096, kmajor=False))
    assert rc == N.OK and p.bound == 0 and p.t_hbm_us > p.t_tensor_us
    # tiny problem: latency-bound, still fused (single tier: no bypass)
    rc, p = _plan(native_lib, _desc(128, 512, 2048))
    # one row of tiles and 32 K blocks: full-width tiles whose K loop is split over 4 CTAs each
    # (partials in the workspace); a short K loop is only narrowed (32 columns, one tile per CTA)
    assert rc == N.OK and p.bound == 2 and p.fuse == 1 and p.cluster == 1
    assert (p.tile_n, p.split_k, p.grid) == (256, 4, 8)
    d = _desc(128, 512, 2048)
    assert native_lib.fuseml_sm100_workspace_bytes(C.byref(d), C.byref(p)) == 4 * 128 * 512 * 4
    rc, p = _plan(native_lib, _desc(128, 512, 256))
    assert rc == N.OK and (p.tile_n, p.split_k, p.grid) == (32, 1, 16)


def test_plan_rasterisation_groups(native_lib):
    """Groups of tile rows whose A slab stays within 32 MiB, or, with more tile rows than tile
    columns, bands of tile columns whose B slab does; with a long K loop (slabs of 8.4 MB)
    square waves instead."""
    for (M, Nn, K), gm, band in (((8192, 16384, 4096), 16, False), ((8192, 4096, 4096), 16, True),
                                 ((16384, 4096, 8192), 8, True), ((256, 16384, 4096), 1, False),
                                 ((8192, 4096, 16384), 8, True), ((32768, 4096, 16384), 8, True),
                                 ((4096, 4096, 16384), 8, False), ((8192, 8192, 8192), 8, False),
                                 ((2048, 4096, 16384), 4, False)):
        rc, p = _plan(native_lib, _desc(M, Nn, K))
        assert rc == N.OK and p.group_m == gm and bool(p.flags & N.PLAN_GROUP_N) == band, (M, Nn, K, p.group_m, p.flags)


def test_plan_follows_device_props(native_lib):
    props = N.DeviceProps()
    native_lib.fuseml_sm100_query(C.byref(props))   # fills B200 defaults when there is no device
    assert props.sm_count >= 1 and props.tmem_cols == 512
    props.sm_count = 64
    rc, p = _plan(native_lib, _desc(8192, 16384, 4096), props)
    assert rc == N.OK and p.grid == 64
    props.smem_per_block_optin = 120 * 1024
    rc, p = _plan(native_lib, _desc(8192, 16384, 4096), props)
    assert p.stages == 3 and p.smem_bytes <= 120 * 1024


def test_plan_reports_unsupported_layout_without_fusing(native_lib):
    d = _desc(); d.b_stride_k, d.b_stride_n = 3, 5
    rc, p = _plan(native_lib, d)
    assert rc == N.E_LAYOUT and p.fuse == 0


def test_workspace_bytes(native_lib):
    w = native_lib.fuseml_sm100_workspace_bytes
    assert w(C.byref(_desc()), None) == 0
    d = _desc(8192, 4096, 4096, kmajor=False)
    d.d = None
    d.reduce.kinds = N.RED_MAX | N.RED_MEAN
    d.reduce.axis = N.AXIS_N
    d.reduce.out_max = 0x40000
    d.reduce.out_mean = 0x50000
    # 16 column tiles x 2 epilogue warps per row x 8192 rows x 4 bytes, two partial arrays
    assert w(C.byref(d), None) == 2 * 16 * 2 * 8192 * 4
    d32 = _desc(128, 2048, 512, ab=N.F32)
    ld = 3 * 512
    # the two expanded operands, plus 6 K slices' worth of fp32 partial tiles (48 K blocks, 8 per slice)
    assert w(C.byref(d32), None) == (128 * ld + 2048 * ld) * 4 + 6 * 128 * 2048 * 4


def test_a_zeroed_or_garbage_plan_is_a_status_code_not_a_crash(native_lib):
    """A caller's plan is checked before any arithmetic divides by its tile shape: a zeroed plan
    with a reduction (or a split K loop) must come back as FUSEML_E_PLAN / -1."""
    d = _desc(8192, 4096, 4096, kmajor=False)
    d.reduce.kinds = N.RED_SUM
    d.reduce.axis = N.AXIS_N
    d.reduce.out_sum = 0x40000
    zero = N.Plan()
    assert native_lib.fuseml_sm100_workspace_bytes(C.byref(d), C.byref(zero)) == -1
    # both launch entries reject it on the host, before any CUDA call is made
    assert native_lib.fuseml_sm100_gemm_epilogue(C.byref(d), C.byref(zero), None) == N.E_PLAN
    assert native_lib.fuseml_sm100_gemm_epilogue_noalloc(C.byref(d), C.byref(zero), None) == N.E_PLAN
    rc, good = _plan(native_lib, d)
    assert rc == N.OK
    for field, value in (("tile_n", 0), ("tile_n", 48), ("tile_m", 64), ("grid", 0), ("group_m", 0), ("cluster", 3),
                         ("split_k", 65), ("flags", 8)):
        bad = N.Plan.from_buffer_copy(good)
        setattr(bad, field, value)
        assert native_lib.fuseml_sm100_workspace_bytes(C.byref(d), C.byref(bad)) == -1, field
        assert native_lib.fuseml_sm100_gemm_epilogue_noalloc(C.byref(d), C.byref(bad), None) == N.E_PLAN, field


def _schedule(native_lib, d, p):
    """Every unit's work items: {unit: [WorkItem, ...]}."""
    n_units = C.c_int32(0)
    buf = (N.WorkItem * 64)()
    out = {}
    n = native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(p), 0, buf, 64, C.byref(n_units))
    assert n >= 0
    for u in range(n_units.value):
        n = native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(p), u, buf, 64, None)
        assert 0 <= n <= 64
        out[u] = [N.WorkItem.from_buffer_copy(buf[i]) for i in range(n)]
    return out


@pytest.mark.parametrize("M,Nn,K,grid", [
    (4096, 4096, 16384, 148),     # 256 tiles on 74 pairs: 34 left, two equal K slices each
    (1024, 4096, 16384, 148),     # 64 tiles: no whole wave, 10 helper pairs take the K tails
    (2048, 4096, 16384, 148),     # 128 tiles: one whole wave, then 54 owners and 20 helpers
    (8192, 4096, 16384, 148),     # 512 tiles: 68 left, 6 helpers
    (600, 1000, 4096, 10),        # 12 tiles on 5 pairs, ragged edges
    (520, 1100, 2048, 14),        # 15 tiles on 7 pairs: 1 left, seven slices
    (2048, 2048, 1024, 18),       # 64 tiles on 9 pairs: 1 left, 16 K blocks in 8 slices
    (1280, 256, 64 * 7, 16),      # 5 tiles on 8 pairs, 7 K blocks: runs of helpers end early
    (1536, 256, 64 * 3, 16),      # 6 tiles on 8 pairs, 3 K blocks: nothing left over, whole tiles
    (256, 256 * 9, 64 * 40, 20),  # 9 tiles on 10 pairs: one helper adds to every tile
])
def test_k_split_schedule_covers_every_k_block_once(native_lib, M, Nn, K, grid):
    """The walk the kernel runs, executed on the host: with FUSEML_PLAN_STREAM_K every K block of
    every tile belongs to exactly one work item, each tile has exactly one finishing item, the
    workspace slots of the later parts are distinct, lie inside the workspace, and are exactly the
    ones the finishing item of their tile reads; units carry about the same number of K blocks."""
    d = _desc(M, Nn, K)
    rc, p = _plan(native_lib, d)
    assert rc == N.OK and p.cluster == 2
    p.grid = grid
    p.flags |= N.PLAN_STREAM_K
    units = grid // 2
    tiles = -(-M // 256) * -(-Nn // p.tile_n)
    num_kb = -(-K // 64)
    sched = _schedule(native_lib, d, p)
    assert len(sched) == units
    cover = {t: [0] * num_kb for t in range(tiles)}
    finishers, parts, load, halves = {}, {}, [], {}
    for u, items in sched.items():
        load.append(sum(w.kb1 - w.kb0 for w in items))
        for w in items:
            assert 0 <= w.tile < tiles and 0 <= w.kb0 < w.kb1 <= num_kb and w.kind in (0, 1, 2, 4)
            for kb in range(w.kb0, w.kb1):
                cover[w.tile][kb] += 1
            if w.kind == 4:
                # two units exchange halves: each writes its own slot and reads the partner's
                assert 0 <= w.slot < units and 0 <= w.after < units and w.slot != w.after
                halves.setdefault(w.tile, []).append(w)
            elif w.kind == 2:
                assert 0 <= w.slot < units and w.slot not in parts
                parts[w.slot] = w.tile
            else:
                assert w.tile not in finishers
                finishers[w.tile] = w
                assert (w.kind == 0) == (w.after == 0) and (w.kind == 0) <= (w.kb1 - w.kb0 == num_kb)
    assert all(c == [1] * num_kb for c in cover.values())
    for t, (a, b) in halves.items():
        assert t not in finishers and {a.kb0, b.kb0} == {0, a.kb1 if a.kb0 == 0 else b.kb1}    # left finisher, right finisher
        assert (a.slot, a.after) == (b.after, b.slot) and a.slot not in parts and b.slot not in parts
    assert all(len(v) == 2 for v in halves.values())
    assert sorted(list(finishers) + list(halves)) == list(range(tiles))
    read = {}
    for t, w in finishers.items():
        for s in range(w.slot, w.slot + w.after):
            assert s not in read
            read[s] = t
    assert read == parts
    whole = tiles // units * num_kb
    rem = tiles % units
    if rem == 0:
        last = 0
    elif rem <= units // 2:
        last = -(-num_kb // (units // rem))                       # equal slices
    else:
        last = num_kb - num_kb * (units - rem) * 3 // (units * 4)  # an owner's part; helpers' runs are no longer
    assert max(load) - whole <= last
    ws = native_lib.fuseml_sm100_workspace_bytes(C.byref(d), C.byref(p))
    assert ws >= grid * 128 * 256 * 4 + grid * 4
    # without the flag: whole tiles only, unit u takes tiles u, u + units, ...
    p.flags &= ~N.PLAN_STREAM_K
    plain = _schedule(native_lib, d, p)
    assert all(w.kind == 0 and w.tile % len(plain) == u for u, items in plain.items() for w in items)
    assert sum(len(v) for v in plain.values()) == tiles


@pytest.mark.parametrize("M,Nn,band,group", [(1500, 2300, False, 4), (1500, 2300, True, 4), (1500, 2300, True, 3),
                                             (8192, 4096, True, 8), (8192, 4096, False, 16), (700, 5000, True, 64),
                                             (5000, 700, False, 64), (300, 300, True, 1)])
def test_rasterisation_visits_every_tile_position_once(native_lib, M, Nn, band, group):
    """Tile index -> (tile row, tile column) is a bijection in both walks (groups of tile rows,
    bands of tile columns), ragged last group or band included, and consecutive tiles stay inside
    one group or band until it is exhausted."""
    d = _desc(M, Nn, 4096)
    rc, p = _plan(native_lib, d)
    assert rc == N.OK
    p.group_m = group
    p.flags = (p.flags | N.PLAN_GROUP_N) if band else (p.flags & ~N.PLAN_GROUP_N)
    p.flags &= ~N.PLAN_STREAM_K
    rows = -(-M // (128 * p.cluster))
    cols = -(-Nn // p.tile_n)
    p.grid = p.cluster * min(rows * cols, 74 if p.cluster == 2 else 148)
    sched = _schedule(native_lib, d, p)
    by_tile = {w.tile: (w.tile_m, w.tile_n) for items in sched.values() for w in items}
    assert sorted(by_tile) == list(range(rows * cols))
    assert sorted(by_tile.values()) == [(r, c) for r in range(rows) for c in range(cols)]
    order = [by_tile[t] for t in range(rows * cols)]
    keys = [(c // group) if band else (r // group) for r, c in order]
    assert keys == sorted(keys)                       # one group / band after the other
    first = [rc_ for rc_, k in zip(order, keys) if k == 0]
    inner = [c for _, c in first] if band else [r for r, _ in first]
    width = min(group, cols if band else rows)
    assert inner[:width] == list(range(width))        # the grouped index runs fastest


def test_two_slice_tiles_are_exchanged_unless_a_reduction_is_fused(native_lib):
    """Two K slices per last-wave tile: the two units exchange halves (kind 4) so that each
    publishes and finishes half a tile; with a fused reduction (whose partials are laid out per
    finishing warp) the first unit finishes the whole tile as with any other slice count."""
    d = _desc(4096, 4096, 16384)
    rc, p = _plan(native_lib, d)
    assert rc == N.OK and p.flags & N.PLAN_STREAM_K
    kinds = sorted({w.kind for items in _schedule(native_lib, d, p).values() for w in items})
    assert kinds == [0, 4]
    d.reduce.kinds = N.RED_SUM
    d.reduce.axis = N.AXIS_N
    d.reduce.out_sum = 0x40000
    p.flags |= N.PLAN_STREAM_K
    kinds = sorted({w.kind for items in _schedule(native_lib, d, p).values() for w in items})
    assert kinds == [0, 1, 2]


def test_saved_register_programs_keep_whole_tiles(native_lib):
    """A program that keeps a second value register runs in a kernel instance without the K-split
    walk: the flag is ignored and the schedule says so.  The gelu*sigmoid diamond is rewritten to
    one op first and does not count."""
    d = _desc(4096, 4096, 16384)
    rc, p = _plan(native_lib, d)
    assert rc == N.OK and p.flags & N.PLAN_STREAM_K          # 256 tiles, 34 left, 256 K blocks
    assert any(w.kind != 0 for items in _schedule(native_lib, d, p).values() for w in items)
    for i, oc in enumerate((N.OP_SAVE, N.OP_RELU, N.OP_ADD_SAVED)):
        d.ops[i].opcode = oc
    d.n_ops = 3
    sched = _schedule(native_lib, d, p)
    assert all(w.kind == 0 for items in sched.values() for w in items)
    assert sum(len(v) for v in sched.values()) == 256
    for i, oc in enumerate((N.OP_SAVE, N.OP_GELU_ERF, N.OP_SWAP, N.OP_SIGMOID, N.OP_MUL_SAVED)):
        d.ops[i].opcode = oc
    d.n_ops = 5
    assert any(w.kind != 0 for items in _schedule(native_lib, d, p).values() for w in items)


def test_schedule_of_a_split_k_plan_and_bad_arguments(native_lib):
    d = _desc(128, 512, 2048)
    rc, p = _plan(native_lib, d)
    assert rc == N.OK and p.split_k == 4
    sched = _schedule(native_lib, d, p)
    assert len(sched) == 2 * 4                        # two 256-column tiles, four K slices each
    assert sorted((w.tile, w.kb0, w.kb1) for items in sched.values() for w in items) == \
        [(t, 8 * s, 8 * s + 8) for t in range(2) for s in range(4)]
    assert all(len(items) == 1 and items[0].kind == 3 for items in sched.values())
    buf = (N.WorkItem * 1)()
    assert native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(p), 8, buf, 1, None) == -N.E_PLAN
    assert native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(p), -1, buf, 1, None) == -N.E_PLAN
    assert native_lib.fuseml_sm100_schedule(C.byref(d), None, 0, buf, 1, None) == -N.E_NULL
    assert native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(N.Plan()), 0, buf, 1, None) == -N.E_PLAN
    assert native_lib.fuseml_sm100_schedule(C.byref(d), C.byref(p), 0, None, 0, None) == 1   # count only


def test_struct_layout_matches_header():
    assert C.sizeof(N.EpiOp) == 16
    assert C.sizeof(N.Operand) == 32
    assert C.sizeof(N.Reduce) == 48
    assert C.sizeof(N.GemmDesc) == 664
    assert C.sizeof(N.Plan) == 96
    assert C.sizeof(N.DeviceProps) == 40


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(N.NativeLibraryError):
        N.load(tmp_path / "nope.so")


def test_cpu_tensors_are_rejected_not_emulated(native_lib):
    import torch
    from fuseml_b200.kernels import fused_gemm

    with pytest.raises(RuntimeError):
        fused_gemm(torch.zeros(128, 64, dtype=torch.bfloat16), torch.zeros(64, 256, dtype=torch.bfloat16))

"""Multi-GPU host logic on CPU: core slices, per-rank plans (plan-only device), slab exchange over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import Session
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.runtime import PlanOnlyDevice
from ktir_cpu_b200.sharded import broadcast_slabs, check_disjoint, core_slice, exchange


def _plan(src, fn, tensors, rank, world, scalars=None):
    func = KTIRParser().parse_module(src).get_function(fn)
    return Session(PlanOnlyDevice(), func, tensors, scalars or {}, shard=(rank, world), arena_ptr=0)


def test_core_slices_cover_the_grid():
    for n in (1, 7, 32, 64):
        for world in (1, 2, 3, 8):
            sl = [core_slice(n, r, world) for r in range(world)]
            assert sl[0][0] == 0 and sl[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
            assert max(h - l for l, h in sl) - min(h - l for l, h in sl) <= 1
    with pytest.raises(ValueError):
        core_slice(8, 2, 2)


@pytest.mark.parametrize("world", [2, 4])
def test_softmax_slabs_are_contiguous_row_ranges(world):
    rows, cols = 256, 512
    t = [("output_ptr", (rows, cols), np.dtype(np.float16)), ("input_ptr", (rows, cols), np.dtype(np.float16))]
    full = _plan(K.softmax_rows(rows, cols, 8, 4, True), "softmax_kernel", t, 0, 1).written_ranges()
    assert len(full) == 1 and full[0][1] - full[0][0] == rows * cols * 2
    per_rank = [_plan(K.softmax_rows(rows, cols, 8, 4, True), "softmax_kernel", t, r, world).written_ranges()
                for r in range(world)]
    check_disjoint(per_rank)
    assert all(len(r) == 1 for r in per_rank)
    assert per_rank[0][0][0] == full[0][0] and per_rank[-1][0][1] == full[0][1]
    assert all(a[0][1] == b[0][0] for a, b in zip(per_rank, per_rank[1:]))


def test_matmul_slabs_partition_c():
    t = [(n, (256, 256), np.dtype(np.float16)) for n in ("a_ptr", "b_ptr", "c_ptr")]
    src = K.tiled_matmul(256, 256, 256, 64, 64, 64, 4, True)
    per_rank = [_plan(src, "matmul_kernel", t, r, 2).written_ranges() for r in range(2)]
    check_disjoint(per_rank)
    assert sum(h - l for rs in per_rank for l, h in rs) == 256 * 256 * 2


def test_ordered_scatter_is_split_by_destination_rows():
    n_rows, n_idx = 1024, 4096
    t = [("table_ptr", (n_rows, 128), np.dtype(np.float16)), ("idx_ptr", (n_idx,), np.dtype(np.int32)),
         ("out_ptr", (n_rows, 128), np.dtype(np.float16))]
    src = K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8)
    sessions = [_plan(src, "gather_scale_scatter", t, r, 4) for r in range(4)]
    per_rank = [s.written_ranges() for s in sessions]
    check_disjoint(per_rank)
    assert [h - l for rs in per_rank for l, h in rs] == [n_rows // 4 * 128 * 2] * 4
    # every rank still walks every tile (order between cores matters), but owns a quarter of the rows
    for s in sessions:
        (stmt,) = s.plan.statements
        assert stmt.args.n_tiles == n_idx // 64 and stmt.args.dst_rows == n_rows // 4


def test_regular_fragments_are_recognised():
    from ktir_cpu_b200.sharded import _regular
    assert _regular([(100 + 64 * i, 132 + 64 * i) for i in range(10)]) == (100, 32, 64, 10)
    assert _regular([(0, 32), (64, 96)]) is None
    assert _regular([(64 * i, 64 * i + (32 if i != 3 else 16)) for i in range(8)]) is None


def test_overlapping_slabs_are_rejected():
    with pytest.raises(ValueError, match="both write"):
        check_disjoint([[(0, 128)], [(64, 256)]])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 64, 256
        t = [("output_ptr", (rows, cols), np.dtype(np.float16)), ("input_ptr", (rows, cols), np.dtype(np.float16))]
        sess = _plan(K.softmax_rows(rows, cols, 4, 4, True), "softmax_kernel", t, rank, world)
        arena = torch.zeros(sess.arena_bytes, dtype=torch.uint8)
        mine = sess.written_ranges()
        for lo, hi in mine:                      # stand-in for this rank's launches: mark its slab
            arena[lo:hi] = rank + 1
        all_ranges = exchange(arena, mine, dist)
        off, nbytes, _, _ = sess.layout["output_ptr"]
        got = arena[off:off + nbytes].numpy().copy()
        want = np.concatenate([np.full(hi - lo, r + 1, np.uint8) for r, rs in enumerate(all_ranges) for lo, hi in rs])
        ok = bool((got == want).all()) and int(arena[:off].sum()) == 0
        # a second step reuses the slab lists (no object collective)
        arena[off:off + nbytes] = 0
        for lo, hi in mine:
            arena[lo:hi] = 10 + rank
        broadcast_slabs(arena, all_ranges, dist)
        ok = ok and sorted(set(arena[off:off + nbytes].tolist())) == [10 + r for r in range(world)]
        # strided fragments (a column block per rank of a [16, 64]-byte matrix)
        m = torch.zeros(16 * 64, dtype=torch.uint8)
        frag = [[(r * 32 + 64 * i, r * 32 + 32 + 64 * i) for i in range(16)] for r in range(world)]
        m.view(16, 64)[:, rank * 32:(rank + 1) * 32] = 50 + rank
        broadcast_slabs(m, frag, dist)
        ok = ok and all(bool((m.view(16, 64)[:, r * 32:(r + 1) * 32] == 50 + r).all()) for r in range(world))
        out[rank] = ok
    finally:
        dist.destroy_process_group()


def test_slab_exchange_over_gloo_world2():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


SHIFT = """module {
  func.func @shift(%x_ptr: index) attributes {grid = [4, 1]} {
    %c = ktdp.get_compute_tile_id : index
    %c1 = arith.constant 1 : index
    %c4 = arith.constant 4 : index
    %blk = arith.constant 64 : index
    %n1 = arith.addi %c, %c1 : index
    %nb = arith.remui %n1, %c4 : index
    %src = arith.muli %nb, %blk : index
    %dst = arith.muli %c, %blk : index
    %v = ktdp.construct_memory_view %x_ptr, sizes: [256], strides: [1] {
      coordinate_set = affine_set<(d0) : (d0 >= 0, -d0 + 255 >= 0)>, memory_space = #ktdp.memory_space<global>
    } : memref<256xf16>
    %rt = ktdp.construct_access_tile %v[%src] {
      access_tile_set = affine_set<(d0) : (d0 >= 0, -d0 + 63 >= 0)>, access_tile_order = affine_map<(d0) -> (d0)>
    } : memref<256xf16> -> !ktdp.access_tile<64xindex>
    %wt = ktdp.construct_access_tile %v[%dst] {
      access_tile_set = affine_set<(d0) : (d0 >= 0, -d0 + 63 >= 0)>, access_tile_order = affine_map<(d0) -> (d0)>
    } : memref<256xf16> -> !ktdp.access_tile<64xindex>
    %t = ktdp.load %rt : !ktdp.access_tile<64xindex> -> tensor<64xf16>
    ktdp.store %t, %wt : tensor<64xf16>, !ktdp.access_tile<64xindex>
    return
  }
}
"""


def test_cross_rank_read_after_write_is_rejected():
    """Core c reads the block core c+1 writes: the sequential core order matters.  One GPU runs the
    cores one group after the other; across ranks there is no such order, and inside one rank's slice
    nothing clashes (with one core per rank there is no second core at all), so the whole grid has to
    be checked."""
    from ktir_cpu_b200.trace import Unsupported
    t = [("x_ptr", (256,), np.dtype(np.float16))]
    assert _plan(SHIFT, "shift", t, 0, 1).plan.core_groups == [(0, 1), (1, 2), (2, 3), (3, 4)]
    for rank in range(4):
        with pytest.raises(Unsupported, match="sequential core order"):
            _plan(SHIFT, "shift", t, rank, 4)


def test_a_rank_moves_only_its_own_slabs():
    rows, cols = 4096, 4096
    t = [("output_ptr", (rows, cols), np.dtype(np.float16)), ("input_ptr", (rows, cols), np.dtype(np.float16))]
    s = _plan(K.softmax_rows(rows, cols, 32, 8, True), "softmax_kernel", t, 1, 4)
    tp = s.transfer_plan()
    assert tp.partial and tp.host_only == []
    assert tp.h2d_bytes == tp.d2h_bytes == rows * cols * 2 // 4
    in_off = s.layout["input_ptr"][0]
    lo = min(r.off for c in tp.chunks for r in c.uploads)
    assert lo == in_off + rows * cols * 2 // 4          # rank 1 starts at its first row
    sc = _plan(K.gather_scale_scatter(1024, 128, 16384, 64, 8), "gather_scale_scatter",
               [("table_ptr", (1024, 128), np.dtype(np.float16)), ("idx_ptr", (16384,), np.dtype(np.int32)),
                ("out_ptr", (1024, 128), np.dtype(np.float16))], 2, 4)
    tps = sc.transfer_plan()
    assert not tps.split and tps.d2h_bytes == 1024 * 128 * 2 // 4       # only the destination rows it owns come back

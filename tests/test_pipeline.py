"""Transfer plans of pipelined execution (host logic, plan-only device): every byte a kernel reads
is uploaded exactly once before the part that needs it, every byte it writes is read back."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import runtime as R
from ktir_cpu_b200.interpreter import Session
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.pipeline import Region, TransferPlan, merge_intervals, tile_regions

F16, I32 = np.dtype(np.float16), np.dtype(np.int32)


@pytest.fixture(autouse=True)
def small_parts(monkeypatch):
    """4 MiB per part instead of the default, so that modest sizes split into several parts."""
    monkeypatch.setattr(Session, "PIPELINE_PIECE", 4 << 20)


def _session(src, fn, tensors, scalars=None):
    f = KTIRParser().parse_module(src).get_function(fn)
    return Session(R.PlanOnlyDevice(), f, tensors, scalars or {})


def _mark(mask, r: Region):
    for row in range(r.height):
        a = r.off + row * (r.pitch or r.width)
        mask[a:a + r.width] += 1


def _check(sess, expect_split=True):
    tp = sess.transfer_plan()
    assert tp.split == expect_split
    size = max(off + nb for off, nb in tp.tensors.values())
    up, seen_before = np.zeros(size, np.int16), np.zeros(size, np.int16)
    down = np.zeros(size, np.int16)
    for c in tp.chunks:
        for r in c.uploads:
            _mark(up, r)
        for r in c.reads:                       # everything a part reads is on the device by then
            if tp.owner(r) in tp.no_upload:
                continue
            m = np.zeros(size, np.int16)
            _mark(m, r)
            assert (up[m > 0] == 1).all()
        for r in c.writes:
            _mark(down, r)
    assert up.max() <= 1                        # nothing is sent twice
    for name, (off, nb) in tp.tensors.items():
        sl = slice(off, off + nb)
        if name in tp.no_upload or name in tp.host_only:
            assert not up[sl].any()
        else:
            assert up[sl].all(), name            # the caller's copy is complete
        if name in sess.written:
            assert down[sl].all() if name in tp.no_upload else down[sl].any()
        else:
            assert not down[sl].any()
    return tp


def test_interval_helpers():
    assert merge_intervals(np.array([10, 0, 4]), np.array([12, 4, 8])) == [(0, 8), (10, 12)]
    r = tile_regions(np.array([0, 64, 128]), 2, 32, 32, 2)
    assert r == [Region(0, 384)]
    assert tile_regions(np.arange(64) * 1024, 1, 8, 8, 2, limit=8) is None


def test_softmax_splits_into_row_ranges():
    sess = _session(K.softmax_rows(2048, 4096, 32, 8, True), "softmax_kernel",
                    [("output_ptr", (2048, 4096), F16), ("input_ptr", (2048, 4096), F16)])
    tp = _check(sess)
    assert len(tp.chunks) == 8 and tp.h2d_bytes == tp.d2h_bytes == 2048 * 4096 * 2
    assert all(len(c.uploads) == 1 and len(c.writes) == 1 for c in tp.chunks)


def test_vector_add_splits_and_small_plans_run_as_one_part():
    n = 1 << 22
    sess = _session(K.vector_add(n, 16384, 32), "add_kernel",
                    [("x_ptr", (n,), F16), ("y_ptr", (n,), F16), ("output_ptr", (n,), F16)], {"BLOCK_SIZE": 16384})
    _check(sess)
    small = _session(K.vector_add(4096, 128, 32), "add_kernel",
                     [("x_ptr", (4096,), F16), ("y_ptr", (4096,), F16), ("output_ptr", (4096,), F16)], {"BLOCK_SIZE": 128})
    assert len(_check(small).chunks) == 1          # one part, still only the regions the kernel touches


def test_matmul_splits_into_row_blocks_with_b_first():
    M = 2048
    sess = _session(K.tiled_matmul(M, M, M, 64, 64, 64, 32, True), "matmul_kernel",
                    [("a_ptr", (M, M), F16), ("b_ptr", (M, M), F16), ("c_ptr", (M, M), F16)])
    tp = _check(sess)
    b_off, b_bytes = tp.tensors["b_ptr"]
    assert Region(b_off, b_bytes) in tp.chunks[0].uploads
    assert all(Region(b_off, b_bytes) not in c.uploads for c in tp.chunks[1:])


@pytest.mark.parametrize("H,Hkv", [(16, 16), (16, 4)])
def test_attention_splits_into_head_groups(H, Hkv):
    S, T, D = 1024, 128, 128
    nt = S // T
    sess = _session(K.paged_attention(S, S, H, Hkv, D, T, T // (H // Hkv)), "paged_attention_kernel",
                    [("output_ptr", (S, H, D), F16), ("query_ptr", (S, H, D), F16), ("key_cache_ptr", (nt, T, Hkv, D), F16),
                     ("value_cache_ptr", (nt, T, Hkv, D), F16), ("block_tables_ptr", (1, nt), I32)],
                    dict(cur_batch_start_index=0, block_table_offset=0, num_tiles=nt, context_len=0, scale=np.float32(0.1)))
    tp = _check(sess)
    assert len(tp.chunks) > 1 and all(r.height == S for c in tp.chunks for r in c.writes)


def test_unsplittable_plan_moves_whole_tensors_and_skips_untouched_uploads():
    src = K.gather_scale_scatter(4096, 128, 16384, 64, 4)
    sess = _session(src, "gather_scale_scatter",
                    [("table_ptr", (4096, 128), F16), ("idx_ptr", (16384,), I32), ("out_ptr", (4096, 128), F16)])
    tp = _check(sess, expect_split=False)
    assert len(tp.chunks) == 1 and tp.d2h_bytes == 4096 * 128 * 2


def test_partial_coverage_falls_back_to_a_whole_upload():
    tensors = {"x": (0x10000, 4096), "y": (0x10000 + 4096, 4096)}
    from ktir_cpu_b200.pipeline import Chunk
    chunks = [Chunk(None, [Region(0x10000, 1024)], [Region(0x10000 + 4096, 1024)]),
              Chunk(None, [Region(0x10000 + 2048, 1024)], [Region(0x10000 + 4096 + 1024, 1024)])]
    tp = TransferPlan(tensors, ["y"], [], chunks)
    assert tp.chunks[0].uploads[0] == Region(0x10000, 4096) and tp.chunks[1].uploads == []
    assert tp.host_only == ["y"]            # y is partly written and never read: the copy fills the rest

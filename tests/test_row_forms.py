"""Row addressing the planner hands to the row gather kernel (host logic, no GPU): the per-tile
bases, index offsets and strides of a RowsStatement are replayed in NumPy for a plain copy and
compared with the fancy-indexed gather the reference computes (ktir_cpu/ops/memory_ops.py:488-576)."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import runtime as R
from ktir_cpu_b200.interpreter import Session, arena_layout
from ktir_cpu_b200.parser import KTIRParser


class RecordingDevice(R.PlanOnlyDevice):
    """upload() keeps the host array and returns a handle the test can resolve."""

    def __init__(self):
        self.arrays = {}

    def upload(self, arr) -> int:
        h = 0x1000 + 16 * len(self.arrays)
        self.arrays[h] = np.array(arr, copy=True)
        return h


def replay_rows(stmt, dev, arena_bytes):
    """What ktb_rows_program_kernel computes for a one-input copy: row (t, pos) of the destination
    takes `cols` elements from the row of the input its base, lookups and strides address."""
    a = stmt.args
    src, dst = a.inp[0], a.out
    assert a.n_in == 1 and src.dtype == dst.dtype == R.DTYPE_CODE["f16"]
    data = arena_bytes.view(np.float16)
    ints = {R.DTYPE_CODE["i32"]: arena_bytes.view(np.int32), R.DTYPE_CODE["i64"]: arena_bytes.view(np.int64)}

    def rows_of(op):
        t = np.arange(a.n_tiles)[:, None]
        pos = np.arange(a.tile_rows)[None, :]
        addr = dev.arrays[op.dev_base][t] + pos * op.pos_stride
        if op.indirect >= 1:
            addr = addr + ints[op.idx_dtype][dev.arrays[op.dev_idx_off][t] + pos * op.idx_stride].astype(np.int64) * op.idx_mult
        if op.indirect >= 2:
            addr = addr + ints[op.idx2_dtype][dev.arrays[op.dev_idx2_off][t] + pos * op.idx2_stride].astype(np.int64) * op.idx2_mult
        return addr.reshape(-1)

    s, d = rows_of(src), rows_of(dst)
    assert s.min() >= src.lo and s.max() + a.cols <= src.hi and d.min() >= dst.lo and d.max() + a.cols <= dst.hi
    c = np.arange(a.cols)[None, :]
    data[d[:, None] + c] = data[s[:, None] + c]


@pytest.mark.parametrize("shape,sel", [((40, 24, 64), (3, 5)), ((12, 10, 6, 32), (4, 3)), ((9, 7, 5, 3, 16), (2, 3)),
                                        ((32, 4, 64, 64), (3,)), ((64, 96, 128), (5,)), ((6, 5, 1024), (3, 2)),
                                        ((6, 5, 8), (6, 5))])
def test_block_gather_row_addressing(shape, sel):
    rng = np.random.default_rng(5)
    rshape = tuple(sel) + tuple(shape[len(sel):])
    kw = {"src_ptr": rng.standard_normal(shape).astype(np.float16)}
    for i, n in enumerate(sel):
        kw[f"idx{i}_ptr"] = rng.choice(shape[i], n, replace=False).astype(np.int32)
    kw["out_ptr"] = np.zeros(rshape, np.float16)
    func = KTIRParser().parse_module(K.blocked_gather(shape, sel)).get_function("blocked_gather")
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items()]
    dev = RecordingDevice()
    sess = Session(dev, func, tensors, {}, arena_ptr=0)
    (stmt,) = sess.plan.statements
    assert stmt.kind == "rows_program"
    layout, _ = arena_layout(tensors)
    arena = np.zeros(max(o + n for o, n, _, _ in layout.values()) + 256, np.uint8)
    for name, (off, nb, _, _) in layout.items():
        arena[off:off + nb] = np.ascontiguousarray(kw[name]).view(np.uint8).reshape(-1)
    replay_rows(stmt, dev, arena)
    off, nb, _, _ = layout["out_ptr"]
    got = arena[off:off + nb].view(np.float16).reshape(rshape)
    want = kw["src_ptr"][np.ix_(*[kw[f"idx{i}_ptr"] for i in range(len(sel))])]
    np.testing.assert_array_equal(got, want)
    assert stmt.args.inp[0].indirect == len(sel)

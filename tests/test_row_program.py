"""Row-program lowering (host logic, no GPU): the phases, row scalars and register programs that
``lower_rowprog.RowProgramStatement`` hands to ``ktb_launch_row_program`` are replayed in NumPy — register
programs op by op with f16 rounding where flagged, reductions folded x[i] (op) x[i + h] like the
reference's linalg.reduce (ktir_cpu/dialects/linalg_ops.py:86-133) — and compared with the oracle."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import lower as L
from ktir_cpu_b200 import runtime as R
from ktir_cpu_b200.interpreter import Session, arena_layout
from ktir_cpu_b200.parser import KTIRParser
from oracle.numpy_interp import OracleInterpreter
from test_row_forms import RecordingDevice

NAMES = {v: k for k, v in R.VM.items()}


def run_program(prog, inputs):
    """``inputs``: list of float32 arrays (one per input register); returns the result register."""
    regs = list(inputs) + [None] * (R.VM_REGS - len(inputs))
    for o in list(prog.ops)[:prog.n_ops]:
        a = np.float32(o.imm) if o.opcode & R.VM_IMM_A else regs[o.a]
        b = np.float32(o.imm) if o.opcode & R.VM_IMM_B else regs[o.b]
        name = NAMES[o.opcode & 0xff]
        with np.errstate(all="ignore"):
            x = {"MOV": lambda: a, "CONST": lambda: np.float32(o.imm), "ADD": lambda: a + b, "SUB": lambda: a - b,
                 "MUL": lambda: a * b, "DIV": lambda: a / b, "SQRT": lambda: np.sqrt(a), "EXP": lambda: np.exp(a),
                 "LOG": lambda: np.log(a), "MAXNUM": lambda: np.fmax(a, b)}[name]()
        x = np.asarray(x, np.float32)
        regs[o.dst] = x.astype(np.float16).astype(np.float32) if o.opcode & R.VM_ROUND16 else x
    return regs[prog.result_reg]


def fold(x, op, r16):
    """x: [rows, cols] float32, cols a power of two; pairs (i, i + h), h = cols / 2 ... 1."""
    x = x.copy()
    while x.shape[1] > 1:
        h = x.shape[1] // 2
        x = (x[:, :h] + x[:, h:]) if op == R.RP_OPS["add"] else \
            np.fmax(x[:, :h], x[:, h:]) if op == R.RP_OPS["maxnum"] else np.maximum(x[:, :h], x[:, h:])
        if r16:
            x = x.astype(np.float16).astype(np.float32)
    return x[:, 0]


def replay(stmt, dev, arena):
    a = stmt.args
    table = dev.arrays[a.dev_item_offsets].reshape(a.n_items, a.n_in + 1 + a.n_side)
    npdt = {R.DTYPE_CODE["f16"]: np.float16, R.DTYPE_CODE["f32"]: np.float32}
    R_, Ccols = a.rows_per_item, a.cols
    r = np.arange(R_)[None, :, None]
    c = np.arange(Ccols)[None, None, :]

    def index(k, jb):
        return (table[:, k][:, None, None] + r * a.row_stride[k] + jb * a.blk_stride[k] + c).reshape(-1, Ccols)

    def tile(k, jb=0):
        return arena.view(npdt[a.dtype[k]])[index(k, jb)].astype(np.float32)        # [rows, cols]

    rows = a.n_items * R_
    red, scal, done = [], [None] * a.n_scal, 0
    for p in range(a.n_red + 1):
        while done < a.n_scal and a.scal[done].ready_after < p:
            scal[done] = run_program(a.scal[done].prog, red + [np.zeros(rows, np.float32)] * (a.n_red - len(red)))
            done += 1
        if p == a.n_red and a.out_per_row:
            out = run_program(a.out.prog, red)
            mem = arena.view(npdt[a.dtype[a.n_in]])
            idx = (table[:, a.n_in][:, None] + np.arange(R_)[None, :] * a.row_stride[a.n_in]).reshape(-1)
            mem[idx] = out.astype(mem.dtype)
            return
        if p == a.n_red:
            for s in range(a.n_side):               # per-row results stored beside the output tile
                mem = arena.view(npdt[a.side[s].dtype])
                idx = (table[:, a.n_in + 1 + s][:, None] + np.arange(R_)[None, :] * a.side[s].row_stride).reshape(-1)
                mem[idx] = run_program(a.side[s].prog, red).astype(mem.dtype)
        ph = a.red[p] if p < a.n_red else a.out
        acc = np.full((rows, Ccols), ph.acc_init, np.float32)
        for jb in range(a.n_blocks if ph.blocked else 1):
            ins = [tile(k, jb) for k in range(a.n_in)]
            ins += [np.broadcast_to(s[:, None], (rows, Ccols)) if s is not None else None for s in scal]
            val = np.broadcast_to(run_program(ph.prog, ins), (rows, Ccols)).astype(np.float32)
            if p < a.n_red and ph.blocked:
                acc = acc + val
                if ph.acc_round16:
                    acc = acc.astype(np.float16).astype(np.float32)
            elif p < a.n_red:
                acc = val
            else:
                mem = arena.view(npdt[a.dtype[a.n_in]])
                mem[index(a.n_in, jb)] = val.astype(mem.dtype)
        if p < a.n_red:
            red.append(fold(acc, ph.op, bool(ph.round16)))


def plan_and_replay(src, fn, kw):
    func = KTIRParser().parse_module(src).get_function(fn)
    scalars = {k: v for k, v in kw.items() if not isinstance(v, np.ndarray)}
    kw = {k: v for k, v in kw.items() if isinstance(v, np.ndarray)}
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items()]
    dev = RecordingDevice()
    sess = Session(dev, func, tensors, scalars, arena_ptr=0)
    layout, _ = arena_layout(tensors)
    arena = np.zeros(max(o + n for o, n, _, _ in layout.values()) + 256, np.uint8)
    for name, (off, nb, _, _) in layout.items():
        arena[off:off + nb] = np.ascontiguousarray(kw[name]).view(np.uint8).reshape(-1)
    for stmt in sess.plan.statements:
        assert stmt.kind == "row_program"
        replay(stmt, dev, arena)
    return {name: arena[off:off + nb].view(dt).reshape(shape).copy() for name, (off, nb, shape, dt) in layout.items()}, sess


@pytest.fixture(params=[True, False], ids=["one_launch", "per_row_statements"])
def fuse_row_results(request, monkeypatch):
    """With and without per-row results joining the launch of the statement whose reductions they are."""
    monkeypatch.setattr(L, "FUSE_ROW_RESULTS", request.param)
    return request.param


@pytest.mark.parametrize("rows,cols,cores", [(16, 64, 4), (12, 1024, 3), (8, 8, 2)])
def test_layernorm_phases_give_the_oracle_bits(rows, cols, cores, fuse_row_results):
    rng = np.random.default_rng(rows + cols)
    kw = dict(x_ptr=(rng.standard_normal((rows, cols)) * 2 + 1).astype(np.float16), w_ptr=rng.standard_normal(cols).astype(np.float16),
              b_ptr=rng.standard_normal(cols).astype(np.float16), y_ptr=np.zeros((rows, cols), np.float16),
              mean_ptr=np.zeros(rows, np.float32))
    src = K.layernorm_rows(rows, cols, cores)
    got, sess = plan_and_replay(src, "layernorm_kernel", kw)
    if fuse_row_results:
        y_stmt, = sess.plan.statements          # the row means leave with the launch that sums the rows anyway
        assert (y_stmt.args.n_side, y_stmt.args.side[0].dtype, y_stmt.args.side[0].row_stride) == (1, R.DTYPE_CODE["f32"], 1)
    else:
        y_stmt, m_stmt = sess.plan.statements
        assert (m_stmt.args.n_red, m_stmt.args.n_scal, m_stmt.args.out_per_row) == (1, 0, 1)
    assert (y_stmt.args.n_red, y_stmt.args.n_scal, y_stmt.args.out_per_row) == (2, 2, 0)
    assert y_stmt.args.red[0].prog.n_ops == 0 and y_stmt.args.out.load_mask == 0b111      # sum of x as it is; x, w, b at the end
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("layernorm_kernel", **kw)
    for k in ("y_ptr", "mean_ptr"):
        np.testing.assert_array_equal(got[k].view(np.uint8), want[k].view(np.uint8), err_msg=k)


@pytest.mark.parametrize("rows,cols,cores,tile_rows", [(16, 64, 2, 4), (8, 256, 1, 8)])
def test_rmsnorm_tiles_of_several_rows(rows, cols, cores, tile_rows, fuse_row_results):
    rng = np.random.default_rng(cols)
    kw = dict(x_ptr=(rng.standard_normal((rows, cols)) * 2).astype(np.float16), y_ptr=np.zeros((rows, cols), np.float16),
              rstd_ptr=np.zeros(rows, np.float32))
    src = K.rmsnorm_rows(rows, cols, cores, tile_rows)
    got, sess = plan_and_replay(src, "rmsnorm_kernel", kw)
    assert [s.args.rows_per_item for s in sess.plan.statements] == [tile_rows] * (1 if fuse_row_results else 2)
    assert sess.plan.statements[0].args.n_side == int(fuse_row_results)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("rmsnorm_kernel", **kw)
    for k in ("y_ptr", "rstd_ptr"):
        np.testing.assert_array_equal(got[k].view(np.uint8), want[k].view(np.uint8), err_msg=k)


def test_a_weight_row_shared_by_the_rows_of_a_tile_is_an_operand_whose_rows_do_not_advance():
    rng = np.random.default_rng(5)
    kw = dict(x_ptr=(rng.standard_normal((32, 128)) * 2).astype(np.float16), w_ptr=rng.standard_normal(128).astype(np.float16),
              y_ptr=np.zeros((32, 128), np.float16), rstd_ptr=np.zeros(32, np.float32))
    src = K.rmsnorm_rows(32, 128, 2, 4, weight=True)
    got, sess = plan_and_replay(src, "rmsnorm_kernel", kw)
    a = sess.plan.statements[0].args
    assert (a.n_in, a.rows_per_item, list(a.row_stride)[:3]) == (2, 4, [128, 0, 128])
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("rmsnorm_kernel", **kw)
    for k in ("y_ptr", "rstd_ptr"):
        np.testing.assert_array_equal(got[k].view(np.uint8), want[k].view(np.uint8), err_msg=k)


@pytest.mark.parametrize("rows,cols,block,cores", [(8, 512, 256, 2), (6, 1024, 128, 3), (5, 64, 8, 5)])
def test_column_blocked_layernorm_is_taken_row_by_row(rows, cols, block, cores, fuse_row_results):
    """The layer norm of examples/triton-ktir/layernorm_fwd_ktir.mlir: f16 throughout, rows walked in column
    blocks whose elementwise sums are carried through loops, mean and rstd stored per row, the output written
    block by block in a third loop.  All three statements become row programs over rows of `cols / block`
    blocks: blocked reduction phases (accumulate, then fold) and a blocked output phase."""
    rng = np.random.default_rng(rows * cols)
    kw = dict(X=rng.standard_normal((rows, cols)).astype(np.float16), Y=np.zeros((rows, cols), np.float16),
              W=rng.standard_normal((rows, cols)).astype(np.float16), B=rng.standard_normal((rows, cols)).astype(np.float16),
              Mean=np.zeros(rows, np.float16), Rstd=np.zeros(rows, np.float16), N=cols, eps=np.float16(1e-5), BLOCK_SIZE=block)
    src = K.layernorm_blocked(rows, cols, block, cores)
    got, sess = plan_and_replay(src, "_layer_norm_fwd_fused", kw)
    nb = cols // block
    if fuse_row_results:
        # Mean and Rstd are stored outside the loop over column blocks that the output statement has absorbed:
        # both leave with its launch, from the sums it folds anyway
        y_s, = sess.plan.statements
        assert (y_s.args.n_side, y_s.args.n_blocks, y_s.table.shape) == (2, nb, (rows, 6))
    else:
        mean_s, rstd_s, y_s = sess.plan.statements
        assert [s.args.n_blocks for s in sess.plan.statements] == [nb] * 3
        assert (mean_s.args.out_per_row, mean_s.args.n_red, rstd_s.args.n_red) == (1, 1, 2)
    assert (y_s.args.n_in, y_s.args.n_red, y_s.args.n_scal, y_s.args.out.blocked, y_s.args.n_items) == (3, 2, 2, 1, rows)
    assert list(y_s.args.blk_stride)[:4] == [block] * 4 and y_s.args.red[0].blocked and y_s.args.red[1].acc_round16
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("_layer_norm_fwd_fused", **kw)
    for k in ("Y", "Mean", "Rstd"):
        np.testing.assert_array_equal(got[k].view(np.uint16), want[k].view(np.uint16), err_msg=k)


def test_log_softmax_uses_two_kinds_of_reduction():
    """max (maxnumf) and sum of an expression of the max, an output that uses both row values."""
    rng = np.random.default_rng(8)
    kw = dict(x_ptr=(rng.standard_normal((16, 128)) * 3).astype(np.float16), y_ptr=np.zeros((16, 128), np.float16))
    src = K.log_softmax_rows(16, 128, 2, 4)
    got, sess = plan_and_replay(src, "log_softmax_kernel", kw)
    a = sess.plan.statements[0].args
    assert [a.red[k].op for k in range(a.n_red)] == [R.RP_OPS["maxnum"], R.RP_OPS["add"]] and a.n_scal == 2
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("log_softmax_kernel", **kw)
    np.testing.assert_array_equal(got["y_ptr"].view(np.uint16), want["y_ptr"].view(np.uint16))


def test_registers_are_reused_and_misfits_are_refused():
    from ktir_cpu_b200.runtime import PlanOnlyDevice
    f16, f32 = np.dtype(np.float16), np.dtype(np.float32)
    t = [("x_ptr", (16, 48), f16), ("w_ptr", (48,), f16), ("b_ptr", (48,), f16), ("y_ptr", (16, 48), f16), ("mean_ptr", (16,), f32)]
    sess = Session(PlanOnlyDevice(), KTIRParser().parse_module(K.layernorm_rows(16, 48, 4)).get_function("layernorm_kernel"), t, {}, arena_ptr=0)
    assert [s.kind for s in sess.plan.statements] == ["generic", "generic"]          # 48 columns: no power of two
    t = [(n, (16, 64) if s == (16, 48) else (64,) if s == (48,) else s, d) for n, s, d in t]
    sess = Session(PlanOnlyDevice(), KTIRParser().parse_module(K.layernorm_rows(16, 64, 4)).get_function("layernorm_kernel"), t, {}, arena_ptr=0)
    out = sess.plan.statements[0].args.out.prog
    regs = {o.dst for o in list(out.ops)[:out.n_ops]}
    assert out.n_ops == 5 and len(regs) == 1                     # sub, mul, mul, add, round: one temporary, reused


def test_run_overlap_check_behind_the_absorption_of_per_row_results():
    """A per-row result joins its neighbour's launch only if its bytes are apart from everything that launch
    touches; the check takes sorted or unsorted runs, nested and touching ones."""
    from ktir_cpu_b200.lower_rowprog import _runs_overlap
    a = lambda *v: np.array(v, np.int64)                                     # noqa: E731
    assert not _runs_overlap(a(0, 10), a(4, 14), a(4, 14), a(10, 20))        # touching ends do not meet
    assert _runs_overlap(a(0, 10), a(4, 15), a(4, 14), a(10, 20))
    assert _runs_overlap(a(100), a(101), a(300, 0), a(400, 1000))            # inside a long run listed second
    assert not _runs_overlap(a(1000), a(1001), a(300, 0), a(400, 1000))
    assert not _runs_overlap(a(5000, 6000), a(5002, 6002), a(0, 64), a(64, 128))   # apart altogether
    rng = np.random.default_rng(0)
    for _ in range(200):
        s0 = rng.integers(0, 200, 5); e0 = s0 + rng.integers(1, 8, 5)
        s1 = rng.integers(0, 200, 7); e1 = s1 + rng.integers(1, 30, 7)
        want = bool(((s0[:, None] < e1[None, :]) & (s1[None, :] < e0[:, None])).any())
        assert _runs_overlap(s0, e0, s1, e1) == want

"""The C-ABI launchers refuse malformed argument blocks before anything reaches the GPU.

Each case plans a real kernel, copies the argument block its statement would pass, breaks one field and
calls the ``extern "C"`` entry point directly: the call must return a negative code, leave a message that
names the launcher, launch nothing, and leave the context usable (the untouched statement still runs and
still matches the oracle).  Nothing here reaches a kernel with bad arguments: every refusal happens on the
host, in the launcher's own checks.
"""
import ctypes as C

import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K, runtime as R
from ktir_cpu_b200.interpreter import KTIRInterpreter
from oracle.numpy_interp import OracleInterpreter

pytestmark = pytest.mark.gpu

E_ARG, E_UNSUPPORTED = -2, -3


def _session(src, fn, kw):
    interp = KTIRInterpreter()
    interp.load(src)
    sess, _ = interp.session(fn, **kw)
    return interp, sess


def _copy(args, arena):
    out = type(args)()
    C.memmove(C.byref(out), C.byref(args), C.sizeof(type(args)))
    out.arena = arena
    return out


def _refused(dev, launch, args, code, *words):
    before = dev.launch_count()
    rc = launch(dev.h, C.byref(args))
    msg = dev.lib.ktb_last_error(dev.h).decode()
    assert rc == code, (rc, msg)
    for w in words:
        assert w in msg, msg
    assert dev.launch_count() == before
    with pytest.raises((R.DeviceError, NotImplementedError)):
        dev.check(rc)
    assert dev.sync().wait_timeout == 0


def _still_matches(interp, src, fn, kw, outs):
    got = interp.execute_function(fn, **kw)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function(fn, **kw)
    for name, exact in outs.items():
        if exact:
            np.testing.assert_array_equal(got[name], want[name])
        else:
            np.testing.assert_allclose(got[name].astype(np.float32), want[name].astype(np.float32),
                                       rtol=2e-3, atol=1e-2)


def _only(sess, kind):
    stmts = [s for s in sess.plan.statements if s.kind == kind]
    assert stmts, [s.kind for s in sess.plan.statements]
    return stmts[0]


def test_elementwise_launcher_refuses_bad_programs(build_lib):
    rng = np.random.default_rng(1)
    n = 1 << 16
    kw = dict(x_ptr=rng.standard_normal(n).astype(np.float16), y_ptr=rng.standard_normal(n).astype(np.float16),
              output_ptr=np.zeros(n, np.float16), BLOCK_SIZE=2048)
    src = K.vector_add(n, 2048, 32)
    interp, sess = _session(src, "add_kernel", kw)
    dev, stmt = sess.dev, _only(sess, "ew_stream")
    launch = dev.lib.ktb_launch_ew_stream
    a = _copy(stmt.args, sess.arena)
    a.program.n_ops = R.VM_MAX_OPS + 1
    _refused(dev, launch, a, E_ARG, "ew_stream", "program header")
    a = _copy(stmt.args, sess.arena)
    a.program.ops[0].opcode = len(R.VM_OPS)
    _refused(dev, launch, a, E_ARG, "ew_stream", "program op")
    a = _copy(stmt.args, sess.arena)
    a.program.ops[0].a = R.VM_REGS
    _refused(dev, launch, a, E_ARG, "ew_stream", "program op")
    a = _copy(stmt.args, sess.arena)
    a.dtype[0] = 99
    _refused(dev, launch, a, E_UNSUPPORTED, "ew_stream", "dtype")
    _still_matches(interp, src, "add_kernel", kw, {"output_ptr": True})
    interp.close()


def test_softmax_launcher_refuses_bad_rows(build_lib):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 1024)).astype(np.float16)
    kw = dict(output_ptr=np.zeros_like(x), input_ptr=x)
    src = K.softmax_rows(64, 1024, 4, 8)
    interp, sess = _session(src, "softmax_kernel", kw)
    dev, stmt = sess.dev, _only(sess, "row_softmax")
    launch = dev.lib.ktb_launch_row_softmax
    for cols in (1000, 4, 32768):
        a = _copy(stmt.args, sess.arena)
        a.cols = cols
        _refused(dev, launch, a, E_UNSUPPORTED, "row_softmax", "power of two")
    a = _copy(stmt.args, sess.arena)
    a.in_dtype = 7
    _refused(dev, launch, a, E_UNSUPPORTED, "row_softmax", "dtype")
    a = _copy(stmt.args, sess.arena)
    a.in_row_stride = 1028
    _refused(dev, launch, a, E_UNSUPPORTED, "row_softmax", "multiples of 8")
    _still_matches(interp, src, "softmax_kernel", kw, {"output_ptr": False})
    interp.close()


def test_row_program_launcher_refuses_bad_phases(build_lib):
    rng = np.random.default_rng(3)
    rows, cols = 64, 256
    kw = dict(x_ptr=rng.standard_normal((rows, cols)).astype(np.float16), w_ptr=rng.standard_normal(cols).astype(np.float16),
              b_ptr=rng.standard_normal(cols).astype(np.float16), y_ptr=np.zeros((rows, cols), np.float16),
              mean_ptr=np.zeros(rows, np.float32))
    src = K.layernorm_rows(rows, cols, 4)
    interp, sess = _session(src, "layernorm_kernel", kw)
    dev = sess.dev
    stmt = [s for s in sess.plan.statements if s.kind == "row_program" and not s.args.out_per_row][0]
    assert stmt.args.n_red == 2 and stmt.args.n_scal >= 2
    launch = dev.lib.ktb_launch_row_program
    a = _copy(stmt.args, sess.arena)
    a.n_red = R.RP_MAX_RED + 1
    _refused(dev, launch, a, E_ARG, "row_program", "counts")
    a = _copy(stmt.args, sess.arena)
    a.n_in = 0
    _refused(dev, launch, a, E_ARG, "row_program", "counts")
    a = _copy(stmt.args, sess.arena)
    a.cols = 384
    _refused(dev, launch, a, E_UNSUPPORTED, "row_program", "power of two")
    a = _copy(stmt.args, sess.arena)
    a.n_blocks = 2                                   # no phase walks column blocks
    _refused(dev, launch, a, E_ARG, "row_program", "column-block")
    a = _copy(stmt.args, sess.arena)
    a.red[1].op = 9
    _refused(dev, launch, a, E_UNSUPPORTED, "row_program", "add or max")
    a = _copy(stmt.args, sess.arena)
    a.red[0].prog.result_reg = R.VM_REGS
    _refused(dev, launch, a, E_ARG, "row_program", "program header")
    a = _copy(stmt.args, sess.arena)
    a.out.prog.ops[0].dst = -1
    _refused(dev, launch, a, E_ARG, "row_program", "program op")
    a = _copy(stmt.args, sess.arena)
    a.scal[1].ready_after = -1                       # sorted by the last reduction they read
    a.scal[0].ready_after = 1
    _refused(dev, launch, a, E_ARG, "row_program", "sorted")
    a = _copy(stmt.args, sess.arena)
    a.row_stride[0] = cols + 4
    _refused(dev, launch, a, E_UNSUPPORTED, "row_program", "multiples of 8")
    a = _copy(stmt.args, sess.arena)
    a.red[1].prog.ops[0].opcode |= R.VM_IMM_B        # immediates are for the row-value programs
    _refused(dev, launch, a, E_ARG, "row_program", "immediate operands")
    assert stmt.args.n_side == 1                     # the row means leave with this launch
    a = _copy(stmt.args, sess.arena)
    a.n_side = R.RP_MAX_SIDE + 1
    _refused(dev, launch, a, E_ARG, "row_program", "side result")
    a = _copy(stmt.args, sess.arena)
    a.side[0].dtype = R.DTYPE_CODE["i32"]
    _refused(dev, launch, a, E_UNSUPPORTED, "row_program", "side result dtype")
    a = _copy(stmt.args, sess.arena)
    a.side[0].prog.n_in = a.n_red + 1
    _refused(dev, launch, a, E_ARG, "row_program", "program header")
    _still_matches(interp, src, "layernorm_kernel", kw, {"y_ptr": True, "mean_ptr": True})
    interp.close()


def test_gemm_launcher_refuses_shapes_the_tiles_cannot_cover(build_lib):
    rng = np.random.default_rng(4)
    M = N = Kd = 256
    kw = dict(a_ptr=rng.uniform(-1, 1, (M, Kd)).astype(np.float16), b_ptr=rng.uniform(-1, 1, (Kd, N)).astype(np.float16),
              c_ptr=np.zeros((M, N), np.float16))
    src = K.tiled_matmul(M, N, Kd, 64, 64, 64, 4, True)
    interp, sess = _session(src, "matmul_kernel", kw)
    dev, stmt = sess.dev, _only(sess, "gemm_f16")
    launch = dev.lib.ktb_launch_gemm_f16
    a = _copy(stmt.args, sess.arena)
    a.c_dtype = 5
    _refused(dev, launch, a, E_UNSUPPORTED, "gemm_f16", "f16 or f32")
    a = _copy(stmt.args, sess.arena)
    a.N = 48
    _refused(dev, launch, a, E_UNSUPPORTED, "gemm_f16", "multiple of 32")
    a = _copy(stmt.args, sess.arena)
    a.lda = Kd + 4
    _refused(dev, launch, a, E_UNSUPPORTED, "gemm_f16", "multiples of 8")
    _still_matches(interp, src, "matmul_kernel", kw, {"c_ptr": False})
    interp.close()


def test_attention_launcher_refuses_other_head_sizes_and_pages(build_lib):
    from test_gpu_parity import _attention_inputs
    S, H, D, tn = 256, 2, 128, 64
    _, _, _, kw = _attention_inputs(np.random.default_rng(5), S, H, D, tn)
    src = K.causal_attention(S, H, D, 128, tn)
    interp, sess = _session(src, "attention_kernel", kw)
    dev, stmt = sess.dev, _only(sess, "attention_fwd")
    launch = dev.lib.ktb_launch_attention_fwd
    a = _copy(stmt.args, sess.arena)
    a.head_dim = 64
    _refused(dev, launch, a, E_UNSUPPORTED, "attention_fwd", "head_dim")
    a = _copy(stmt.args, sess.arena)
    a.page = 48
    _refused(dev, launch, a, E_UNSUPPORTED, "attention_fwd", "page")
    a = _copy(stmt.args, sess.arena)
    a.scale = 0.0
    _refused(dev, launch, a, E_UNSUPPORTED, "attention_fwd", "scale")
    a = _copy(stmt.args, sess.arena)
    a.q_row_stride += 4
    _refused(dev, launch, a, E_UNSUPPORTED, "attention_fwd", "multiples of 8")
    _still_matches(interp, src, "attention_kernel", kw, {"output_ptr": False})
    interp.close()


def test_row_gather_launcher_refuses_bad_operands(build_lib):
    rng = np.random.default_rng(6)
    table = rng.standard_normal((256, 128)).astype(np.float16)
    idx = rng.integers(0, 256, 512).astype(np.int32)
    kw = dict(table_ptr=table, idx_ptr=idx, out_ptr=np.zeros((512, 128), np.float16))
    src = K.gather_rows(256, 128, 512, 16, 4)
    interp, sess = _session(src, "gather_rows", kw)
    dev, stmt = sess.dev, _only(sess, "rows_program")
    launch = dev.lib.ktb_launch_rows_program
    a = _copy(stmt.args, sess.arena)
    a.inp[0].dtype = 42
    _refused(dev, launch, a, E_UNSUPPORTED, "rows_program", "f16 or f32")
    a = _copy(stmt.args, sess.arena)
    a.inp[0].idx_dtype = 0
    _refused(dev, launch, a, E_UNSUPPORTED, "rows_program", "i32 or i64")
    a = _copy(stmt.args, sess.arena)
    a.inp[0].indirect = 3
    _refused(dev, launch, a, E_UNSUPPORTED, "rows_program", "two index lookups")
    a = _copy(stmt.args, sess.arena)
    a.tile_rows = 0
    _refused(dev, launch, a, E_ARG, "rows_program", "tile geometry")
    a = _copy(stmt.args, sess.arena)
    a.program.n_in = 9
    _refused(dev, launch, a, E_ARG, "rows_program", "program header")
    _still_matches(interp, src, "gather_rows", kw, {"out_ptr": True})
    interp.close()


def test_generic_step_launcher_refuses_unknown_kinds_and_extents(build_lib):
    dev = R.Device()
    launch = dev.lib.ktb_launch_generic
    a = R.GenOpArgs()
    a.kind, a.points, a.elems, a.ndim = len(R.G_KINDS) + 3, 1, 8, 1
    _refused(dev, launch, a, E_ARG, "generic", "step kind")
    a = R.GenOpArgs()
    a.kind, a.points, a.elems, a.ndim = R.G_KINDS["ew"], 1, 8, R.G_MAXDIM + 1
    _refused(dev, launch, a, E_ARG, "generic", "extents")
    a = R.GenOpArgs()
    a.kind, a.points, a.elems = R.G_KINDS["ew"], -1, 8
    _refused(dev, launch, a, E_ARG, "generic", "extents")
    dev.close()

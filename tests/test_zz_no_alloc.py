"""ktb_launch_scatter_rows_static: the scatter with its scratch in a fixed array inside the library.

Collected last (file name) so that it also runs after every other GPU test has used the context;
it passes alone in a fresh process as well.  The new entry point is called through the C ABI and
compared bit for bit with ktb_launch_scatter_rows on the same statement, twice in a row with
different inputs (the array keeps the previous call's contents).
"""
import ctypes as C

import numpy as np
import pytest

from ktir_cpu_b200 import KTIRInterpreter, kernels as K
from ktir_cpu_b200 import runtime as R

pytestmark = pytest.mark.gpu


def _scatter_statement(sess):
    stmts = [s for s in sess.plan.statements if getattr(s, "kind", "") == "scatter_rows"]
    assert len(stmts) == 1 and len(sess.plan.statements) == 1
    return stmts[0]


def _run(sess, tensors, static):
    dev = sess.dev
    for name, arr in tensors.items():
        sess.upload(name, arr)
    stmt = _scatter_statement(sess)
    stmt.args.arena = sess.arena
    if static:
        args = R.RowsArgs()
        C.memmove(C.byref(args), C.byref(stmt.args), C.sizeof(R.RowsArgs))
        args.dev_rowid_scratch = None          # must be ignored
        dev.check(dev.lib.ktb_launch_scatter_rows_static(dev.h, C.byref(args)))
    else:
        dev.check(dev.lib.ktb_launch_scatter_rows(dev.h, C.byref(stmt.args)))
    out = sess.download("out_ptr")
    dev.sync()
    return out


def _inputs(seed, n_rows, n_idx, rmw):
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, n_rows, n_idx).astype(np.int32)
    idx[::7] = idx[3]                           # heavy reuse of one row, within and across tiles
    out = rng.standard_normal((n_rows, 128)).astype(np.float16)
    if rmw:
        return dict(table_ptr=rng.standard_normal((n_rows, 128)).astype(np.float16), idx_ptr=idx, out_ptr=out)
    return dict(src_ptr=rng.standard_normal((n_idx, 128)).astype(np.float16), idx_ptr=idx, out_ptr=out)


@pytest.mark.parametrize("rmw", [False, True])
def test_static_scratch_scatter_matches_allocating_entry_point(rmw, build_lib):
    n_rows, n_idx = 1024, 16384
    interp = KTIRInterpreter()
    if rmw:
        interp.load(K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8))
        fn = "gather_scale_scatter"
    else:
        interp.load(K.scatter_rows(n_rows, 128, n_idx, 64, 8))
        fn = "scatter_rows"
    first = _inputs(11, n_rows, n_idx, rmw)
    sess, _ = interp.session(fn, **first)
    for seed in (11, 12):                       # two calls in a row, different data
        tensors = _inputs(seed, n_rows, n_idx, rmw)
        want = _run(sess, tensors, static=False)
        got = _run(sess, tensors, static=True)
        np.testing.assert_array_equal(got, want)
        assert not np.array_equal(want, tensors["out_ptr"])
    interp.close()


def test_static_scratch_scatter_rejects_statements_beyond_the_array(build_lib):
    interp = KTIRInterpreter()
    interp.load(K.scatter_rows(1024, 128, 16384, 64, 8))
    tensors = _inputs(13, 1024, 16384, False)
    sess, _ = interp.session("scatter_rows", **tensors)
    dev = sess.dev
    stmt = _scatter_statement(sess)
    args = R.RowsArgs()
    C.memmove(C.byref(args), C.byref(stmt.args), C.sizeof(R.RowsArgs))
    args.arena = sess.arena
    args.dst_rows = 1 << 22                     # bucket table alone would need > 8 MiB
    assert int(dev.lib.ktb_scatter_scratch_bytes(16384, 1 << 22)) > (8 << 20)
    rc = dev.lib.ktb_launch_scatter_rows_static(dev.h, C.byref(args))
    assert rc != 0
    msg = dev.lib.ktb_last_error(dev.h).decode()
    assert "built-in array" in msg and "ktb_launch_scatter_rows" in msg
    # nothing was launched and the context is still usable
    want = _run(sess, tensors, static=False)
    got = _run(sess, tensors, static=True)
    np.testing.assert_array_equal(got, want)
    interp.close()

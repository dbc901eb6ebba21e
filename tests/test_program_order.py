"""Order of a core's loads and stores (host logic, no GPU): a load sees memory as it is at the load's
position in the program (ktir_cpu/interpreter.py:196-281), so a statement whose tile was loaded before
an earlier store to the same bytes has to run first — or the plan is refused."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import Session
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.runtime import PlanOnlyDevice
from ktir_cpu_b200.trace import Unsupported
from oracle.numpy_interp import OracleInterpreter
from test_generic_lowering import run_generic

F16 = np.dtype(np.float16)


def _plan(src, fn, tensors):
    return Session(PlanOnlyDevice(), KTIRParser().parse_module(src).get_function(fn), tensors, {}, arena_ptr=0)


def _written_first(sess):
    """Name of the tensor the first statement of the plan writes."""
    fp = next(f for f in sess.plan.statements[0].footprints() if f.write)
    return sess.arena_map.find(int(fp.starts[0])).name


@pytest.mark.parametrize("loop,n_rows", [(True, 64), (False, 16)])
def test_store_of_an_earlier_load_moves_in_front_of_the_store_that_overwrites_it(loop, n_rows):
    src = K.update_in_place(n_rows, 64, 8, 2, loop)
    sess = _plan(src, "update_in_place", [("x_ptr", (n_rows, 64), F16), ("old_ptr", (n_rows, 64), F16)])
    assert len(sess.plan.statements) == 2 and _written_first(sess) == "old_ptr"
    rng = np.random.default_rng(3)
    kw = dict(x_ptr=rng.standard_normal((n_rows, 64)).astype(np.float16), old_ptr=np.zeros((n_rows, 64), np.float16))
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("update_in_place", **{k: v.copy() for k, v in kw.items()})
    np.testing.assert_array_equal(want["old_ptr"], kw["x_ptr"])
    got, _ = run_generic(src, "update_in_place", kw)
    for k in want:
        np.testing.assert_array_equal(got[k], want[k])


def test_program_order_is_kept_when_nothing_is_loaded_early():
    """Two stores fed by the same load, nothing overwritten: max row first, then the sum row, as written."""
    sess = _plan(K.region_reduce_rows(16, 37, 4), "region_reduce",
                 [("x_ptr", (16, 37), F16), ("mx_ptr", (16,), F16), ("sa_ptr", (16,), F16)])
    first = [sess.arena_map.find(int(next(f for f in s.footprints() if f.write).starts[0])).name
             for s in sess.plan.statements]
    assert first == ["mx_ptr", "sa_ptr"]


def test_a_store_that_needs_memory_from_before_and_after_an_earlier_store_is_refused():
    src = K.update_in_place(64, 64, 8, 2, True, reuse_new=True)
    with pytest.raises(Unsupported, match="loaded before an earlier store"):
        _plan(src, "update_in_place", [("x_ptr", (64, 64), F16), ("old_ptr", (64, 64), F16)])


def test_a_load_of_the_next_iterations_store_unrolls_the_loop():
    """b[i] = 2 a[i]; c[i] = b[i + 1] inside one loop: as two whole statements the second would see the
    new b everywhere, so the loop runs iteration by iteration (2 statements x 8 iterations)."""
    src = K.shifted_reuse()
    sess = _plan(src, "shifted_reuse", [(k, (64, 64), F16) for k in ("a_ptr", "b_ptr", "c_ptr")])
    assert sess.plan.unrolled_groups == [(0, 1)] and len(sess.plan.statements) == 16
    rng = np.random.default_rng(6)
    kw = {k: rng.standard_normal((64, 64)).astype(np.float16) for k in ("a_ptr", "b_ptr", "c_ptr")}
    want_c = np.roll(kw["b_ptr"], -8, axis=0)
    want_c[-8:] = 2 * kw["a_ptr"][:8]
    got, _ = run_generic(src, "shifted_reuse", kw, core_groups=sess.plan.core_groups, unrolled=sess.plan.unrolled_groups)
    np.testing.assert_array_equal(got["c_ptr"], want_c)
    np.testing.assert_array_equal(got["b_ptr"], 2 * kw["a_ptr"])
    ora = OracleInterpreter()
    ora.load(src)
    np.testing.assert_array_equal(ora.execute_function("shifted_reuse", **kw)["c_ptr"], want_c)


def _core_groups(src, fn, tensors):
    return _plan(src, fn, tensors).plan.core_groups


@pytest.mark.parametrize("n_cores", [1, 5, 8])
def test_cores_that_read_each_others_rows_run_one_after_the_other(n_cores):
    """x[c + 1] += x[c] on core c: running sums only come out in the reference's core order."""
    src = K.core_chain(n_cores, 64)
    groups = _core_groups(src, "core_chain", [("x_ptr", (n_cores + 1, 64), F16)])
    assert groups == ([(c, c + 1) for c in range(n_cores)] if n_cores > 1 else None)
    x = np.random.default_rng(9).standard_normal((n_cores + 1, 64)).astype(np.float16)
    want = x.copy()
    for c in range(n_cores):
        want[c + 1] = want[c + 1] + want[c]
    ora = OracleInterpreter()
    ora.load(src)
    np.testing.assert_array_equal(ora.execute_function("core_chain", x_ptr=x.copy())["x_ptr"], want)
    got, _ = run_generic(src, "core_chain", dict(x_ptr=x.copy()), core_groups=groups)
    np.testing.assert_array_equal(got["x_ptr"], want)


def test_core_groups_are_as_large_as_the_clashes_allow():
    """Blocks shifted down by one with wrap-around: cores 0..2 read old blocks, core 3 reads what core 0 wrote."""
    from test_sharded import SHIFT
    x = np.arange(256, dtype=np.float16)
    groups = _core_groups(SHIFT, "shift", [("x_ptr", (256,), F16)])
    got, _ = run_generic(SHIFT, "shift", dict(x_ptr=x.copy()), core_groups=groups)
    want = x.copy()
    for c in range(4):
        want[c * 64:(c + 1) * 64] = want[((c + 1) % 4) * 64:((c + 1) % 4 + 1) * 64]
    np.testing.assert_array_equal(got["x_ptr"], want)
    ora = OracleInterpreter()
    ora.load(SHIFT)
    np.testing.assert_array_equal(ora.execute_function("shift", x_ptr=x.copy())["x_ptr"], want)


@pytest.mark.parametrize("n_cores,per_core", [(4, 6), (1, 3), (3, 1)])
def test_loop_iterations_that_read_what_the_last_one_wrote_run_one_by_one(n_cores, per_core):
    """acc[c] += x[i] with the running row re-loaded every iteration: the loop is unrolled into one
    statement per iteration (all cores at once — they do not touch each other's rows)."""
    src = K.accumulate_rows(n_cores, per_core, 64)
    rows = n_cores * per_core
    sess = _plan(src, "accumulate_rows", [("x_ptr", (rows, 64), F16), ("acc_ptr", (n_cores, 64), F16)])
    if per_core > 1:
        assert sess.plan.core_groups == [(0, n_cores)] and sess.plan.unrolled_groups == [(0, n_cores)]
        assert len(sess.plan.statements) == per_core
    else:
        assert sess.plan.core_groups is None
    rng = np.random.default_rng(4)
    kw = dict(x_ptr=rng.standard_normal((rows, 64)).astype(np.float16), acc_ptr=rng.standard_normal((n_cores, 64)).astype(np.float16))
    want = kw["acc_ptr"].copy()
    for c in range(n_cores):
        for i in range(per_core):
            want[c] = want[c] + kw["x_ptr"][c * per_core + i]
    ora = OracleInterpreter()
    ora.load(src)
    np.testing.assert_array_equal(ora.execute_function("accumulate_rows", **{k: v.copy() for k, v in kw.items()})["acc_ptr"], want)
    got, _ = run_generic(src, "accumulate_rows", kw, core_groups=sess.plan.core_groups, unrolled=sess.plan.unrolled_groups)
    np.testing.assert_array_equal(got["acc_ptr"], want)


def test_a_single_core_kernel_whose_index_tensor_overlaps_its_destination_plans_step_by_step():
    """Nothing runs concurrently on one core with one load and one store; the statement only has to read
    all its inputs before it writes — the step-by-step form does, a fused gather does not promise it."""
    from test_gpu_parity import _aliased_gather_source
    func = KTIRParser().parse_module(_aliased_gather_source()).get_function("gather_elements")
    sess = Session(PlanOnlyDevice(), func, [], {}, arena_ptr=0, seeded=[(0, 1024, "f16"), (1024, 512, "i32")])
    assert [s.kind for s in sess.plan.statements] == ["generic"]

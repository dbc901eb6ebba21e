"""The step-by-step fallback lowering, executed with the NumPy stand-in for the device steps and
compared with outputs of the unmodified reference (tests/golden/*.npz) — host logic, no GPU."""
import numpy as np
import pytest

import gen_emulator
from conftest import load_golden
from ktir_cpu_b200.dtypes import to_ktir_dtype
from ktir_cpu_b200.interpreter import Session, arena_layout
from ktir_cpu_b200.lower import Allocation, ArenaMap, _points
from ktir_cpu_b200.lower_generic import build_generic
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.runtime import PlanOnlyDevice
from ktir_cpu_b200.trace import Tracer


def run_generic(src, fn, kw):
    """Every store of the kernel through build_generic + the emulator, in program order."""
    func = KTIRParser().parse_module(src).get_function(fn)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items() if isinstance(v, np.ndarray)]
    scalars = {k: v for k, v in kw.items() if not isinstance(v, np.ndarray)}
    layout, ptrs = arena_layout(tensors)
    arena = np.zeros(max(o + n for o, n, _, _ in layout.values()) + 256, np.uint8)
    allocs = []
    for name, (off, nb, _, dt) in layout.items():
        arena[off:off + nb] = np.ascontiguousarray(kw[name]).view(np.uint8).reshape(-1)
        allocs.append(Allocation(name, off, off + nb, to_ktir_dtype(dt)))
    amap = ArenaMap(allocs)
    kinds = set()
    for st in Tracer(func, scalars, ptrs).run():
        sel, _ = _points(st)
        prog = build_generic(st, amap, sel)[0]
        kinds.update(op.kind for op in prog.ops)
        assert all(b.offset >= 0 for op in prog.ops for b in ([op.dst] if op.dst else []))
        flags = gen_emulator.run(prog, arena)
        assert not flags["negative_index"]
    out = {name: arena[off:off + nb].view(dt).reshape(shape).copy() for name, (off, nb, shape, dt) in layout.items()}
    return out, kinds


EXACT = ("vector_add_4096", "gather_elements_8x16", "matmul_f16acc_128", "elementwise_f16_suite")
CLOSE = ("layernorm_16x64", "naive_attention_32x16", "softmax_f32_64x256", "softmax_f16_64x256",
         "matmul_f32acc_128", "causal_attention_128x2")


@pytest.mark.parametrize("name", EXACT + CLOSE)
def test_generic_steps_reproduce_the_reference(name):
    src, fn, kw, want = load_golden(name)
    got, kinds = run_generic(src, fn, kw)
    for k, w in want.items():
        if name in EXACT and "erf" not in k:
            np.testing.assert_array_equal(got[k], w)
            np.testing.assert_array_equal(np.signbit(got[k]) | np.isnan(w), np.signbit(w) | np.isnan(w))
        else:
            # transcendental f16/f32 ufuncs differ by <= 1 ulp between hosts; f32 matmul order differs
            np.testing.assert_allclose(got[k].astype(np.float32), w.astype(np.float32), rtol=2e-3, atol=2e-3)
    assert "store" in kinds or "scatter" in kinds


def test_step_kinds_cover_reduction_matmul_and_indirect_access():
    _, k1 = run_generic(*load_golden("layernorm_16x64")[:3])
    _, k2 = run_generic(*load_golden("naive_attention_32x16")[:3])
    _, k3 = run_generic(*load_golden("gather_elements_8x16")[:3])
    assert {"load", "redl", "ew", "store"} <= k1
    assert {"matmul", "map", "redl"} <= k2
    assert {"addr", "idxadd", "gather"} <= k3


def test_scratch_is_reused():
    src, fn, kw, _ = load_golden("layernorm_16x64")
    func = KTIRParser().parse_module(src).get_function(fn)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items() if isinstance(v, np.ndarray)]
    sess = Session(PlanOnlyDevice(), func, tensors, {}, arena_ptr=0)
    gen = [s for s in sess.plan.statements if s.kind == "generic"]
    assert gen, [s.kind for s in sess.plan.statements]
    for s in gen:
        total = sum(b.elems * s.prog.P * 8 for b in s.prog.bufs)
        assert s.prog.scratch_bytes < total          # buffers share space once their readers are done


def test_read_modify_write_scatter_is_not_taken_by_the_fallback():
    """All points are read before any is written, so a cross-tile RMW must stay with the ordered scatter."""
    from ktir_cpu_b200.trace import Unsupported
    with pytest.raises(Unsupported, match="ordered row scatter"):
        run_generic(*load_golden("gather_scale_scatter_256")[:3])


def test_negative_index_is_flagged():
    src, fn, kw, _ = load_golden("gather_elements_8x16")
    kw = dict(kw)
    kw["idx_ptr"] = kw["idx_ptr"].copy()
    kw["idx_ptr"][2, 3] = -1
    with pytest.raises(AssertionError):
        run_generic(src, fn, kw)

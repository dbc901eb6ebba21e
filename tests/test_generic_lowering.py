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
from ktir_cpu_b200.order import program_order
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.runtime import PlanOnlyDevice
from ktir_cpu_b200.trace import Tracer


def run_generic(src, fn, kw, core_groups=None, unrolled=()):
    """Every store of the kernel through build_generic + the emulator, in launch order.  ``core_groups``
    = [(lo, hi), ...] runs the cores group after group, as a plan does whose cores cannot all run at once;
    the groups listed in ``unrolled`` are traced with their loops unrolled."""
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
    stores = []
    for rng in core_groups or [None]:
        tracer = Tracer(func, scalars, ptrs, core_range=rng)
        tracer.arena, tracer.unroll_loops = amap, rng in tuple(unrolled)
        part = tracer.run()
        stores += [part[k] for k in program_order(part, amap)]
    for st in stores:
        sel, _ = _points(st)
        prog = build_generic(st, amap, sel)[0]
        kinds.update(op.kind for op in prog.ops)
        assert all(b.offset >= 0 for op in prog.ops for b in ([op.dst] if op.dst else []))
        flags = gen_emulator.run(prog, arena)
        assert not flags["negative_index"]
    out = {name: arena[off:off + nb].view(dt).reshape(shape).copy() for name, (off, nb, shape, dt) in layout.items()}
    return out, kinds


EXACT = ("vector_add_4096", "gather_elements_8x16", "matmul_f16acc_128", "elementwise_f16_suite",
         "ring_allreduce_4x4_add_f16", "ring_allreduce_8x2_max_f32_strided", "ring_allreduce_6x3_mul_f16_loop",
         "ring_allreduce_16x16_add_f16", "ring_allreduce_16x4_add_f16", "shared_slot_store_12x5",
         "vector_add_short_4000", "sharded_scale_64x64_shift0", "sharded_scale_64x64_shift3", "sharded_center_8x256",
         "paged_gather_4x64", "region_reduce_16x37", "generic_contraction_4x8x13",
         "gather_rows_transposed_64x16", "update_in_place_64x64", "update_in_place_16x64_flat", "rmsnorm_weighted_32x128",
         "layernorm_blocked_8x512")
SEQUENTIAL = {"core_chain_16x64": ([(c, c + 1) for c in range(16)], ()), "accumulate_rows_4x6": ([(0, 4)], [(0, 4)])}
CLOSE = ("layernorm_16x64", "naive_attention_32x16", "softmax_f32_64x256", "softmax_f16_64x256",
         "matmul_f32acc_128", "causal_attention_128x2")


@pytest.mark.parametrize("name", EXACT + CLOSE + tuple(SEQUENTIAL))
def test_generic_steps_reproduce_the_reference(name):
    src, fn, kw, want = load_golden(name)
    groups, unrolled = SEQUENTIAL.get(name, (None, ()))
    got, kinds = run_generic(src, fn, kw, core_groups=groups, unrolled=unrolled)
    for k, w in want.items():
        if (name in EXACT or name in SEQUENTIAL) and "erf" not in k:
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


def test_distributed_view_tiles_resolve_to_address_tables_or_plain_tiles():
    """A tile that crosses partition boundaries becomes a per-element address table (holes where no
    partition backs it); tiles that lie whole inside one partition stay ordinary strided tiles."""
    _, k1 = run_generic(*load_golden("sharded_scale_64x64_shift3")[:3])
    _, k2 = run_generic(*load_golden("sharded_center_8x256")[:3])
    assert {"table", "gather", "scatter"} <= k1 and "load" not in k1
    assert {"load", "store", "ringred"} <= k2 and "table" not in k2
    src, fn, kw, _ = load_golden("sharded_scale_64x64_shift3")
    func = KTIRParser().parse_module(src).get_function(fn)
    sess = Session(PlanOnlyDevice(), func, [(k, tuple(v.shape), v.dtype) for k, v in kw.items()], {}, arena_ptr=0)
    (stmt,) = sess.plan.statements
    (sc,) = [op for op in stmt.prog.ops if op.kind == "scatter"]
    assert sc.attrs["any_order"]                      # every element has its own address: no ordering needed
    tables = [op.attrs["values"] for op in stmt.prog.ops if op.kind == "table"]
    assert all((t_ == -1).any() for t_ in tables)     # the last tile of the last core hangs over the end
    assert sess.plan.written == {"o0_ptr", "o1_ptr"}


def test_ring_reduce_uses_clusters_for_small_equal_groups():
    """Groups of at most 8 cores of equal size become thread-block clusters (sources are ranks inside
    the cluster); a 16-core group reads its partials from global memory (sources are points)."""
    src, fn, kw, _ = load_golden("ring_allreduce_16x4_add_f16")
    func = KTIRParser().parse_module(src).get_function(fn)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items()]
    sess = Session(PlanOnlyDevice(), func, tensors, {}, arena_ptr=0)
    (ring,) = [op for s in sess.plan.statements for op in s.prog.ops if op.kind == "ringred"]
    assert ring.attrs["cluster"] == 4 and ring.attrs["sources"].max() == 3 and sorted(ring.attrs["order"]) == list(range(16))
    assert (ring.attrs["counts"] == 3).all()
    src, fn, kw, _ = load_golden("ring_allreduce_16x16_add_f16")
    func = KTIRParser().parse_module(src).get_function(fn)
    sess = Session(PlanOnlyDevice(), func, [(k, tuple(v.shape), v.dtype) for k, v in kw.items()], {}, arena_ptr=0)
    (ring,) = [op for s in sess.plan.statements for op in s.prog.ops if op.kind == "ringred"]
    assert ring.attrs["cluster"] == 0 and (ring.attrs["counts"] == 15).all()
    # core 5 hears from 4, 3, 2, ... in that order
    assert list(ring.attrs["sources"][5][:6]) == [4, 3, 2, 1, 0, 15]


def test_a_core_that_skips_the_exchange_is_a_deadlock():
    from ktir_cpu_b200 import kernels as K
    func = KTIRParser().parse_module(K.ring_allreduce(4, 4, 128, absent_core=2)).get_function("ring_allreduce")
    t = [("in_ptr", (4, 128), np.dtype(np.float16)), ("out_ptr", (4, 128), np.dtype(np.float16))]
    with pytest.raises(RuntimeError, match="Deadlock detected: core 3 waiting on recv from core 2"):
        Session(PlanOnlyDevice(), func, t, {}, arena_ptr=0)


def test_scratch_is_reused():
    src, fn, kw, _ = load_golden("layernorm_16x64")
    func = KTIRParser().parse_module(src).get_function(fn)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items() if isinstance(v, np.ndarray)]
    sess = Session(PlanOnlyDevice(), func, tensors, {}, arena_ptr=0, fused=False)
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

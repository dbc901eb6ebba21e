"""Host-side logic that needs no GPU: parser, whole-grid trace, launch plans, C-ABI exports."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT, golden_names, load_golden
from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import runtime as R
from ktir_cpu_b200.affine import parse_affine_map, parse_affine_set
from ktir_cpu_b200.interpreter import KTIRInterpreter, Session
from ktir_cpu_b200.parser import KTIRParser
from ktir_cpu_b200.trace import Unsupported

F16 = np.dtype(np.float16)


def _plan(src, fn, tensors, scalars):
    m = KTIRParser().parse_module(src)
    return Session(R.PlanOnlyDevice(), m.get_function(fn), tensors, scalars)


def test_affine_parse_and_box():
    s = parse_affine_set("affine_set<(d0, d1) : (d0 >= 0, -d0 + 31 >= 0, d1 >= 0, -d1 + 127 >= 0)>")
    assert s.box() == ((0, 0), (32, 128))
    m = parse_affine_map("affine_map<(d0, d1) -> (d1, d0 * 2 + 1)>")
    assert m.eval([3, 5]) == (5, 7)
    assert not m.is_identity() and parse_affine_map("affine_map<(d0) -> (d0)>").is_identity()
    tri = parse_affine_set("affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, d0 - d1 >= 0)>")
    assert tri.box() is None
    assert tri.enumerate((4, 4)) == [(i, j) for i in range(4) for j in range(4) if j <= i]


def test_parser_function_metadata():
    m = KTIRParser().parse_module(K.vector_add())
    f = m.get_function("add_kernel")
    assert f.grid == (32, 1, 1)
    assert f.arg_names == ["x_ptr", "y_ptr", "output_ptr", "BLOCK_SIZE"]
    assert f.tensor_sizes["x_ptr"] == {"shape": (4096,), "dtype": "f16"}
    with pytest.raises(ValueError, match="not found in module"):
        m.get_function("nope")


def test_interpreter_api_errors():
    it = KTIRInterpreter()
    with pytest.raises(RuntimeError, match="No module loaded"):
        it.arg_names("f")
    with pytest.raises(RuntimeError, match="No module loaded"):
        it.tensor_input_output_sizes("f")
    it.load(K.vector_add())
    assert it.arg_names("add_kernel")[0] == "x_ptr"
    assert it.get_latency_report() is None


def test_plan_vector_add():
    t = [("x_ptr", (4096,), F16), ("y_ptr", (4096,), F16), ("output_ptr", (4096,), F16)]
    s = _plan(K.vector_add(), "add_kernel", t, dict(BLOCK_SIZE=128))
    (st,) = s.plan.statements
    assert st.kind == "ew_stream" and st.args.n_items == 32 and st.args.cols == 128
    assert st.program.n_ops == 1 and st.program.ops[0].opcode == (R.VM["ADD"] | R.VM_ROUND16)
    # KTIR pointer values are element indices of byte addresses starting at 0x10000
    assert st.table[0].tolist() == [0x10000 // 2, (0x10000 + 8192) // 2, (0x10000 + 16384) // 2]
    assert st.table[1, 0] - st.table[0, 0] == 128
    assert s.written == {"output_ptr"}


def test_plan_softmax_flattens_loop_into_launch():
    t = [("output_ptr", (8192, 4096), F16), ("input_ptr", (8192, 4096), F16)]
    s = _plan(K.softmax_rows(8192, 4096, 32, 8, True), "softmax_kernel", t, {})
    (st,) = s.plan.statements
    assert st.kind == "row_softmax"
    assert st.args.n_items == 32 * 32 and st.args.rows_per_item == 8 and st.args.cols == 4096
    assert st.args.f16_arith == 0 and st.args.max_init == float("-inf")
    assert st.bytes_moved() == 2 * 8192 * 4096 * 2


def test_cores_storing_to_the_same_tile_are_launched_in_core_order():
    """The reference runs its cores one after the other, so the last core's store survives
    (ktir_cpu/grid.py:595-613); the plan launches colliding stores in as many ordered rounds."""
    src = K.vector_add(4096, 128, 32).replace("%offset = arith.muli %core_id, %BLOCK_SIZE : index",
                                              "%offset = arith.constant 0 : index")
    t = [("x_ptr", (4096,), F16), ("y_ptr", (4096,), F16), ("output_ptr", (4096,), F16)]
    (stmt,) = _plan(src, "add_kernel", t, dict(BLOCK_SIZE=128)).plan.statements
    assert stmt.rounds == [(i, i + 1) for i in range(32)] and stmt.launches == 32
    sess = _plan(K.shared_slot_store(12, 5, 64), "shared_slot", [("x_ptr", (12, 64), F16), ("out_ptr", (5, 64), F16)], {})
    (stmt,) = sess.plan.statements
    assert stmt.rounds == [(0, 5), (5, 10), (10, 12)]         # cores 0-4, 5-9, 10-11
    assert sess.transfer_plan().split is False                  # ordered launches are not pipelined


def test_unmapped_pointer_raises_value_error():
    src = K.vector_add(4096, 128, 32)
    t = [("x_ptr", (4096,), F16), ("y_ptr", (4096,), F16)]
    with pytest.raises(ValueError, match="unmapped address"):
        _plan(src, "add_kernel", t, dict(output_ptr=0, BLOCK_SIZE=128))


def test_unknown_op_is_reported_at_execution():
    src = K.vector_add().replace("arith.addf %x, %y", "arith.frobnicate %x, %y")
    t = [("x_ptr", (4096,), F16), ("y_ptr", (4096,), F16), ("output_ptr", (4096,), F16)]
    with pytest.raises(ValueError, match="Unknown operation: arith.frobnicate"):
        _plan(src, "add_kernel", t, dict(BLOCK_SIZE=128))


def test_library_exports_every_declared_symbol(build_lib):
    header = open(os.path.join(ROOT, "include", "ktir_b200.h")).read()
    declared = set(re.findall(r"\b(ktb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(build_lib)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/ktir_b200.h but not exported"
    assert declared == set(R.SYMBOLS), "ctypes binding and header disagree"


def test_launchers_answer_null_handles_without_touching_a_device(build_lib):
    """Every launcher checks its two pointers before anything else: no context, no CUDA call."""
    lib = R.lib()
    for name in sorted(n for n in R.SYMBOLS if n.startswith("ktb_launch_") and n != "ktb_launch_count"):
        assert getattr(lib, name)(None, None) == -2, name       # KTB_E_ARG


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("paged_attention_ref")])
def test_reference_generated_attention_text_plans_as_the_tensor_core_kernel(name):
    """Kernel text written by the reference's own generator (stored in the fixture): one fused
    attention launch, with the grouping, context offset and page walk read off the text."""
    src, fn, kw, _ = load_golden(name)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items() if isinstance(v, np.ndarray)]
    scalars = {k: v for k, v in kw.items() if not isinstance(v, np.ndarray)}
    sess = _plan(src, fn, tensors, scalars)
    assert [s.kind for s in sess.plan.statements] == ["attention_fwd"]
    a = sess.plan.statements[0].args
    S, H, _ = kw["query_ptr"].shape
    Hkv = kw["key_cache_ptr"].shape[2]
    assert (a.seq_q, a.heads, max(a.kv_group, 1)) == (S, H, H // Hkv)
    assert a.causal == 1 and a.causal_delta == kw["context_len"] and a.num_tiles == kw["num_tiles"]
    assert sess.plan.fully_overwritten == {"output_ptr"}


def test_own_paged_attention_text_plans_like_the_reference_generator():
    sess = _plan(K.paged_attention(256, 384, 8, 2, 128, 64, 16), "paged_attention_kernel",
                 [("output_ptr", (256, 8, 128), F16), ("query_ptr", (256, 8, 128), F16),
                  ("key_cache_ptr", (6, 64, 2, 128), F16), ("value_cache_ptr", (6, 64, 2, 128), F16),
                  ("block_tables_ptr", (1, 6), np.dtype(np.int32))],
                 dict(cur_batch_start_index=0, block_table_offset=0, num_tiles=6, context_len=128, scale=np.float32(0.1)))
    a = sess.plan.statements[0].args
    assert sess.plan.statements[0].kind == "attention_fwd"
    assert (a.seq_q, a.heads, a.kv_group, a.causal_delta, a.page, a.num_tiles) == (256, 8, 4, 128, 64, 6)


def test_generic_opcode_tables_agree_between_host_and_device():
    """``lower_generic.EW_OPS`` is the order of the ``G_*`` enum in ``csrc/generic_ops.cu``."""
    from ktir_cpu_b200.lower_generic import EW_OPS
    text = open(os.path.join(ROOT, "ktir_cpu_b200", "csrc", "generic_ops.cu")).read()
    names = re.search(r"enum \{ (G_MOV.*?) \};", text, re.S).group(1).replace("\n", " ").split(",")
    assert [n.strip()[2:].lower() for n in names] == [o.rstrip("_") for o in EW_OPS]

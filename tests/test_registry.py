"""The op plug-in seam: an op the backend does not know is added from outside and runs through the
same lowering (here checked on the NumPy stand-in for the device steps and on a plan-only device)."""
import numpy as np
import pytest

import gen_emulator  # noqa: F401  (path set-up)
from ktir_cpu_b200 import KTIRParser, Unsupported, register, runtime as R
from ktir_cpu_b200.interpreter import Session
from ktir_cpu_b200.latency import HardwareConfig, LatencyCategory
from ktir_cpu_b200.registry import unregister
from test_generic_lowering import run_generic

SRC = """module {
  func.func @leaky(%x_ptr: index, %y_ptr: index) attributes {grid = [4, 1]} {
    %c = ktdp.get_compute_tile_id : index
    %c0 = arith.constant 0 : index
    %xv = ktdp.construct_memory_view %x_ptr, sizes: [4, 64], strides: [64, 1] {
      coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 63 >= 0)>, memory_space = #ktdp.memory_space<global>
    } : memref<4x64xf16>
    %yv = ktdp.construct_memory_view %y_ptr, sizes: [4, 64], strides: [64, 1] {
      coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 63 >= 0)>, memory_space = #ktdp.memory_space<global>
    } : memref<4x64xf16>
    %xt = ktdp.construct_access_tile %xv[%c, %c0] {
      access_tile_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 0 >= 0, d1 >= 0, -d1 + 63 >= 0)>, access_tile_order = affine_map<(d0, d1) -> (d0, d1)>
    } : memref<4x64xf16> -> !ktdp.access_tile<1x64xindex>
    %yt = ktdp.construct_access_tile %yv[%c, %c0] {
      access_tile_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 0 >= 0, d1 >= 0, -d1 + 63 >= 0)>, access_tile_order = affine_map<(d0, d1) -> (d0, d1)>
    } : memref<4x64xf16> -> !ktdp.access_tile<1x64xindex>
    %x = ktdp.load %xt : !ktdp.access_tile<1x64xindex> -> tensor<1x64xf16>
    %y = mylib.leaky_relu %x {slope = 0.25} : tensor<1x64xf16>
    ktdp.store %y, %yt : tensor<1x64xf16>, !ktdp.access_tile<1x64xindex>
    return
  }
}
"""


@pytest.fixture
def leaky():
    @register("mylib.leaky_relu", latency_category=LatencyCategory.COMPUTE_FLOAT)
    def leaky_relu(op, context, env):
        x = context.get_value(op.operands[0])
        assert list(context.core_id) == [0, 1, 2, 3] and context.num_cores == 4
        slope = env.constant(op.attrs.get("slope", 0.01), like=x)
        return env.elementwise("arith.maximumf", x, env.elementwise("arith.mulf", x, slope))
    yield
    unregister("mylib.leaky_relu")


def test_unregistered_op_is_unknown():
    with pytest.raises((ValueError, Exception), match="Unknown operation|mylib"):
        func = KTIRParser().parse_module(SRC).get_function("leaky")
        Session(R.PlanOnlyDevice(), func, [("x_ptr", (4, 64), np.dtype("f2")), ("y_ptr", (4, 64), np.dtype("f2"))], {})


def test_registered_op_is_traced_lowered_and_charged(leaky):
    x = np.linspace(-4, 4, 256).astype(np.float16).reshape(4, 64)
    got, _ = run_generic(SRC, "leaky", dict(x_ptr=x, y_ptr=np.zeros_like(x)))
    want = np.maximum(x, (x * np.float16(0.25)).astype(np.float16))
    np.testing.assert_array_equal(got["y_ptr"], want)
    func = KTIRParser().parse_module(SRC).get_function("leaky")
    sess = Session(R.PlanOnlyDevice(), func, [("x_ptr", (4, 64), np.dtype("f2")), ("y_ptr", (4, 64), np.dtype("f2"))], {},
                   latency=True)
    assert [s.kind for s in sess.plan.statements] == ["ew_stream"]          # fused like a built-in elementwise op
    mine = [r for r in sess.latency_records if r.op_type == "mylib.leaky_relu"]
    assert len(mine) == 1 and mine[0].category == LatencyCategory.COMPUTE_FLOAT and mine[0].n_elems == 64

"""The NumPy oracle against outputs of the unmodified reference interpreter (tests/golden)."""
import numpy as np
import pytest

from conftest import golden_names, load_golden
from oracle.numpy_interp import OracleInterpreter


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_fixture(name):
    src, fn, kwargs, expected = load_golden(name)
    interp = OracleInterpreter()
    interp.load(src)
    got = interp.execute_function(fn, **kwargs)
    assert set(got) == set(expected)
    for k in expected:
        # bit-exact, including f16 transcendentals on the generating host's NumPy build;
        # softmax fixtures allow 1 f16 ulp because np.exp(f16) is host-dependent
        if "softmax_f16" in name:
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32),
                                       rtol=2e-3, atol=1e-6)
        else:
            np.testing.assert_array_equal(got[k], expected[k])


def test_inputs_are_not_mutated_and_outputs_are_fresh():
    src, fn, kwargs, _ = load_golden("vector_add_4096")
    before = {k: v.copy() for k, v in kwargs.items() if isinstance(v, np.ndarray)}
    interp = OracleInterpreter()
    interp.load(src)
    got = interp.execute_function(fn, **kwargs)
    for k, v in before.items():
        np.testing.assert_array_equal(kwargs[k], v)
        assert got[k] is not kwargs[k]


def test_scatter_last_writer_wins():
    """Known-answer case of the reference's collision test (tests/test_indirect_access.py:405-441):
    every destination index is 0, so the last enumerated source row wins."""
    src = """module { func.func @scatter(%x: index, %i: index, %y: index) attributes {grid = [1]} {
      %c0 = arith.constant 0 : index
      %xv = ktdp.construct_memory_view %x, sizes: [4, 4], strides: [4, 1] {
        coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 3 >= 0)>,
        memory_space = #ktdp.memory_space<global>} : memref<4x4xf16>
      %iv = ktdp.construct_memory_view %i, sizes: [4], strides: [1] {
        coordinate_set = affine_set<(d0) : (d0 >= 0, -d0 + 3 >= 0)>,
        memory_space = #ktdp.memory_space<global>} : memref<4xi32>
      %yv = ktdp.construct_memory_view %y, sizes: [4, 4], strides: [4, 1] {
        coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 3 >= 0)>,
        memory_space = #ktdp.memory_space<global>} : memref<4x4xf16>
      %xt = ktdp.construct_access_tile %xv[%c0, %c0] {
        access_tile_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 3 >= 0)>,
        access_tile_order = affine_map<(d0, d1) -> (d0, d1)>} : memref<4x4xf16> -> !ktdp.access_tile<4x4xindex>
      %yt = ktdp.construct_indirect_access_tile intermediate_variables(%m, %k)
        %yv[ind(%iv[%m]), (%k)] {
        variables_space_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 3 >= 0, d1 >= 0, -d1 + 3 >= 0)>,
        variables_space_order = affine_map<(d0, d1) -> (d0, d1)>}
        : memref<4x4xf16>, memref<4xi32> -> !ktdp.access_tile<4x4xindex>
      %t = ktdp.load %xt : !ktdp.access_tile<4x4xindex> -> tensor<4x4xf16>
      ktdp.store %t, %yt : tensor<4x4xf16>, !ktdp.access_tile<4x4xindex>
      return } }"""
    x = np.arange(16, dtype=np.float16).reshape(4, 4)
    interp = OracleInterpreter()
    interp.load(src)
    got = interp.execute_function("scatter", x=x, i=np.zeros(4, np.int32), y=np.full((4, 4), -1, np.float16))
    np.testing.assert_array_equal(got["y"][0], x[3])
    np.testing.assert_array_equal(got["y"][1:], np.full((3, 4), -1, np.float16))


def test_negative_index_raises():
    src, fn, kwargs, _ = load_golden("gather_scale_scatter_256")
    kwargs["idx_ptr"] = kwargs["idx_ptr"].copy()
    kwargs["idx_ptr"][5] = -3
    interp = OracleInterpreter()
    interp.load(src)
    with pytest.raises(IndexError, match="negative"):
        interp.execute_function(fn, **kwargs)


def test_deadlock_message_when_a_core_skips_the_exchange():
    """The message of the reference's scheduler (ktir_cpu/grid.py:615-621), core by core."""
    from ktir_cpu_b200 import kernels as K
    interp = OracleInterpreter()
    interp.load(K.ring_allreduce(4, 4, 128, absent_core=2))
    x = np.ones((4, 128), np.float16)
    with pytest.raises(RuntimeError, match="Deadlock detected: core 3 waiting on recv from core 2; core 0 waiting on recv "
                                           "from core 3; core 1 waiting on recv from core 0"):
        interp.execute_function("ring_allreduce", in_ptr=x, out_ptr=np.zeros_like(x))

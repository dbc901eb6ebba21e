"""CUDA path vs. the oracle and the reference fixtures, through the public API / C ABI."""
import numpy as np
import pytest

from conftest import golden_names, load_golden
from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import KTIRInterpreter
from oracle.numpy_interp import OracleInterpreter

pytestmark = pytest.mark.gpu

# f16 ulp-level tolerance for paths containing exp/sum (exp differs from NumPy's by <= 1 ulp)
TOL = dict(rtol=2e-3, atol=2e-6)


def _run_both(src, fn, kwargs):
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function(fn, **kwargs)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function(fn, **kwargs)
    gpu.close()
    return got, want


def _exact(name):
    return name.startswith(("vector_add", "gather"))


SUPPORTED = [n for n in golden_names() if n.startswith(("vector_add", "softmax"))]


@pytest.mark.parametrize("name", SUPPORTED)
def test_gpu_matches_reference_fixture(name, build_lib):
    src, fn, kwargs, expected = load_golden(name)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function(fn, **kwargs)
    gpu.close()
    assert set(got) == set(expected)
    for k in expected:
        assert got[k].dtype == expected[k].dtype and got[k].shape == expected[k].shape
        if _exact(name):
            np.testing.assert_array_equal(got[k], expected[k])
        else:
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32), **TOL)


def test_vector_add_bit_exact_and_inputs_untouched(build_lib):
    rng = np.random.default_rng(11)
    n = 1 << 20
    x = rng.standard_normal(n).astype(np.float16)
    y = (rng.standard_normal(n) * 100).astype(np.float16)
    x[:4] = [np.inf, -np.inf, np.nan, 6.1e-5]
    x0, y0 = x.copy(), y.copy()
    out = np.full(n, 7, np.float16)
    got, want = _run_both(K.vector_add(n, 4096, 32), "add_kernel",
                          dict(x_ptr=x, y_ptr=y, output_ptr=out, BLOCK_SIZE=4096))
    np.testing.assert_array_equal(got["output_ptr"], want["output_ptr"])
    np.testing.assert_array_equal(got["x_ptr"], x0)
    np.testing.assert_array_equal(x, x0)
    np.testing.assert_array_equal(y, y0)
    assert got["x_ptr"] is not x and (out == 7).all()


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("shape,cores,r", [((128, 4096), 4, 8), ((64, 64), 2, 1), ((32, 16384), 2, 1)])
def test_softmax_matches_oracle(f32, shape, cores, r, build_lib):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(shape) * 2).astype(np.float16)
    got, want = _run_both(K.softmax_rows(shape[0], shape[1], cores, r, f32), "softmax_kernel",
                          dict(output_ptr=np.zeros_like(x), input_ptr=x))
    np.testing.assert_allclose(got["output_ptr"].astype(np.float32), want["output_ptr"].astype(np.float32),
                               rtol=2e-3 if f32 else 1e-2, atol=2e-6 if f32 else 1e-5)
    # size-independent property: every row sums to one
    np.testing.assert_allclose(got["output_ptr"].astype(np.float64).sum(1), 1.0, atol=5e-3)


def test_softmax_full_size_properties(build_lib):
    """BASELINE size (8192 x 4096): rows sum to 1, order of elements follows the input."""
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((8192, 4096)) * 2).astype(np.float16)
    gpu = KTIRInterpreter()
    gpu.load(K.softmax_rows(8192, 4096, 32, 8, True))
    y = gpu.execute_function("softmax_kernel", output_ptr=np.zeros_like(x), input_ptr=x)["output_ptr"]
    gpu.close()
    np.testing.assert_allclose(y.astype(np.float64).sum(1), 1.0, atol=5e-3)
    rows = rng.integers(0, 8192, 64)
    xf = x[rows].astype(np.float32)
    e = np.exp(xf - xf.max(1, keepdims=True))
    np.testing.assert_allclose(y[rows].astype(np.float32), e / e.sum(1, keepdims=True), rtol=2e-3, atol=2e-6)
    assert (np.argmax(y, 1) == np.argmax(x, 1)).mean() > 0.99

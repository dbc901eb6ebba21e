"""Every elementwise op of the arith / math dialects on the device against the oracle, over ALL f16
bit patterns: once through the fused register-program kernel, once through the step-by-step path."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import KTIRInterpreter
from oracle.numpy_interp import OracleInterpreter

pytestmark = pytest.mark.gpu

EXACT_OPS = ["add", "sub", "mul", "div", "maximum", "maxnum", "minimum", "minnum", "neg", "abs", "sqrt", "rsqrt"]
ULP_OPS = ["exp", "log", "log2", "tanh", "sin", "cos", "erf"]
# second operands: zeros of both signs, +-1, a subnormal, the largest finite value, inf, nan and ordinary values
Y_BITS = [0x0000, 0x8000, 0x3c00, 0xbc00, 0x0001, 0x83ff, 0x7bff, 0xfbff, 0x7c00, 0xfc00, 0x7e00, 0x3555, 0x4200,
          0xc500, 0x1400, 0x6400]


def assert_same_bits(got, want, what=""):
    """Same NaN positions; everywhere else the same bits (so -0 and +0 differ)."""
    g, w = np.ascontiguousarray(got), np.ascontiguousarray(want)
    assert g.dtype == w.dtype and g.shape == w.shape, what
    nan = np.isnan(w)
    np.testing.assert_array_equal(np.isnan(g), nan, err_msg=what)
    ui = {2: np.uint16, 4: np.uint32}[g.dtype.itemsize]
    bad = (g.view(ui) != w.view(ui)) & ~nan
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} differ, first at {np.flatnonzero(bad.reshape(-1))[:4]}"


def ulp_distance_f16(got, want):
    """Distance in f16 steps on the monotone integer line (NaN positions must agree, they count as 0)."""
    def key(a):
        b = a.view(np.uint16).astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7fff), b)
    nan = np.isnan(want)
    np.testing.assert_array_equal(np.isnan(got), nan)
    return np.where(nan, 0, np.abs(key(got) - key(want)))


def _run(src, kw, fused):
    gpu = KTIRInterpreter(fused_kernels=fused)
    gpu.load(src)
    got = gpu.execute_function("elementwise_kernel", **kw)
    kinds = {s.kind for sess in gpu._sessions.values() for s in sess.plan.statements}
    gpu.close()
    ora = OracleInterpreter()
    ora.load(src)
    with np.errstate(all="ignore"):
        want = ora.execute_function("elementwise_kernel", **kw)
    return got, want, kinds


def _all_patterns():
    x = np.tile(np.arange(65536, dtype=np.uint16), len(Y_BITS))
    y = np.repeat(np.array(Y_BITS, np.uint16), 65536)
    return x.view(np.float16), y.view(np.float16)


@pytest.mark.parametrize("fused", [True, False], ids=["register_program", "step_by_step"])
def test_f16_ops_bit_exact_on_every_bit_pattern(fused, build_lib):
    x, y = _all_patterns()
    n = x.size
    src = K.elementwise_suite(EXACT_OPS, n, 4096, 32, "f16", "olt")
    names = [f"out_{o}_ptr" for o in EXACT_OPS] + ["out_select_ptr", "out_ext_add_ptr"]
    kw = dict(x_ptr=x, y_ptr=y, **{k: np.zeros(n, np.float16) for k in names})
    got, want, kinds = _run(src, kw, fused)
    assert ("ew_stream" in kinds) == fused and ("generic" in kinds or fused)
    for k in names:
        assert_same_bits(got[k], want[k], k)
    assert_same_bits(got["x_ptr"], x, "input x returned unchanged")


@pytest.mark.parametrize("pred", ["oeq", "ogt", "ole", "one", "une", "ult", "ord", "uno"])
def test_f16_compare_select_bit_exact(pred, build_lib):
    x, y = _all_patterns()
    n = x.size
    src = K.elementwise_suite([], n, 4096, 32, "f16", pred)
    kw = dict(x_ptr=x, y_ptr=y, out_select_ptr=np.zeros(n, np.float16), out_ext_add_ptr=np.zeros(n, np.float16))
    got, want, _ = _run(src, kw, True)
    assert_same_bits(got["out_select_ptr"], want["out_select_ptr"], pred)


_F64 = {"exp": np.exp, "log": np.log, "log2": np.log2, "tanh": np.tanh, "sin": np.sin, "cos": np.cos}


@pytest.mark.parametrize("fused", [True, False], ids=["register_program", "step_by_step"])
def test_f16_transcendentals_on_every_bit_pattern(fused, build_lib):
    """The device computes in f32 and rounds once, so it must sit within 1 f16 step of the correctly
    rounded value.  NumPy's half-precision loops are host-dependent (2-3 steps off correct rounding
    on AVX-512 hosts), so against the oracle the allowance is the oracle's own distance plus one.
    erf is a chain of ~20 f16 roundings around one exp (cancelling near 0): absolute tolerance."""
    x = np.arange(65536, dtype=np.uint16).view(np.float16)
    n = x.size
    src = K.elementwise_suite(ULP_OPS, n, 2048, 32, "f16")
    names = [f"out_{o}_ptr" for o in ULP_OPS]
    kw = dict(x_ptr=x, y_ptr=x, out_ext_add_ptr=np.zeros(n, np.float16), **{k: np.zeros(n, np.float16) for k in names})
    got, want, _ = _run(src, kw, fused)
    for o in ULP_OPS:
        g, w = got[f"out_{o}_ptr"], want[f"out_{o}_ptr"]
        if o == "erf":
            np.testing.assert_array_equal(np.isnan(g), np.isnan(w))
            np.testing.assert_allclose(g.astype(np.float32), w.astype(np.float32), rtol=0, atol=2e-3)
            continue
        with np.errstate(all="ignore"):
            correct = _F64[o](x.astype(np.float64)).astype(np.float16)
        d_correct = ulp_distance_f16(g, correct)
        assert d_correct.max() <= 1, f"{o}: {int(d_correct.max())} steps from correct rounding at {int(d_correct.argmax()):#06x}"
        slack = ulp_distance_f16(w, correct) + 1
        d = ulp_distance_f16(g, w)
        assert (d <= slack).all(), f"{o}: {int((d - slack).max())} steps beyond the oracle's own error at {int((d - slack).argmax()):#06x}"


@pytest.mark.parametrize("fused", [True, False], ids=["register_program", "step_by_step"])
def test_f32_ops_bit_exact(fused, build_lib):
    rng = np.random.default_rng(11)
    n = 1 << 18
    x = (rng.standard_normal(n) * np.exp2(rng.integers(-30, 30, n))).astype(np.float32)
    y = (rng.standard_normal(n) * np.exp2(rng.integers(-30, 30, n))).astype(np.float32)
    x[:6] = [np.inf, -np.inf, np.nan, 1e-42, 3.0e38, -3.0e38]          # specials; no (+0, -0) pairs: NumPy's
    y[:6] = [np.inf, np.inf, 1.0, 1e-42, 3.0e38, 3.0e38]                # f32 SIMD max/min tie rule is host-dependent
    ops = ["add", "sub", "mul", "div", "maximum", "maxnum", "minimum", "minnum", "neg", "abs", "sqrt"]
    src = K.elementwise_suite(ops, n, 4096, 32, "f32", "olt")
    names = [f"out_{o}_ptr" for o in ops] + ["out_select_ptr"]
    kw = dict(x_ptr=x, y_ptr=y, **{k: np.zeros(n, np.float32) for k in names})
    got, want, _ = _run(src, kw, fused)
    for k in names:
        assert_same_bits(got[k], want[k], k)

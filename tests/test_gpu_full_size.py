"""The benchmark configurations at their full sizes, device result against the oracle itself
(whole array where the oracle finishes in seconds, whole slabs / heads of it otherwise)."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import KTIRInterpreter
from oracle.numpy_interp import OracleInterpreter

pytestmark = pytest.mark.gpu


def _oracle(src, fn, **kw):
    o = OracleInterpreter()
    o.load(src)
    return o.execute_function(fn, **kw)


def test_softmax_8192x4096_whole_array_against_oracle(build_lib):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((8192, 4096), dtype=np.float32) * 2).astype(np.float16)
    src = K.softmax_rows(8192, 4096, 32, 8, True)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("softmax_kernel", output_ptr=np.zeros_like(x), input_ptr=x)
    gpu.close()
    want = _oracle(src, "softmax_kernel", output_ptr=np.zeros_like(x), input_ptr=x)
    # f32 statistics on both sides; the f16 result may differ by one rounding step
    np.testing.assert_allclose(got["output_ptr"].astype(np.float32), want["output_ptr"].astype(np.float32),
                               rtol=2e-3, atol=2e-6)
    np.testing.assert_array_equal(got["input_ptr"], x)


def test_matmul_4096_row_slabs_against_oracle(build_lib):
    """C = A B at 4096^3 on the device; the oracle runs the same kernel text on two 256-row slabs of A
    (an output row depends on its own row of A only, and the K order is the same)."""
    rng = np.random.default_rng(4)
    a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    gpu = KTIRInterpreter()
    gpu.load(K.tiled_matmul(4096, 4096, 4096, 64, 64, 64, 32, True))
    c = gpu.execute_function("matmul_kernel", a_ptr=a, b_ptr=b, c_ptr=np.zeros((4096, 4096), np.float16))["c_ptr"]
    gpu.close()
    slab_src = K.tiled_matmul(256, 4096, 4096, 64, 64, 64, 32, True)
    for r0 in (0, 3840):
        want = _oracle(slab_src, "matmul_kernel", a_ptr=np.ascontiguousarray(a[r0:r0 + 256]), b_ptr=b,
                       c_ptr=np.zeros((256, 4096), np.float16))["c_ptr"]
        # f32 accumulation on both sides; summation order differs: at most one f16 step at |C| <= 64
        np.testing.assert_allclose(c[r0:r0 + 256].astype(np.float32), want.astype(np.float32), rtol=2e-3, atol=1e-2)


def test_causal_attention_B8_H32_S2048_heads_against_oracle(build_lib):
    """The full attention configuration (batch 8 x 32 heads folded into 256 heads, S = 2048, D = 128,
    tiles 128 x 128) on the device; the oracle runs the same kernel shape on single heads of it."""
    S, H, D, T = 2048, 256, 128, 128
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((S, H, D), dtype=np.float32).astype(np.float16) for _ in range(3))
    nt = S // T
    kw = dict(query_ptr=q, key_cache_ptr=k.reshape(nt, T, H, D), value_cache_ptr=v.reshape(nt, T, H, D),
              block_tables_ptr=np.arange(nt, dtype=np.int32).reshape(1, -1), cur_batch_start_index=0,
              block_table_offset=0, num_tiles=nt, context_len=0, scale=np.float32(1.0 / np.sqrt(D)))
    gpu = KTIRInterpreter()
    gpu.load(K.paged_attention(S, S, H, H, D, T, T))
    o = gpu.execute_function("paged_attention_kernel", output_ptr=np.zeros_like(q), **kw)["output_ptr"]
    kinds = [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]
    gpu.close()
    assert kinds == ["attention_fwd"]
    one = K.paged_attention(S, S, 1, 1, D, T, T)
    for h in (0, 131, 255):
        kw1 = dict(kw, query_ptr=np.ascontiguousarray(q[:, h:h + 1]),
                   key_cache_ptr=np.ascontiguousarray(kw["key_cache_ptr"][:, :, h:h + 1]),
                   value_cache_ptr=np.ascontiguousarray(kw["value_cache_ptr"][:, :, h:h + 1]))
        want = _oracle(one, "paged_attention_kernel", output_ptr=np.zeros((S, 1, D), np.float16), **kw1)["output_ptr"]
        # the device rounds the probabilities to f16 before the second matmul (<= 2^-11 relative)
        np.testing.assert_allclose(o[:, h].astype(np.float32), want[:, 0].astype(np.float32), rtol=1e-2, atol=2e-3)

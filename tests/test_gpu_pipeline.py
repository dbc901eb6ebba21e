"""Pipelined execute_function (split plans, three streams, staged uploads) against the plain
upload / launch / read-back sequence: bit-identical results, fresh arrays, inputs untouched."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import KTIRInterpreter

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def small_parts(monkeypatch):
    """4 MiB per part instead of the default, so that these sizes split into many parts."""
    from ktir_cpu_b200.interpreter import Session
    monkeypatch.setattr(Session, "PIPELINE_PIECE", 4 << 20)


def _both(src, fn, kw):
    gpu = KTIRInterpreter()
    gpu.load(src)
    before = {k: v.copy() for k, v in kw.items() if isinstance(v, np.ndarray)}
    got = gpu.execute_function(fn, **kw)
    sess, kw2 = gpu.session(fn, **kw)
    tp = sess.transfer_plan()
    arrays = {k: v for k, v in kw2.items() if isinstance(v, np.ndarray)}
    plain = gpu._execute_simple(sess, arrays, {})
    again = gpu.execute_function(fn, **kw)            # result buffers are recycled between calls
    for k, v in before.items():
        np.testing.assert_array_equal(kw[k], v)      # inputs untouched
        assert got[k] is not kw[k] and not np.shares_memory(got[k], kw[k])
        assert got[k].view(np.uint8).tobytes() == plain[k].view(np.uint8).tobytes(), k
        assert again[k].view(np.uint8).tobytes() == plain[k].view(np.uint8).tobytes(), k
    gpu.close()
    return tp


def test_softmax_pipelined_equals_plain(build_lib):
    x = (np.random.default_rng(0).standard_normal((4096, 4096), dtype=np.float32) * 2).astype(np.float16)
    tp = _both(K.softmax_rows(4096, 4096, 32, 8, True), "softmax_kernel", dict(output_ptr=np.zeros_like(x), input_ptr=x))
    assert tp.split and len(tp.chunks) >= 8


def test_vector_add_pipelined_equals_plain(build_lib):
    rng = np.random.default_rng(1)
    n = 1 << 23
    x, y = (rng.standard_normal(n, dtype=np.float32).astype(np.float16) for _ in range(2))
    tp = _both(K.vector_add(n, 16384, 32), "add_kernel", dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(n, np.float16), BLOCK_SIZE=16384))
    assert tp.split


def test_matmul_pipelined_equals_plain(build_lib):
    rng = np.random.default_rng(2)
    M = 2048
    a, b = (rng.uniform(-1, 1, (M, M)).astype(np.float16) for _ in range(2))
    tp = _both(K.tiled_matmul(M, M, M, 64, 64, 64, 32, True), "matmul_kernel",
               dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((M, M), np.float16)))
    assert tp.split


@pytest.mark.parametrize("H,Hkv", [(32, 32), (32, 8)])
def test_attention_pipelined_equals_plain(H, Hkv, build_lib):
    rng = np.random.default_rng(3)
    S, T, D = 1024, 128, 128
    nt = S // T
    q = rng.standard_normal((S, H, D), dtype=np.float32).astype(np.float16)
    kc, vc = (rng.standard_normal((nt, T, Hkv, D), dtype=np.float32).astype(np.float16) for _ in range(2))
    tp = _both(K.paged_attention(S, S, H, Hkv, D, T, T // (H // Hkv)), "paged_attention_kernel",
               dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=kc, value_cache_ptr=vc,
                    block_tables_ptr=rng.permutation(nt).astype(np.int32).reshape(1, -1), cur_batch_start_index=0,
                    block_table_offset=0, num_tiles=nt, context_len=0, scale=np.float32(1.0 / np.sqrt(D))))
    assert tp.split


def test_scatter_runs_as_one_part_and_accumulates_from_the_given_output(build_lib):
    rng = np.random.default_rng(4)
    table = rng.standard_normal((8192, 128), dtype=np.float32).astype(np.float16)
    idx = rng.integers(0, 8192, 65536).astype(np.int32)
    out0 = rng.standard_normal((8192, 128), dtype=np.float32).astype(np.float16)
    tp = _both(K.gather_scale_scatter(8192, 128, 65536, 64, 8), "gather_scale_scatter",
               dict(table_ptr=table, idx_ptr=idx, out_ptr=out0))
    assert not tp.split


def test_non_contiguous_and_read_only_inputs(build_lib):
    rng = np.random.default_rng(5)
    big = (rng.standard_normal((2048, 8192), dtype=np.float32) * 2).astype(np.float16)
    x = big[:, ::2]                                    # a strided view
    x.flags.writeable = False
    _both(K.softmax_rows(2048, 4096, 32, 8, True), "softmax_kernel", dict(output_ptr=np.zeros((2048, 4096), np.float16), input_ptr=x))

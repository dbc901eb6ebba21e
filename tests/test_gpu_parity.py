"""CUDA path vs. the oracle and the reference fixtures, through the public API / C ABI."""
import numpy as np
import pytest

from conftest import golden_names, load_golden
from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import kernels as K_
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
    return name.startswith(("vector_add", "gather", "ring_allreduce", "shared_slot", "sharded_", "paged_gather", "region_reduce", "generic_contraction", "update_in_place", "core_chain", "accumulate_rows", "rmsnorm_weighted", "layernorm_blocked"))


SUPPORTED = golden_names()


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
        if name.startswith("elementwise"):
            from test_gpu_elementwise import assert_same_bits
            if "erf" in k:          # a chain of f16 roundings around one host-dependent exp, cancelling near 0
                np.testing.assert_array_equal(np.isnan(got[k]), np.isnan(expected[k]))
                np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32), rtol=0, atol=2e-3)
            else:
                assert_same_bits(got[k], expected[k], k)
        elif _exact(name):
            np.testing.assert_array_equal(got[k], expected[k])
        elif name.startswith("matmul_f32acc"):
            # f32 accumulation on both sides, only the summation order differs: <= 1 f16 ulp
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32),
                                       rtol=2e-3, atol=1e-2)
        elif name.startswith(("causal_attention", "paged_attention")):
            # probabilities pass through f16 before the second matmul (<= 2^-11 relative)
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32),
                                       rtol=1e-2, atol=2e-3)
        elif name.startswith("matmul_f16acc"):
            # the reference rounds to f16 at every K-step; tolerance of its own matmul test
            # (tests/test_examples.py:468 of the reference)
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32),
                                       rtol=2e-2, atol=2e-1)
        else:
            np.testing.assert_allclose(got[k].astype(np.float32), expected[k].astype(np.float32), **TOL)


@pytest.mark.parametrize("fused", [True, False])
def test_colliding_stores_keep_the_last_core(fused, build_lib):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((40, 256)).astype(np.float16)
    src = K.shared_slot_store(40, 7, 256)
    gpu = KTIRInterpreter(fused_kernels=fused)
    gpu.load(src)
    got = gpu.execute_function("shared_slot", x_ptr=x, out_ptr=np.zeros((7, 256), np.float16))["out_ptr"]
    gpu.close()
    want = np.stack([(x[max(c for c in range(40) if c % 7 == s)] * np.float16(2)) for s in range(7)])
    np.testing.assert_array_equal(got, want)
    ora = OracleInterpreter()
    ora.load(src)
    np.testing.assert_array_equal(got, ora.execute_function("shared_slot", x_ptr=x, out_ptr=np.zeros((7, 256), np.float16))["out_ptr"])


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


@pytest.mark.parametrize("rows,cols,cores,r", [(2405, 1024, 5, 13), (2400, 2048, 4, 8), (2372, 4096, 4, 1)])
def test_softmax_many_ragged_rows(rows, cols, cores, r, build_lib):
    """Thousands of rows of 2 .. 8 KB with row counts that are no multiple of the rows a CTA takes per
    iteration and row tiles that straddle them; a constant row and a row with one huge value."""
    rng = np.random.default_rng(rows)
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float16)
    x[7] = 0                      # a constant row: every element 1 / cols
    x[11, 5] = np.float16(60000)  # one huge value: that element takes everything
    gpu = KTIRInterpreter()
    gpu.load(K.softmax_rows(rows, cols, cores, r, True))
    y = gpu.execute_function("softmax_kernel", output_ptr=np.full_like(x, 9), input_ptr=x)["output_ptr"]
    gpu.close()
    xf = x.astype(np.float32)
    e = np.exp(xf - xf.max(1, keepdims=True))
    np.testing.assert_allclose(y.astype(np.float32), e / e.sum(1, keepdims=True), rtol=2e-3, atol=2e-6)
    assert y[11, 5] == 1 and (np.delete(y[11], 5) == 0).all()


def _dup_indices(rng, n_rows, n_idx, tile_rows, dup):
    idx = rng.integers(0, n_rows, n_idx)
    for t in range(n_idx // tile_rows):
        pos = rng.choice(tile_rows, 2 * dup, replace=False)
        idx[t * tile_rows + pos[:dup]] = idx[t * tile_rows + pos[dup:]]
    return idx


@pytest.mark.parametrize("idx_dtype", ["i32", "i64"])
def test_gather_rows_bit_exact(idx_dtype, build_lib):
    rng = np.random.default_rng(7)
    table = rng.standard_normal((512, 128)).astype(np.float16)
    idx = rng.integers(0, 512, 4096).astype(np.int32 if idx_dtype == "i32" else np.int64)
    got, want = _run_both(K.gather_rows(512, 128, 4096, 64, 8, idx_dtype), "gather_rows",
                          dict(table_ptr=table, idx_ptr=idx, out_ptr=np.zeros((4096, 128), np.float16)))
    np.testing.assert_array_equal(got["out_ptr"], want["out_ptr"])
    np.testing.assert_array_equal(got["out_ptr"], table[idx])


@pytest.mark.parametrize("cols,tile_rows", [(128, 64), (32, 16), (20, 8)])
def test_scatter_rows_last_writer_wins(cols, tile_rows, build_lib):
    rng = np.random.default_rng(8)
    n_idx = tile_rows * 64
    src = rng.standard_normal((n_idx, cols)).astype(np.float16)
    idx = _dup_indices(rng, 96, n_idx, tile_rows, max(1, tile_rows // 8)).astype(np.int32)
    got, want = _run_both(K.scatter_rows(96, cols, n_idx, tile_rows, 4), "scatter_rows",
                          dict(src_ptr=src, idx_ptr=idx, out_ptr=np.full((96, cols), -1, np.float16)))
    np.testing.assert_array_equal(got["out_ptr"], want["out_ptr"])


@pytest.mark.parametrize("n_rows,n_idx", [(1024, 16384), (64, 8192), (1, 1024)])
def test_gather_scale_scatter_ordered_rmw(n_rows, n_idx, build_lib):
    """Heavy row reuse: the tile-sequential read-modify-write order must be reproduced bit for bit."""
    rng = np.random.default_rng(9)
    table = rng.standard_normal((n_rows, 128)).astype(np.float16)
    idx = _dup_indices(rng, n_rows, n_idx, 64, 6).astype(np.int32)
    kw = dict(table_ptr=table, idx_ptr=idx, out_ptr=rng.standard_normal((n_rows, 128)).astype(np.float16))
    got, want = _run_both(K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8), "gather_scale_scatter", kw)
    np.testing.assert_array_equal(got["out_ptr"], want["out_ptr"])
    # deterministic: a second run on the same inputs gives the same bits
    got2, _ = _run_both(K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8), "gather_scale_scatter", kw)
    np.testing.assert_array_equal(got["out_ptr"], got2["out_ptr"])


def test_one_row_hit_by_a_thousand_tiles_is_ordered_and_quick(build_lib):
    """Far more tiles land on one destination row than a bucket holds: the row's entries are collected
    and ordered once, then replayed.  Bit-exact against the oracle (1024 f16 roundings in tile order)
    and finished in well under a second."""
    import time
    rng = np.random.default_rng(12)
    n_rows, n_idx = 64, 65536
    table = rng.standard_normal((n_rows, 128)).astype(np.float16)
    idx = rng.integers(0, n_rows, n_idx).astype(np.int32)
    idx[::64] = 3                                   # every tile hits row 3 ...
    idx[1::64] = 3                                  # ... twice (the later entry of a tile wins)
    idx[5::128] = 9                                 # and every other tile row 9
    src = K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8)
    kw = dict(table_ptr=table, idx_ptr=idx, out_ptr=rng.standard_normal((n_rows, 128)).astype(np.float16))
    gpu = KTIRInterpreter()
    gpu.load(src)
    gpu.execute_function("gather_scale_scatter", **kw)
    t0 = time.perf_counter()
    got = gpu.execute_function("gather_scale_scatter", **kw)
    dt = time.perf_counter() - t0
    gpu.close()
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("gather_scale_scatter", **kw)
    np.testing.assert_array_equal(got["out_ptr"], want["out_ptr"])
    assert dt < 1.0, f"{dt:.3f} s"


def test_cached_plan_replayed_as_graph_follows_new_inputs(build_lib):
    """From its second run on a multi-launch plan is replayed as one CUDA graph: every replay must see the
    inputs of its own call (new table, indices and destination), bit for bit like the oracle."""
    n_rows, n_idx = 512, 4096
    src = K.gather_scale_scatter(n_rows, 128, n_idx, 64, 8)
    gpu = KTIRInterpreter()
    gpu.load(src)
    ora = OracleInterpreter()
    ora.load(src)
    for seed in range(4):
        rng = np.random.default_rng(100 + seed)
        kw = dict(table_ptr=rng.standard_normal((n_rows, 128)).astype(np.float16),
                  idx_ptr=_dup_indices(rng, n_rows, n_idx, 64, 6).astype(np.int32),
                  out_ptr=rng.standard_normal((n_rows, 128)).astype(np.float16))
        got = gpu.execute_function("gather_scale_scatter", **kw)
        want = ora.execute_function("gather_scale_scatter", **kw)
        np.testing.assert_array_equal(got["out_ptr"], want["out_ptr"])
    sessions = list(gpu._sessions.values()) if hasattr(gpu, "_sessions") else []
    if sessions:
        assert any(s._graph is not None for s in sessions)      # the replay path was the one exercised
    gpu.close()


def test_negative_index_raises_index_error(build_lib):
    src, fn, kwargs, _ = load_golden("gather_scale_scatter_256")
    kwargs["idx_ptr"] = kwargs["idx_ptr"].copy()
    kwargs["idx_ptr"][5] = -3
    gpu = KTIRInterpreter()
    gpu.load(src)
    with pytest.raises(IndexError, match="negative"):
        gpu.execute_function(fn, **kwargs)
    # the context stays usable after the error
    kwargs["idx_ptr"][5] = 3
    gpu.execute_function(fn, **kwargs)
    gpu.close()


def test_gather_scale_scatter_full_size_properties(build_lib):
    """BASELINE size (65536 x 128 table, 262144 indices): untouched rows stay zero and every
    touched row equals h (+) h ... n times with h = 0.5 * table[row] (f16 rounding per add),
    n = number of tiles containing the row."""
    rng = np.random.default_rng(3)
    table = rng.standard_normal((65536, 128)).astype(np.float16)
    idx = _dup_indices(rng, 65536, 262144, 64, 6).astype(np.int32)
    gpu = KTIRInterpreter()
    gpu.load(K.gather_scale_scatter())
    out = gpu.execute_function("gather_scale_scatter", table_ptr=table, idx_ptr=idx,
                               out_ptr=np.zeros_like(table))["out_ptr"]
    gpu.close()
    tiles = idx.reshape(-1, 64)
    counts = np.zeros(65536, np.int64)
    for t in range(tiles.shape[0]):
        counts[np.unique(tiles[t])] += 1
    assert (out[counts == 0] == 0).all()
    h = (table * np.float16(0.5)).astype(np.float16)
    acc = np.zeros_like(table)
    for n in range(1, int(counts.max()) + 1):
        m = counts >= n
        acc[m] = acc[m] + h[m]
    np.testing.assert_array_equal(out, acc)


@pytest.mark.parametrize("f32_acc", [True, False])
@pytest.mark.parametrize("M,N,K,cores", [(256, 256, 256, 4), (128, 512, 192, 2), (384, 128, 64, 3),
                                         # few tiles: the left-over tiles are cut into half-width units
                                         (512, 1024, 1024, 8), (256, 384, 832, 6)])
def test_tiled_matmul_matches_oracle(M, N, K, cores, f32_acc, build_lib):
    rng = np.random.default_rng(4)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float16)
    src = K_.tiled_matmul(M, N, K, 64, 64, 64, cores, f32_acc)
    got, want = _run_both(src, "matmul_kernel", dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((M, N), np.float16)))
    gpu = KTIRInterpreter()
    gpu.load(src)
    for _ in range(3):                     # every run gives the same bits
        again = gpu.execute_function("matmul_kernel", a_ptr=a, b_ptr=b, c_ptr=np.zeros((M, N), np.float16))
        np.testing.assert_array_equal(again["c_ptr"], got["c_ptr"])
    gpu.close()
    tol = dict(rtol=2e-3, atol=1e-2) if f32_acc else dict(rtol=2e-2, atol=2e-1)
    np.testing.assert_allclose(got["c_ptr"].astype(np.float32), want["c_ptr"].astype(np.float32), **tol)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    np.testing.assert_allclose(got["c_ptr"].astype(np.float64), exact, rtol=2e-3, atol=1e-2)


def test_tiled_matmul_full_size_properties(build_lib):
    """BASELINE size 4096^3: sampled rows/columns against an f64 product, plus linearity in A."""
    rng = np.random.default_rng(4)
    a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    gpu = KTIRInterpreter()
    gpu.load(K_.tiled_matmul(4096, 4096, 4096, 64, 64, 64, 32, True))
    c = gpu.execute_function("matmul_kernel", a_ptr=a, b_ptr=b, c_ptr=np.zeros((4096, 4096), np.float16))["c_ptr"]
    rows = rng.integers(0, 4096, 24)
    cols = rng.integers(0, 4096, 24)
    b64 = b.astype(np.float64)
    np.testing.assert_allclose(c[rows].astype(np.float64), a[rows].astype(np.float64) @ b64, rtol=2e-3, atol=5e-2)
    np.testing.assert_allclose(c[:, cols].astype(np.float64), a.astype(np.float64) @ b64[:, cols], rtol=2e-3, atol=5e-2)
    c2 = gpu.execute_function("matmul_kernel", a_ptr=(a * np.float16(0.5)).astype(np.float16), b_ptr=b,
                              c_ptr=np.zeros((4096, 4096), np.float16))["c_ptr"]
    gpu.close()
    np.testing.assert_allclose(c2.astype(np.float32) * 2, c.astype(np.float32), rtol=2e-3, atol=5e-2)


def _attention_inputs(rng, S, H, D, tn, shuffle_pages=False):
    q, k, v = (rng.standard_normal((S, H, D)).astype(np.float16) for _ in range(3))
    nb = S // tn
    table = np.arange(nb, dtype=np.int32)
    kc, vc = k.reshape(nb, tn, H, D), v.reshape(nb, tn, H, D)
    if shuffle_pages:                       # pages stored in a permuted order, found through the table
        perm = rng.permutation(nb)
        table = np.argsort(perm).astype(np.int32)
        kc, vc = kc[perm], vc[perm]
    kw = dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=np.ascontiguousarray(kc),
              value_cache_ptr=np.ascontiguousarray(vc), block_tables_ptr=table.reshape(1, -1),
              num_tiles=nb, context_len=0, scale=float(1.0 / np.sqrt(D)))
    return q, k, v, kw


def _attention_f64(q, k, v, D):
    qf, kf, vf = (x.astype(np.float64).transpose(1, 0, 2) for x in (q, k, v))
    sc = np.einsum("hqd,hkd->hqk", qf, kf) / np.sqrt(D)
    S = sc.shape[-1]
    sc = np.where(np.tril(np.ones((S, S), bool)), sc, -np.inf)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return np.einsum("hqk,hkd->hqd", p, vf).transpose(1, 0, 2)


@pytest.mark.parametrize("tm,tn", [(32, 32), (64, 128), (128, 64), (128, 128)])
def test_causal_attention_matches_oracle(tm, tn, build_lib):
    rng = np.random.default_rng(5)
    S, H, D = 256, 2, 128
    q, k, v, kw = _attention_inputs(rng, S, H, D, tn, shuffle_pages=True)
    got, want = _run_both(K_.causal_attention(S, H, D, tm, tn), "attention_kernel", kw)
    np.testing.assert_allclose(got["output_ptr"].astype(np.float32), want["output_ptr"].astype(np.float32),
                               rtol=1e-2, atol=2e-3)
    np.testing.assert_allclose(got["output_ptr"].astype(np.float64), _attention_f64(q, k, v, D), rtol=1e-2, atol=2e-3)


def test_causal_attention_long_sequence_properties(build_lib):
    """S = 2048 (BASELINE sequence length, 4 heads): first row attends to one position only,
    every output lies in the convex hull of V, sampled heads match an f64 computation."""
    rng = np.random.default_rng(6)
    S, H, D, tn = 2048, 4, 128, 128
    q, k, v, kw = _attention_inputs(rng, S, H, D, tn)
    gpu = KTIRInterpreter()
    gpu.load(K_.causal_attention(S, H, D, 128, tn))
    o = gpu.execute_function("attention_kernel", **kw)["output_ptr"]
    gpu.close()
    np.testing.assert_allclose(o[0].astype(np.float32), v[0].astype(np.float32), rtol=2e-3, atol=2e-3)
    assert (o.astype(np.float32).max(0) <= v.astype(np.float32).max(0) + 1e-2).all()
    np.testing.assert_allclose(o.astype(np.float64), _attention_f64(q, k, v, D), rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("S,H", [(512, 320), (768, 160), (640, 200)])
def test_causal_attention_many_tiles_per_cta(S, H, build_lib):
    """More work items than SMs, so a persistent CTA walks several tile pairs one after another
    (barrier phases carry over); 768 has an odd number of tile pairs (an item with one half only),
    640 an odd number of tiles (a pair whose second tile does not exist)."""
    rng = np.random.default_rng(S + H)
    D, tn = 128, 128
    q, k, v, kw = _attention_inputs(rng, S, H, D, tn, shuffle_pages=True)
    gpu = KTIRInterpreter()
    gpu.load(K_.causal_attention(S, H, D, 128, tn))
    o = gpu.execute_function("attention_kernel", **kw)["output_ptr"]
    gpu.close()
    np.testing.assert_allclose(o.astype(np.float64), _attention_f64(q, k, v, D), rtol=1e-2, atol=2e-3)


def test_latency_report_through_execute_function(build_lib):
    """With a latency_config the device run also feeds the latency model (same report as the host-only estimate)."""
    from ktir_cpu_b200 import HardwareConfig
    src, fn, kwargs, outs = load_golden("gather_scale_scatter_256")
    gpu = KTIRInterpreter(latency_config=HardwareConfig())
    gpu.load(src)
    res = gpu.execute_function(fn, **kwargs)
    np.testing.assert_array_equal(res["out_ptr"], outs["out_ptr"])
    rep = gpu.get_latency_report()
    est = gpu.estimate_latency(fn, **kwargs)
    assert rep.kernel_cycles == est.kernel_cycles == 6304.0 and rep.bottleneck == "memory"
    gpu.close()


def _sharded_on_one_gpu(src, fn, kw, world, out_name):
    """Runs every rank's shard one after another on this GPU and merges the slabs on the host."""
    from ktir_cpu_b200.interpreter import Session
    gpu = KTIRInterpreter()
    gpu.load(src)
    func = gpu.module.get_function(fn)
    tensors = [(k, tuple(v.shape), v.dtype) for k, v in kw.items() if isinstance(v, np.ndarray)]
    scalars = {k: v for k, v in kw.items() if not isinstance(v, np.ndarray)}
    merged = kw[out_name].copy().reshape(-1).view(np.uint8)
    covered = 0
    for rank in range(world):
        sess = Session(gpu.device, func, tensors, scalars, shard=(rank, world))
        for k, v in kw.items():
            if isinstance(v, np.ndarray):
                sess.upload(k, v)
        sess.run()
        part = sess.download(out_name)
        gpu.device.sync()
        off = sess.layout[out_name][0]
        for lo, hi in sess.written_ranges():
            merged[lo - off:hi - off] = part.reshape(-1).view(np.uint8)[lo - off:hi - off]
            covered += hi - lo
        sess.close()
    gpu.close()
    return merged.view(kw[out_name].dtype).reshape(kw[out_name].shape), covered


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_ranks_reproduce_the_full_result(world, build_lib):
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((96, 512)) * 2).astype(np.float16)
    src = K.softmax_rows(96, 512, 6, 4, True)
    kw = dict(output_ptr=np.zeros_like(x), input_ptr=x)
    full, _ = _run_both(src, "softmax_kernel", kw)
    got, covered = _sharded_on_one_gpu(src, "softmax_kernel", kw, world, "output_ptr")
    np.testing.assert_array_equal(got, full["output_ptr"])
    assert covered == x.nbytes
    # ordered read-modify-write scatter: split by destination rows, still bit-exact
    table = rng.standard_normal((257, 128)).astype(np.float16)
    idx = _dup_indices(rng, 257, 4096, 64, 6).astype(np.int32)
    kw = dict(table_ptr=table, idx_ptr=idx, out_ptr=rng.standard_normal((257, 128)).astype(np.float16))
    src = K.gather_scale_scatter(257, 128, 4096, 64, 8)
    full, want = _run_both(src, "gather_scale_scatter", kw)
    got, _ = _sharded_on_one_gpu(src, "gather_scale_scatter", kw, world, "out_ptr")
    np.testing.assert_array_equal(got, want["out_ptr"])
    # tensor-core GEMM: ranks own disjoint tiles of C
    a = rng.uniform(-1, 1, (256, 256)).astype(np.float16)
    b = rng.uniform(-1, 1, (256, 256)).astype(np.float16)
    kw = dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((256, 256), np.float16))
    src = K.tiled_matmul(256, 256, 256, 64, 64, 64, 4, True)
    full, _ = _run_both(src, "matmul_kernel", kw)
    got, covered = _sharded_on_one_gpu(src, "matmul_kernel", kw, world, "c_ptr")
    np.testing.assert_array_equal(got, full["c_ptr"])
    assert covered == a.nbytes
    if world == 2:
        # attention: a core slice that is a whole number of heads becomes a head range
        S, H, D, tm, tn = 256, 4, 128, 64, 64
        q, k, v = (rng.standard_normal((S, H, D)).astype(np.float16) for _ in range(3))
        kw = dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k.reshape(S // tn, tn, H, D),
                  value_cache_ptr=v.reshape(S // tn, tn, H, D),
                  block_tables_ptr=np.arange(S // tn, dtype=np.int32).reshape(1, -1),
                  num_tiles=S // tn, context_len=0, scale=float(1.0 / np.sqrt(D)))
        src = K.causal_attention(S, H, D, tm, tn)
        full, _ = _run_both(src, "attention_kernel", kw)
        got, covered = _sharded_on_one_gpu(src, "attention_kernel", kw, world, "output_ptr")
        np.testing.assert_array_equal(got, full["output_ptr"])
        assert covered == q.nbytes


def test_fallback_steps_match_the_oracle(build_lib):
    """Kernels no fused kernel covers run step by step on the device (statement kind 'generic')."""
    rng = np.random.default_rng(31)
    cases = [
        # (200 columns: rows that are a power of two long go to the fused row kernel)
        (K.layernorm_rows(64, 200, 4), "layernorm_kernel",
         dict(x_ptr=rng.standard_normal((64, 200)).astype(np.float16), w_ptr=rng.standard_normal((1, 200)).astype(np.float16),
              b_ptr=rng.standard_normal((1, 200)).astype(np.float16), y_ptr=np.zeros((64, 200), np.float16),
              mean_ptr=np.zeros(64, np.float32)), 2e-3),
        (K.naive_attention(64, 32, 2), "naive_attention",
         dict(q_ptr=rng.standard_normal((64, 32)).astype(np.float16), k_ptr=rng.standard_normal((64, 32)).astype(np.float16),
              v_ptr=rng.standard_normal((64, 32)).astype(np.float16), o_ptr=np.zeros((64, 32), np.float16)), 2e-3),
        (K.gather_elements(32, 16, 64), "gather_elements",
         dict(src_ptr=rng.standard_normal((64, 16)).astype(np.float16), idx_ptr=rng.integers(0, 64, (32, 16)).astype(np.int32),
              out_ptr=np.zeros((32, 16), np.float16)), 0.0),
    ]
    for src, fn, kw, tol in cases:
        gpu = KTIRInterpreter()
        gpu.load(src)
        sess, _ = gpu.session(fn, **kw)
        assert any(s.kind == "generic" for s in sess.plan.statements)
        gpu.close()
        got, want = _run_both(src, fn, kw)
        for k in want:
            if tol == 0.0:
                np.testing.assert_array_equal(got[k], want[k])
            else:
                np.testing.assert_allclose(got[k].astype(np.float32), want[k].astype(np.float32), rtol=tol, atol=tol)
    # a negative index on the step-by-step path raises like the fused kernels do
    src, fn, kw, _ = cases[2]
    kw = dict(kw)
    kw["idx_ptr"] = kw["idx_ptr"].copy()
    kw["idx_ptr"][1, 1] = -5
    gpu = KTIRInterpreter()
    gpu.load(src)
    with pytest.raises(IndexError, match="negative"):
        gpu.execute_function(fn, **kw)
    gpu.close()


FIXED_ADDRESS_KERNEL = """
module {
  func.func @scale_rows() attributes {grid = [2, 1]} {
    %pid = ktdp.get_compute_tile_id : index
    %c0 = arith.constant 0 : index
    %c8 = arith.constant 8 : index
    %row = arith.muli %pid, %c8 : index
    %src_ptr = arith.constant 0 : index
    %dst_ptr = arith.constant 1024 : index
    %two = arith.constant 2.0 : f16
    %src = ktdp.construct_memory_view %src_ptr, sizes: [16, 64], strides: [64, 1] {
      coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 15 >= 0, d1 >= 0, -d1 + 63 >= 0)>,
      memory_space = #ktdp.memory_space<global>
    } : memref<16x64xf16>
    %dst = ktdp.construct_memory_view %dst_ptr, sizes: [16, 64], strides: [64, 1] {
      coordinate_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 15 >= 0, d1 >= 0, -d1 + 63 >= 0)>,
      memory_space = #ktdp.memory_space<global>
    } : memref<16x64xf16>
    %s_tile = ktdp.construct_access_tile %src[%row, %c0] {
      access_tile_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 7 >= 0, d1 >= 0, -d1 + 63 >= 0)>,
      access_tile_order = affine_map<(d0, d1) -> (d0, d1)>
    } : memref<16x64xf16> -> !ktdp.access_tile<8x64xindex>
    %d_tile = ktdp.construct_access_tile %dst[%row, %c0] {
      access_tile_set = affine_set<(d0, d1) : (d0 >= 0, -d0 + 7 >= 0, d1 >= 0, -d1 + 63 >= 0)>,
      access_tile_order = affine_map<(d0, d1) -> (d0, d1)>
    } : memref<16x64xf16> -> !ktdp.access_tile<8x64xindex>
    %x = ktdp.load %s_tile : !ktdp.access_tile<8x64xindex> -> tensor<8x64xf16>
    %t = tensor.splat %two : tensor<8x64xf16>
    %y = arith.mulf %x, %t : tensor<8x64xf16>
    ktdp.store %y, %d_tile : tensor<8x64xf16>, !ktdp.access_tile<8x64xindex>
    return
  }
}
"""


def test_memory_seeded_at_fixed_addresses(build_lib):
    """Kernels with hard-coded pointers: data placed through interp.memory.hbm.write before the run
    (the way the reference's tests wrap _prepare_execution) and read back with hbm.read afterwards."""
    rng = np.random.default_rng(41)
    x = rng.standard_normal((16, 64)).astype(np.float16)
    gpu = KTIRInterpreter()
    gpu.load(FIXED_ADDRESS_KERNEL)
    orig = gpu._prepare_execution

    def prepare_and_seed(grid_shape):
        orig(grid_shape)
        gpu.memory.hbm.write(0, x.reshape(-1))                    # element 0 of f16 = stick 0
        gpu.memory.hbm.write(16, np.zeros(16 * 64, np.float16))   # element 1024 of f16 = byte 2048 = stick 16
    gpu._prepare_execution = prepare_and_seed
    gpu.execute_function("scale_rows")
    got = gpu.memory.hbm.read(16, 16 * 64, "f16").reshape(16, 64)
    np.testing.assert_array_equal(got, (x * np.float16(2)).astype(np.float16))
    np.testing.assert_array_equal(gpu.memory.hbm.read(0, 16 * 64, "f16").reshape(16, 64), x)
    assert len(gpu.grid_executor.cores) == 2
    with pytest.raises(ValueError, match="unmapped"):
        gpu.memory.hbm.read(4096, 4, "f16")
    gpu.close()


@pytest.mark.parametrize("shape,sel,kind", [((64, 96, 128), (5,), "rows_program"), ((32, 4, 64, 64), (3,), "rows_program"),
                                            ((16, 40, 8), (9,), "rows_program"), ((40, 24, 64), (3, 5), "rows_program"),
                                            ((12, 10, 6, 32), (4, 3), "rows_program"), ((6, 5, 2048), (3, 2), "rows_program"),
                                            ((6, 5, 7), (4, 3), "rows_program"), ((8, 6, 4, 16), (3, 2, 2), "generic")])
def test_block_gathers_match_numpy(shape, sel, kind, build_lib):
    """The block gathers of the reference's indirect-load benchmark at small sizes: leading dims looked up
    through index vectors, the rest taken whole.  One or two indices: the fused row kernel (trailing dims
    folded into columns, long rows cut into segments, the first of two lookups fixed per tile); three: the
    step-by-step path."""
    rng = np.random.default_rng(21)
    rshape = tuple(sel) + tuple(shape[len(sel):])
    kw = {"src_ptr": rng.standard_normal(shape).astype(np.float16)}
    for i, n in enumerate(sel):
        kw[f"idx{i}_ptr"] = rng.choice(shape[i], n, replace=False).astype(np.int32)
    kw["out_ptr"] = np.zeros(rshape, np.float16)
    gpu = KTIRInterpreter()
    gpu.load(K_.blocked_gather(shape, sel))
    got = gpu.execute_function("blocked_gather", **kw)
    kinds = [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]
    gpu.close()
    assert kinds == [kind]
    want = kw["src_ptr"][np.ix_(*[kw[f"idx{i}_ptr"] for i in range(len(sel))])]
    np.testing.assert_array_equal(got["out_ptr"], want)
    np.testing.assert_array_equal(got["src_ptr"], kw["src_ptr"])


def test_cores_run_in_order_where_they_touch_each_others_memory(build_lib):
    """Running sums down the rows (core c adds row c into row c + 1) and blocks shifted with wrap-around:
    both results exist only in the reference's core-after-core order (ktir_cpu/grid.py:595-613).  Called
    three times, so that the recorded CUDA graph of the group-after-group plan is replayed as well."""
    from test_sharded import SHIFT
    rng = np.random.default_rng(77)
    gpu = KTIRInterpreter()
    gpu.load(K_.core_chain(32, 256))
    for _ in range(3):
        x = rng.standard_normal((33, 256)).astype(np.float16)
        want = x.copy()
        for c in range(32):
            want[c + 1] = want[c + 1] + want[c]
        got = gpu.execute_function("core_chain", x_ptr=x)
        np.testing.assert_array_equal(got["x_ptr"], want)
    (sess,) = gpu._sessions.values()
    assert sess.plan.core_groups == [(c, c + 1) for c in range(32)]
    gpu.close()
    gpu = KTIRInterpreter()
    gpu.load(SHIFT)
    x = rng.standard_normal(256).astype(np.float16)
    want = x.copy()
    for c in range(4):
        want[c * 64:(c + 1) * 64] = want[((c + 1) % 4) * 64:((c + 1) % 4 + 1) * 64]
    np.testing.assert_array_equal(gpu.execute_function("shift", x_ptr=x)["x_ptr"], want)
    gpu.close()
    # a running row re-loaded and stored back in every loop iteration: one statement per iteration
    gpu = KTIRInterpreter()
    gpu.load(K_.accumulate_rows(8, 40, 128))
    for _ in range(3):
        x, acc = rng.standard_normal((320, 128)).astype(np.float16), rng.standard_normal((8, 128)).astype(np.float16)
        want = acc.copy()
        for i in range(40):
            want = want + x[i::40]
        np.testing.assert_array_equal(gpu.execute_function("accumulate_rows", x_ptr=x, acc_ptr=acc)["acc_ptr"], want)
    (sess,) = gpu._sessions.values()
    assert sess.plan.unrolled_groups == [(0, 8)] and len(sess.plan.statements) == 40
    gpu.close()


def _tile_binop(op, rows, cols, tr, tc, cores):
    """out[tile] = x[tile] (op) y[tile] over [tr, tc] tiles of a [rows, cols] tensor: tiles narrower than the
    tensor, so an item has several rows with a stride; tile (i, j) belongs to core (i * ncol + j) % cores."""
    nrow, ncol = rows // tr, cols // tc
    per_core = nrow * ncol // cores
    assert nrow * tr == rows and ncol * tc == cols and per_core * cores == nrow * ncol
    t, at = f"tensor<{tr}x{tc}xf16>", f"!ktdp.access_tile<{tr}x{tc}xindex>"
    s = (f"module {{\n  func.func @tile_binop(%x_ptr: index, %y_ptr: index, %out_ptr: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %c = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n    %c1 = arith.constant 1 : index\n"
         f"    %per = arith.constant {per_core} : index\n    %ncol = arith.constant {ncol} : index\n"
         f"    %tr = arith.constant {tr} : index\n    %tc = arith.constant {tc} : index\n"
         f"    %b = arith.muli %c, %per : index\n    %e = arith.addi %b, %per : index\n")
    for nm in ("x", "y", "out"):
        s += K_.view(nm, f"{nm}_ptr", [rows, cols], "f16")
    s += ("    scf.for %k = %b to %e step %c1 {\n      %i = arith.divui %k, %ncol : index\n      %j = arith.remui %k, %ncol : index\n"
          "      %r = arith.muli %i, %tr : index\n      %q = arith.muli %j, %tc : index\n")
    for nm in ("x", "y", "out"):
        s += K_.tile(f"{nm}t", nm, ["%r", "%q"], [tr, tc], [rows, cols], "f16", "      ")
    s += (f"      %a = ktdp.load %xt : {at} -> {t}\n      %bb = ktdp.load %yt : {at} -> {t}\n"
          f"      %v = {op} %a, %bb : {t}\n      ktdp.store %v, %outt : {t}, {at}\n      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


@pytest.mark.parametrize("op,fn", [("arith.addf", np.add), ("arith.mulf", np.multiply), ("arith.subf", np.subtract),
                                   ("arith.maximumf", np.maximum)])
@pytest.mark.parametrize("rows,cols,tr,tc,cores", [(96, 320, 8, 64, 4), (60, 1000, 4, 200, 5), (33, 24, 3, 8, 11),
                                                   (40, 36, 5, 12, 3)])
def test_elementwise_on_strided_tiles_bit_exact(op, fn, rows, cols, tr, tc, cores, build_lib):
    """One f16 op on tiles narrower than the tensor (several strided rows per item), chunk counts that are no
    multiple of what a block takes, widths of 8-element vectors and widths that fall back to scalars."""
    rng = np.random.default_rng(rows * cols)
    x = rng.standard_normal((rows, cols)).astype(np.float16)
    y = rng.standard_normal((rows, cols)).astype(np.float16)
    gpu = KTIRInterpreter()
    gpu.load(_tile_binop(op, rows, cols, tr, tc, cores))
    got = gpu.execute_function("tile_binop", x_ptr=x, y_ptr=y, out_ptr=np.full_like(x, 7))["out_ptr"]
    kinds = [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]
    gpu.close()
    assert kinds == ["ew_stream"]
    np.testing.assert_array_equal(got.view(np.uint16), fn(x, y).astype(np.float16).view(np.uint16))


def _aliased_gather_source():
    """out[i, j] = src[idx[i, j], j] at fixed addresses, the destination laid over the second half of the
    index tensor's bytes (src: bytes 0..1024, idx: 1024..1536, out: 1280..1536)."""
    return K_.gather_elements(8, 16, 32).replace("(%src_ptr: index, %idx_ptr: index, %out_ptr: index)", "()").replace(
        "    %c0 = arith.constant 0 : index\n",
        "    %c0 = arith.constant 0 : index\n    %src_ptr = arith.constant 0 : index\n"
        "    %idx_ptr = arith.constant 256 : index\n    %out_ptr = arith.constant 640 : index\n")


def test_a_tile_whose_index_tensor_shares_bytes_with_its_destination(build_lib):
    """One core, one load, one store: the load reads every index before the store overwrites half of them
    (ktir_cpu/ops/memory_ops.py:867-964), so the kernel runs in the step-by-step form, which reads
    before it writes, and the indices that are not overwritten survive."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal((32, 16)).astype(np.float16)
    idx = rng.integers(0, 32, (8, 16)).astype(np.int32)
    gpu = KTIRInterpreter()
    gpu.load(_aliased_gather_source())
    orig = gpu._prepare_execution

    def prepare_and_seed(grid_shape):
        orig(grid_shape)
        gpu.memory.hbm.write(0, x.reshape(-1))
        gpu.memory.hbm.write(8, idx.reshape(-1))                 # stick 8 = byte 1024
    gpu._prepare_execution = prepare_and_seed
    gpu.execute_function("gather_elements")
    kinds = [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]
    got = gpu.memory.hbm.read(10, 128, "f16").reshape(8, 16)     # stick 10 = byte 1280
    kept = gpu.memory.hbm.read(8, 64, "i32")
    gpu.close()
    assert kinds == ["generic"]
    np.testing.assert_array_equal(got, x[idx, np.arange(16)[None, :]])
    np.testing.assert_array_equal(kept, idx.reshape(-1)[:64])


def _kinds(gpu):
    return [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]


@pytest.fixture(params=[True, False], ids=["one_launch", "per_row_statements"])
def fuse_row_results(request, monkeypatch):
    """Per-row results (row means, 1/std) stored by the launch whose reductions they come from, or each by a
    statement of its own."""
    from ktir_cpu_b200 import lower as L
    monkeypatch.setattr(L, "FUSE_ROW_RESULTS", request.param)
    return request.param


@pytest.mark.parametrize("rows,cols,cores", [(64, 256, 4), (96, 1024, 8), (24, 4096, 4), (6, 16384, 2), (40, 8, 5), (33, 64, 3)])
def test_layernorm_runs_as_fused_row_programs(rows, cols, cores, fuse_row_results, build_lib):
    """Layer norm (two reductions, two per-row values broadcast back, per-column weight and bias) and its row
    means (a tile with one value per row): both statements on the fused row kernel, compared with the oracle.
    Sums are folded in the reference's halving order and every op rounds where the reference rounds, so the
    results are the reference's bits."""
    rng = np.random.default_rng(cols + rows)
    kw = dict(x_ptr=(rng.standard_normal((rows, cols)) * 3 + 1).astype(np.float16), w_ptr=rng.standard_normal(cols).astype(np.float16),
              b_ptr=rng.standard_normal(cols).astype(np.float16), y_ptr=np.zeros((rows, cols), np.float16),
              mean_ptr=np.zeros(rows, np.float32))
    src = K_.layernorm_rows(rows, cols, cores)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("layernorm_kernel", **kw)
    kinds = _kinds(gpu)
    gpu.close()
    assert kinds == ["row_program"] * (1 if fuse_row_results else 2)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("layernorm_kernel", **kw)
    np.testing.assert_array_equal(got["mean_ptr"].view(np.uint32), want["mean_ptr"].view(np.uint32))
    np.testing.assert_array_equal(got["y_ptr"].view(np.uint16), want["y_ptr"].view(np.uint16))


@pytest.mark.parametrize("weight", [False, True])
@pytest.mark.parametrize("rows,cols,cores,tile_rows", [(64, 256, 4, 4), (128, 2048, 4, 8), (12, 512, 3, 2), (64, 32, 2, 16)])
def test_rmsnorm_tiles_of_several_rows(rows, cols, cores, tile_rows, weight, fuse_row_results, build_lib):
    """RMS norm on tiles of several rows, with and without a weight row that all rows of a tile share."""
    rng = np.random.default_rng(rows * 7 + cols)
    kw = dict(x_ptr=(rng.standard_normal((rows, cols)) * 2).astype(np.float16))
    if weight:
        kw["w_ptr"] = rng.standard_normal(cols).astype(np.float16)
    kw.update(y_ptr=np.zeros((rows, cols), np.float16), rstd_ptr=np.zeros(rows, np.float32))
    src = K_.rmsnorm_rows(rows, cols, cores, tile_rows, weight=weight)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("rmsnorm_kernel", **kw)
    kinds = _kinds(gpu)
    gpu.close()
    assert kinds == ["row_program"] * (1 if fuse_row_results else 2)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("rmsnorm_kernel", **kw)
    np.testing.assert_array_equal(got["rstd_ptr"].view(np.uint32), want["rstd_ptr"].view(np.uint32))
    np.testing.assert_array_equal(got["y_ptr"].view(np.uint16), want["y_ptr"].view(np.uint16))
    np.testing.assert_array_equal(got["x_ptr"], kw["x_ptr"])


@pytest.mark.parametrize("rows,cols,cores,tile_rows", [(64, 256, 4, 2), (32, 4096, 4, 1), (48, 64, 3, 8)])
def test_log_softmax_on_the_interpreting_row_kernel(rows, cols, cores, tile_rows, build_lib):
    """Phases that are no normalisation skeleton (max with maxnumf, exp, log): the interpreting row kernel.
    exp and log are the device's, so the comparison with the oracle carries the f16 tolerance."""
    rng = np.random.default_rng(rows + cols)
    kw = dict(x_ptr=(rng.standard_normal((rows, cols)) * 3).astype(np.float16), y_ptr=np.zeros((rows, cols), np.float16))
    src = K_.log_softmax_rows(rows, cols, cores, tile_rows)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("log_softmax_kernel", **kw)
    kinds = _kinds(gpu)
    gpu.close()
    assert kinds == ["row_program"]
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("log_softmax_kernel", **kw)
    np.testing.assert_allclose(got["y_ptr"].astype(np.float32), want["y_ptr"].astype(np.float32), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(np.exp(got["y_ptr"].astype(np.float64)).sum(1), 1.0, atol=2e-2)


def test_row_widths_the_row_kernel_does_not_take_run_step_by_step(build_lib):
    """37 columns: no power of two, so the statement keeps the step-by-step form (and the reference's result)."""
    rng = np.random.default_rng(3)
    kw = dict(x_ptr=rng.standard_normal((16, 37)).astype(np.float16), w_ptr=rng.standard_normal(37).astype(np.float16),
              b_ptr=rng.standard_normal(37).astype(np.float16), y_ptr=np.zeros((16, 37), np.float16), mean_ptr=np.zeros(16, np.float32))
    src = K_.layernorm_rows(16, 37, 4)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("layernorm_kernel", **kw)
    kinds = _kinds(gpu)
    gpu.close()
    assert kinds == ["generic", "generic"]
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("layernorm_kernel", **kw)
    np.testing.assert_allclose(got["y_ptr"].astype(np.float32), want["y_ptr"].astype(np.float32), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("rows,cols,block,cores", [(8, 512, 256, 2), (37, 8192, 1024, 32), (12, 1024, 64, 5), (64, 256, 8, 4)])
def test_column_blocked_layernorm_on_the_row_kernel(rows, cols, block, cores, fuse_row_results, build_lib):
    """The reference's layer-norm example shape (f16, column blocks accumulated through loops, mean / rstd
    per row, output block by block; rows that do not divide by the cores): three row programs, the
    reference's bits."""
    rng = np.random.default_rng(rows + cols + block)
    kw = dict(X=rng.standard_normal((rows, cols)).astype(np.float16), Y=np.zeros((rows, cols), np.float16),
              W=rng.standard_normal((rows, cols)).astype(np.float16), B=rng.standard_normal((rows, cols)).astype(np.float16),
              Mean=np.zeros(rows, np.float16), Rstd=np.zeros(rows, np.float16), N=cols, eps=np.float16(1e-5), BLOCK_SIZE=block)
    src = K_.layernorm_blocked(rows, cols, block, cores)
    gpu = KTIRInterpreter()
    gpu.load(src)
    got = gpu.execute_function("_layer_norm_fwd_fused", **kw)
    kinds = _kinds(gpu)
    gpu.close()
    assert kinds == ["row_program"] * (1 if fuse_row_results else 3)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("_layer_norm_fwd_fused", **kw)
    for k in ("Mean", "Rstd", "Y"):
        np.testing.assert_array_equal(got[k].view(np.uint16), want[k].view(np.uint16), err_msg=k)

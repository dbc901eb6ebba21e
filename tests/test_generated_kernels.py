"""Kernels from the generators at drawn sizes: the step-by-step lowering (run by the NumPy stand-in for the
device steps) against the oracle, bit for bit — host logic, no GPU.  Sizes are small so that the whole
file takes seconds; the seeds are fixed."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from oracle.numpy_interp import OracleInterpreter
from test_generic_lowering import run_generic


def _check(src, fn, kw):
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function(fn, **kw)
    got, kinds = run_generic(src, fn, kw)
    for k, w in want.items():
        np.testing.assert_array_equal(got[k].view(np.uint8), np.ascontiguousarray(w).view(np.uint8), err_msg=k)
    return kinds


@pytest.mark.parametrize("seed", range(6))
def test_distributed_view_tiles(seed):
    rng = np.random.default_rng(100 + seed)
    cores = int(rng.choice([1, 2, 4]))
    th = int(rng.choice([2, 4, 8]))
    rows = cores * th * int(rng.integers(1, 4)) * 2
    cols = int(rng.choice([16, 32, 64]))
    shift = int(rng.integers(0, th))
    a = rng.standard_normal((rows, cols)).astype(np.float16)
    h, w = rows // 2, cols // 2
    kw = dict(a0_ptr=np.ascontiguousarray(a[:h]), a1_ptr=np.ascontiguousarray(a[h:, :w].T), a2_ptr=np.ascontiguousarray(a[h:, w:]),
              o0_ptr=np.full((rows, w), 3, np.float16), o1_ptr=np.full((rows, w), 3, np.float16))
    _check(K.sharded_scale(rows, cols, th, cores, shift), "sharded_scale", kw)


@pytest.mark.parametrize("seed", range(5))
def test_region_reductions(seed):
    rng = np.random.default_rng(200 + seed)
    cores = int(rng.choice([1, 2, 4]))
    rows = cores * int(rng.integers(1, 4))
    cols = int(rng.integers(2, 70))
    x = rng.standard_normal((rows, cols)).astype(np.float16)
    kinds = _check(K.region_reduce_rows(rows, cols, cores), "region_reduce",
                   dict(x_ptr=x, mx_ptr=np.zeros(rows, np.float16), sa_ptr=np.zeros(rows, np.float16)))
    n, odd = cols, False
    while n > 1:
        odd |= bool(n % 2)
        n = n // 2 + n % 2
    assert ("concat" in kinds) == odd


@pytest.mark.parametrize("seed", range(4))
def test_paged_gathers(seed):
    rng = np.random.default_rng(300 + seed)
    page = int(rng.choice([4, 8, 16]))
    chunk = page * int(rng.choice([1, 2]))
    seq_len = chunk * int(rng.integers(1, 4))
    n_seq, heads, dim = int(rng.integers(1, 4)), int(rng.choice([1, 2])), int(rng.choice([8, 16]))
    n_pages = n_seq * (seq_len // page) + 3
    pages = rng.standard_normal((n_pages, heads, page, dim)).astype(np.float16)
    table = rng.permutation(n_pages)[:n_seq * (seq_len // page)].reshape(n_seq, -1).astype(np.int32)
    kw = dict(pages_ptr=pages, table_ptr=table, out_ptr=np.zeros((n_seq, seq_len, heads, dim), np.float16))
    _check(K.paged_gather(n_seq, seq_len, page, heads, dim, n_pages, chunk), "paged_gather", kw)


@pytest.mark.parametrize("seed", range(4))
def test_generic_contractions(seed):
    rng = np.random.default_rng(400 + seed)
    cores = int(rng.choice([1, 2]))
    M, N, Kd = cores * int(rng.integers(1, 4)), int(rng.integers(1, 9)), int(rng.integers(2, 20))
    dt, npdt = ("f32", np.float32) if seed % 2 else ("f16", np.float16)
    kw = dict(a_ptr=rng.standard_normal((M, Kd)).astype(npdt), b_ptr=rng.standard_normal((Kd, N)).astype(npdt),
              c_ptr=rng.standard_normal((M, N)).astype(npdt))
    _check(K.generic_contraction(M, N, Kd, cores, dt), "generic_contraction", kw)


@pytest.mark.parametrize("shape,sel", [((6, 4, 8), (3,)), ((5, 3, 2, 8), (2,)), ((7, 6, 8), (3, 2)), ((4, 5, 2, 8), (2, 3))])
def test_block_gathers(shape, sel):
    rng = np.random.default_rng(500)
    rshape = tuple(sel) + tuple(shape[len(sel):])
    kw = {"src_ptr": rng.standard_normal(shape).astype(np.float16)}
    for i, n in enumerate(sel):
        kw[f"idx{i}_ptr"] = rng.choice(shape[i], n, replace=False).astype(np.int32)
    kw["out_ptr"] = np.zeros(rshape, np.float16)
    _check(K.blocked_gather(shape, sel), "blocked_gather", kw)
    want = kw["src_ptr"][np.ix_(*[kw[f"idx{i}_ptr"] for i in range(len(sel))])]
    ora = OracleInterpreter()
    ora.load(K.blocked_gather(shape, sel))
    np.testing.assert_array_equal(ora.execute_function("blocked_gather", **kw)["out_ptr"], want)


@pytest.mark.parametrize("seed", range(3))
def test_transposed_gathers(seed):
    rng = np.random.default_rng(600 + seed)
    cores, tile_rows = int(rng.choice([1, 2])), int(rng.choice([2, 4, 8]))
    n_idx = cores * tile_rows * int(rng.integers(1, 4))
    cols, n_rows = int(rng.choice([4, 8, 16])), int(rng.integers(4, 40))
    kw = dict(table_ptr=rng.standard_normal((n_rows, cols)).astype(np.float16), idx_ptr=rng.integers(0, n_rows, n_idx).astype(np.int32),
              out_ptr=np.zeros((cols, n_idx), np.float16))
    _check(K.gather_rows_transposed(n_rows, cols, n_idx, tile_rows, cores), "gather_rows_transposed", kw)

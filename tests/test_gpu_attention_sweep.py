"""All 27 distinct kernels of the candidate sweep (tile_m, tile_n in {32, 64, 128} x S in
{512, 1024, 2048}) at their real sequence lengths: every head against f64 math, one head against
the oracle.  The text has the shape the reference's own generator writes (grouped tiles, causal
mask through ``arith.divui``), and the plan must be the tensor-core attention kernel."""
import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200.interpreter import KTIRInterpreter
from oracle.numpy_interp import OracleInterpreter

pytestmark = pytest.mark.gpu

D = 128


def attention_f64(q, kc, vc, table, ctx=0, group=1):
    """q [S, H, D]; caches [pages, tn, Hkv, D]; page j of the walk is cache page table[j]."""
    S, H, _ = q.shape
    k = kc[table].reshape(-1, kc.shape[2], D).astype(np.float64)
    v = vc[table].reshape(-1, vc.shape[2], D).astype(np.float64)
    out = np.empty((S, H, D))
    keep = np.arange(k.shape[0])[None, :] <= (np.arange(S) + ctx)[:, None]
    for h in range(H):
        sc = q[:, h].astype(np.float64) @ k[:, h // group].T / np.sqrt(D)
        sc = np.where(keep, sc, -np.inf)
        p = np.exp(sc - sc.max(-1, keepdims=True))
        out[:, h] = (p / p.sum(-1, keepdims=True)) @ v[:, h // group]
    return out


def _inputs(seed, S, H, Hkv, tn, ctx):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((S, H, D), dtype=np.float32).astype(np.float16)
    nt = (S + ctx) // tn
    kc, vc = (rng.standard_normal((nt, tn, Hkv, D), dtype=np.float32).astype(np.float16) for _ in range(2))
    table = rng.permutation(nt).astype(np.int32)
    return q, kc, vc, table, dict(
        output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=kc, value_cache_ptr=vc,
        block_tables_ptr=table.reshape(1, -1), cur_batch_start_index=0, block_table_offset=0, num_tiles=nt,
        context_len=ctx, scale=np.float32(1.0 / np.sqrt(D)))


def _gpu(src, kw):
    gpu = KTIRInterpreter()
    gpu.load(src)
    o = gpu.execute_function("paged_attention_kernel", **kw)["output_ptr"]
    kinds = [s.kind for sess in gpu._sessions.values() for s in sess.plan.statements]
    gpu.close()
    return o, kinds


@pytest.mark.parametrize("S", [512, 1024, 2048])
@pytest.mark.parametrize("tn", [32, 64, 128])
@pytest.mark.parametrize("tm", [32, 64, 128])
def test_sweep_kernel(tm, tn, S, build_lib):
    H = 4
    q, kc, vc, table, kw = _inputs(1000 + S + 3 * tm + tn, S, H, H, tn, 0)
    o, kinds = _gpu(K.paged_attention(S, S, H, H, D, tn, tm), kw)
    assert kinds == ["attention_fwd"]
    np.testing.assert_allclose(o.astype(np.float64), attention_f64(q, kc, vc, table), rtol=1e-2, atol=2e-3)
    ora = OracleInterpreter()
    ora.load(K.paged_attention(S, S, 1, 1, D, tn, tm))
    h = (tm + tn) // 32 % H
    want = ora.execute_function("paged_attention_kernel", **dict(
        kw, output_ptr=np.zeros((S, 1, D), np.float16), query_ptr=np.ascontiguousarray(q[:, h:h + 1]),
        key_cache_ptr=np.ascontiguousarray(kc[:, :, h:h + 1]), value_cache_ptr=np.ascontiguousarray(vc[:, :, h:h + 1])))
    np.testing.assert_allclose(o[:, h].astype(np.float32), want["output_ptr"][:, 0].astype(np.float32),
                               rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("S,H,Hkv,bq,tn,ctx", [(256, 8, 2, 16, 64, 0), (256, 4, 1, 32, 32, 128), (384, 6, 3, 64, 128, 256),
                                               (192, 2, 2, 32, 64, 64)])
def test_grouped_heads_and_context(S, H, Hkv, bq, tn, ctx, build_lib):
    """Several query heads per K/V head (tile rows interleave the heads of a group) and KV positions
    that precede the first query (``context_len`` > 0), whole result against the oracle and f64."""
    q, kc, vc, table, kw = _inputs(S + H + ctx, S, H, Hkv, tn, ctx)
    src = K.paged_attention(S, S + ctx, H, Hkv, D, tn, bq)
    o, kinds = _gpu(src, kw)
    assert kinds == ["attention_fwd"]
    np.testing.assert_allclose(o.astype(np.float64), attention_f64(q, kc, vc, table, ctx, H // Hkv), rtol=1e-2, atol=2e-3)
    ora = OracleInterpreter()
    ora.load(src)
    want = ora.execute_function("paged_attention_kernel", **kw)["output_ptr"]
    np.testing.assert_allclose(o.astype(np.float32), want.astype(np.float32), rtol=1e-2, atol=2e-3)

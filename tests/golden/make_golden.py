"""Regenerates ``tests/golden/*.npz`` by running the UNMODIFIED reference interpreter.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py /path/to/reference [--latency-only] [--only=<case> ...]

Each fixture stores the KTIR source, the seeded inputs and the outputs the
reference produced, plus the NumPy version and CPU features of the generating
host (f16 transcendentals in NumPy are host-dependent by 1 ulp).  The tests
never import the reference; they only read these files.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from ktir_cpu_b200 import kernels as K  # noqa: E402


def _reference_generators(ref_root: str):
    """``notebooks/demo_gen_mlir.py`` of the reference checkout, imported as a module."""
    import importlib.util
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    spec = importlib.util.spec_from_file_location("demo_gen_mlir", os.path.join(ref_root, "notebooks", "demo_gen_mlir.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def paged_attention_inputs(seed, S, H, Hkv, D, tn, ctx):
    """Seeded inputs of a ``paged_attention_kernel`` call: K/V pages stored in a permuted order and
    found through the block table, ``ctx`` KV positions before the first query position."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((S, H, D)).astype(np.float16)
    nt = (S + ctx) // tn
    k, v = (rng.standard_normal((nt, tn, Hkv, D)).astype(np.float16) for _ in range(2))
    table = rng.permutation(nt).astype(np.int32).reshape(1, -1)
    return dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k, value_cache_ptr=v,
                block_tables_ptr=table, cur_batch_start_index=0, block_table_offset=0, num_tiles=nt,
                context_len=ctx, scale=np.float32(1.0 / np.sqrt(D)))


def cases(ref_root=None):
    """name -> (source, function, kwargs). Shared with the tests through the fixture files.

    With ``ref_root`` the kernels the reference's own generator writes
    (``gen_paged_attention_mlir``) are added; their text is stored in the fixture like any other."""
    out = {}
    if ref_root:
        gen = _reference_generators(ref_root)
        # (S, query heads, K/V heads, tile_m, tile_n, context before the queries)
        for S, H, Hkv, tm, tn, ctx in ((128, 2, 2, 32, 32, 0), (256, 2, 2, 64, 128, 0), (256, 1, 1, 128, 128, 0),
                                       (64, 4, 2, 32, 32, 64), (128, 2, 1, 128, 64, 0)):
            src = gen.gen_paged_attention_mlir(num_tokens=S, context_len=S + ctx, num_query_heads=H, num_kv_heads=Hkv,
                                               head_dim=128, block_size=tn, block_q=tm // (H // Hkv))
            out[f"paged_attention_ref_S{S}_H{H}kv{Hkv}_t{tm}x{tn}_ctx{ctx}"] = (
                src, "paged_attention_kernel", paged_attention_inputs(7 + S + tm + tn, S, H, Hkv, 128, tn, ctx))
    rng = np.random.default_rng(1)
    x, y = rng.standard_normal(4096).astype(np.float16), rng.standard_normal(4096).astype(np.float16)
    out["vector_add_4096"] = (K.vector_add(4096, 128, 32), "add_kernel",
                              dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(4096, np.float16), BLOCK_SIZE=128))
    x, y = rng.standard_normal(16384).astype(np.float16), rng.standard_normal(16384).astype(np.float16)
    out["vector_add_loop"] = (K.vector_add(16384, 128, 32), "add_kernel",
                              dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(16384, np.float16), BLOCK_SIZE=128))
    rng = np.random.default_rng(2)
    for f32 in (True, False):
        x = (rng.standard_normal((64, 256)) * 2).astype(np.float16)
        out[f"softmax_{'f32' if f32 else 'f16'}_64x256"] = (
            K.softmax_rows(64, 256, 4, 4, f32), "softmax_kernel",
            dict(output_ptr=np.zeros_like(x), input_ptr=x))
    x = (rng.standard_normal((32, 4096)) * 2).astype(np.float16)
    out["softmax_f32_32x4096"] = (K.softmax_rows(32, 4096, 4, 2, True), "softmax_kernel",
                                  dict(output_ptr=np.zeros_like(x), input_ptr=x))
    rng = np.random.default_rng(3)
    table = rng.standard_normal((256, 128)).astype(np.float16)
    idx = rng.integers(0, 256, 1024).astype(np.int32)
    for t in range(1024 // 64):                     # ~10 % duplicates inside each 64-entry tile
        pos = rng.choice(64, 12, replace=False)
        idx[t * 64 + pos[:6]] = idx[t * 64 + pos[6:]]
    out["gather_scale_scatter_256"] = (
        K.gather_scale_scatter(256, 128, 1024, 64, 4), "gather_scale_scatter",
        dict(table_ptr=table, idx_ptr=idx, out_ptr=np.zeros_like(table)))
    idx0 = np.zeros(256, np.int32)                  # every entry hits row 0
    out["gather_scale_scatter_allzero"] = (
        K.gather_scale_scatter(16, 128, 256, 64, 2), "gather_scale_scatter",
        dict(table_ptr=table[:16].copy(), idx_ptr=idx0, out_ptr=np.zeros((16, 128), np.float16)))
    rng = np.random.default_rng(4)
    for f32 in (True, False):
        a = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
        b = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
        out[f"matmul_{'f32acc' if f32 else 'f16acc'}_128"] = (
            K.tiled_matmul(128, 128, 128, 64, 64, 64, 2, f32), "matmul_kernel",
            dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((128, 128), np.float16)))
    rng = np.random.default_rng(5)
    S, H, D, tm, tn = 128, 2, 128, 32, 64
    q, k, v = (rng.standard_normal((S, H, D)).astype(np.float16) for _ in range(3))
    out["causal_attention_128x2"] = (
        K.causal_attention(S, H, D, tm, tn), "attention_kernel",
        dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k.reshape(S // tn, tn, H, D),
             value_cache_ptr=v.reshape(S // tn, tn, H, D),
             block_tables_ptr=np.arange(S // tn, dtype=np.int32).reshape(1, -1),
             num_tiles=S // tn, context_len=0, scale=float(1.0 / np.sqrt(D))))
    rng = np.random.default_rng(6)
    out["layernorm_16x64"] = (
        K.layernorm_rows(16, 64, 4), "layernorm_kernel",
        dict(x_ptr=rng.standard_normal((16, 64)).astype(np.float16), w_ptr=rng.standard_normal((1, 64)).astype(np.float16),
             b_ptr=rng.standard_normal((1, 64)).astype(np.float16), y_ptr=np.zeros((16, 64), np.float16),
             mean_ptr=np.zeros(16, np.float32)))
    out["naive_attention_32x16"] = (
        K.naive_attention(32, 16, 2), "naive_attention",
        dict(q_ptr=rng.standard_normal((32, 16)).astype(np.float16), k_ptr=rng.standard_normal((32, 16)).astype(np.float16),
             v_ptr=rng.standard_normal((32, 16)).astype(np.float16), o_ptr=np.zeros((32, 16), np.float16)))
    # every exactly-rounded f16 elementwise op on random bit patterns (specials included): pins the
    # rounding, NaN and signed-zero rules of the arith / math dialects
    rng = np.random.default_rng(8)
    ops = ["add", "sub", "mul", "div", "maximum", "maxnum", "minimum", "minnum", "neg", "abs", "sqrt", "erf"]
    x = rng.integers(0, 65536, 4096).astype(np.uint16)
    y = rng.integers(0, 65536, 4096).astype(np.uint16)
    x[:8] = [0x0000, 0x8000, 0x7c00, 0xfc00, 0x7e00, 0x0001, 0x7bff, 0x3c00]
    y[:8] = [0x8000, 0x0000, 0x7c00, 0x7c00, 0x3c00, 0x0001, 0x7bff, 0x7e00]
    names = [f"out_{o}_ptr" for o in ops] + ["out_select_ptr", "out_ext_add_ptr"]
    out["elementwise_f16_suite"] = (
        K.elementwise_suite(ops, 4096, 128, 4, "f16", "olt"), "elementwise_kernel",
        dict(x_ptr=x.view(np.float16), y_ptr=y.view(np.float16), **{n: np.zeros(4096, np.float16) for n in names}))
    # cross-core all-reduce: every core stores what it holds (each folds in its own ring order)
    rng = np.random.default_rng(9)
    for n, g, cols, comb, dt, inner, strided in ((4, 4, 128, "add", "f16", 1, False), (8, 2, 64, "max", "f32", 1, True),
                                                 (6, 3, 32, "mul", "f16", 2, False), (16, 16, 128, "add", "f16", 1, False),
                                                 (16, 4, 256, "add", "f16", 1, False)):
        x = rng.uniform(0.5, 1.5, (n * inner, cols)).astype(np.float16 if dt == "f16" else np.float32)
        out[f"ring_allreduce_{n}x{g}_{comb}_{dt}" + ("_loop" if inner > 1 else "") + ("_strided" if strided else "")] = (
            K.ring_allreduce(n, g, cols, comb, dt, inner, strided), "ring_allreduce", dict(in_ptr=x, out_ptr=np.zeros_like(x)))
    # several cores store to the same rows: the last core in id order wins
    x = rng.standard_normal((12, 64)).astype(np.float16)
    out["shared_slot_store_12x5"] = (K.shared_slot_store(12, 5, 64), "shared_slot",
                                     dict(x_ptr=x, out_ptr=np.zeros((5, 64), np.float16)))
    # tensors shorter than the kernel's views: what a tile reads past the end of its allocation is zero,
    # what it would write there is dropped (the arrays of 4000 elements end inside the last 128-wide block)
    short = np.random.default_rng(11)
    x, y = short.standard_normal(4000).astype(np.float16), short.standard_normal(4000).astype(np.float16)
    out["vector_add_short_4000"] = (K.vector_add(4096, 128, 32), "add_kernel",
                                    dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(4000, np.float16), BLOCK_SIZE=128))
    # one tensor in three differently laid-out pieces behind a distributed memory view; tiles that cross the
    # partition boundaries and hang over the end
    dist = np.random.default_rng(12)
    for shift in (0, 3):
        a = dist.standard_normal((64, 64)).astype(np.float16)
        out[f"sharded_scale_64x64_shift{shift}"] = (
            K.sharded_scale(64, 64, 8, 4, shift), "sharded_scale",
            dict(a0_ptr=np.ascontiguousarray(a[:32]), a1_ptr=np.ascontiguousarray(a[32:, :32].T),
                 a2_ptr=np.ascontiguousarray(a[32:, 32:]), o0_ptr=np.full((64, 32), 7, np.float16),
                 o1_ptr=np.full((64, 32), 7, np.float16)))
    x = dist.standard_normal((8, 256)).astype(np.float16)
    out["sharded_center_8x256"] = (K.sharded_center(256, 4, 8), "sharded_center", dict(x_ptr=x, y_ptr=np.zeros_like(x)))
    # position split into page and slot by floordiv / mod inside the subscripts; permuted store order
    pg = np.random.default_rng(13)
    out["paged_gather_4x64"] = (
        K.paged_gather(4, 64, 16, 2, 32, 32, 32), "paged_gather",
        dict(pages_ptr=pg.standard_normal((32, 2, 16, 32)).astype(np.float16),
             table_ptr=pg.permutation(32)[:16].reshape(4, 4).astype(np.int32),
             out_ptr=np.zeros((4, 64, 2, 32), np.float16)))
    # reductions whose combiner is a region of several ops; 37 columns: an odd slice is carried at three levels
    rr = np.random.default_rng(14)
    x = rr.standard_normal((16, 37)).astype(np.float16)
    out["region_reduce_16x37"] = (K.region_reduce_rows(16, 37, 4), "region_reduce",
                                  dict(x_ptr=x, mx_ptr=np.zeros(16, np.float16), sa_ptr=np.zeros(16, np.float16)))
    # linalg.generic with a reduction iterator: products folded pairwise over k (13: odd levels)
    gc = np.random.default_rng(15)
    out["generic_contraction_4x8x13"] = (
        K.generic_contraction(4, 8, 13, 2, "f16"), "generic_contraction",
        dict(a_ptr=gc.standard_normal((4, 13)).astype(np.float16), b_ptr=gc.standard_normal((13, 8)).astype(np.float16),
             c_ptr=gc.standard_normal((4, 8)).astype(np.float16)))
    # indirect tile enumerated column by column (permuted variables_space_order)
    gt = np.random.default_rng(16)
    out["gather_rows_transposed_64x16"] = (
        K.gather_rows_transposed(32, 16, 64, 8, 2), "gather_rows_transposed",
        dict(table_ptr=gt.standard_normal((32, 16)).astype(np.float16), idx_ptr=gt.integers(0, 32, 64).astype(np.int32),
             out_ptr=np.zeros((16, 64), np.float16)))
    # a tile loaded once, overwritten in place, and stored elsewhere afterwards: the second store holds the old values
    ui = np.random.default_rng(18)
    out["update_in_place_64x64"] = (K.update_in_place(64, 64, 8, 2, True), "update_in_place",
                                    dict(x_ptr=ui.standard_normal((64, 64)).astype(np.float16), old_ptr=np.zeros((64, 64), np.float16)))
    out["update_in_place_16x64_flat"] = (K.update_in_place(16, 64, 8, 2, False), "update_in_place",
                                         dict(x_ptr=ui.standard_normal((16, 64)).astype(np.float16), old_ptr=np.zeros((16, 64), np.float16)))
    # every core reads the row the core before it wrote: running sums in core order
    out["core_chain_16x64"] = (K.core_chain(16, 64), "core_chain", dict(x_ptr=ui.standard_normal((17, 64)).astype(np.float16)))
    # every iteration of a loop reads the row the iteration before it stored
    out["accumulate_rows_4x6"] = (K.accumulate_rows(4, 6, 64), "accumulate_rows",
                                  dict(x_ptr=ui.standard_normal((24, 64)).astype(np.float16), acc_ptr=ui.standard_normal((4, 64)).astype(np.float16)))
    # RMS norm on tiles of four rows with a weight row shared by the rows of a tile, per-row scales stored too
    out["rmsnorm_weighted_32x128"] = (K.rmsnorm_rows(32, 128, 2, 4, weight=True), "rmsnorm_kernel",
                                      dict(x_ptr=(ui.standard_normal((32, 128)) * 2).astype(np.float16), w_ptr=ui.standard_normal(128).astype(np.float16),
                                           y_ptr=np.zeros((32, 128), np.float16), rstd_ptr=np.zeros(32, np.float32)))
    # layer norm written like the reference's example: f16, rows walked in column blocks through scf.for loops
    out["layernorm_blocked_8x512"] = (
        K.layernorm_blocked(8, 512, 128, 3), "_layer_norm_fwd_fused",
        dict(X=ui.standard_normal((8, 512)).astype(np.float16), Y=np.zeros((8, 512), np.float16),
             W=ui.standard_normal((8, 512)).astype(np.float16), B=ui.standard_normal((8, 512)).astype(np.float16),
             Mean=np.zeros(8, np.float16), Rstd=np.zeros(8, np.float16), N=512, eps=np.float16(1e-5), BLOCK_SIZE=128))
    out["gather_elements_8x16"] = (
        K.gather_elements(8, 16, 32), "gather_elements",
        dict(src_ptr=rng.standard_normal((32, 16)).astype(np.float16),
             idx_ptr=rng.integers(0, 32, (8, 16)).astype(np.int32), out_ptr=np.zeros((8, 16), np.float16)))
    return out


def main(ref_root: str, only=None):
    sys.path.insert(0, ref_root)
    from ktir_cpu import KTIRInterpreter
    meta = f"numpy {np.__version__}"
    for name, (src, fn, kw) in cases(ref_root).items():
        if only and name not in only:
            continue
        interp = KTIRInterpreter()
        interp.load(src)
        res = interp.execute_function(fn, **kw)
        payload = {"__source__": np.array(src), "__function__": np.array(fn), "__host__": np.array(meta)}
        for k, v in kw.items():
            payload["in__" + k] = np.asarray(v)
        for k, v in res.items():
            payload["out__" + k] = v
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **payload)
        print("wrote", name)


def latency_main(ref_root: str):
    """``latency.json``: the reference's latency report for every case above (default hardware)."""
    import json
    sys.path.insert(0, ref_root)
    from ktir_cpu import HardwareConfig, KTIRInterpreter
    out = {}
    for name, (src, fn, kw) in cases().items():      # own kernels only: keeps latency.json small
        interp = KTIRInterpreter(latency_config=HardwareConfig())
        interp.load(src)
        interp.execute_function(fn, **kw)
        rep = interp.get_latency_report()
        out[name] = {
            "summary": rep.summary_dict(),
            "roofline": rep.roofline(),
            "flops": {str(c): dict(v.flops_by_category) for c, v in rep.counters.items()},
            "bytes": {str(c): dict(v.bytes_by_category) for c, v in rep.counters.items()},
        }
        print("latency", name, rep.kernel_cycles, rep.bottleneck)
    with open(os.path.join(HERE, "latency.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


def overflow_cases():
    """name -> (source, function, kwargs, lx_size_mb): kernels whose tiles do not fit the scratchpad."""
    x = np.zeros((32, 16384), np.float16)
    v = np.zeros(1 << 21, np.float16)
    return {
        "softmax_32_rows_of_16384_at_once": (K.softmax_rows(32, 16384, 1, 32, True), "softmax_kernel",
                                             dict(output_ptr=np.zeros_like(x), input_ptr=x), 2),
        "vector_add_block_524288_in_1MB": (K.vector_add(1 << 21, 524288, 4), "add_kernel",
                                           dict(x_ptr=v, y_ptr=v, output_ptr=np.zeros_like(v), BLOCK_SIZE=524288), 1),
    }


def lx_main(ref_root: str):
    """``lx.json``: the highest scratchpad use of any core, per case, as the reference accounts it
    (ktir_cpu/grid.py:253-361), and the messages of the cases that overflow."""
    import json
    sys.path.insert(0, ref_root)
    from ktir_cpu import HardwareConfig, KTIRInterpreter
    from ktir_cpu.grid import CoreContext
    peak = {}
    charge = CoreContext._charge_lx

    def watch(self, value):
        charge(self, value)
        peak[self.core_id] = max(peak.get(self.core_id, 0), self.lx.used)
    CoreContext._charge_lx = watch
    out = {"peak_bytes": {}, "overflow": {}}
    for name, (src, fn, kw) in cases(ref_root).items():
        peak.clear()
        interp = KTIRInterpreter()
        interp.load(src)
        interp.execute_function(fn, **kw)
        out["peak_bytes"][name] = int(max(peak.values())) if peak else 0
    for name, (src, fn, kw, mb) in overflow_cases().items():
        interp = KTIRInterpreter(latency_config=HardwareConfig(lx_size_mb=mb))
        interp.load(src)
        try:
            interp.execute_function(fn, **kw)
            raise SystemExit(f"{name}: expected an LX overflow")
        except MemoryError as e:
            out["overflow"][name] = str(e)
            print("overflow", name, e)
    CoreContext._charge_lx = charge
    with open(os.path.join(HERE, "lx.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    root = args[0] if args else os.environ.get("KTIR_REFERENCE", "")
    if not root:
        sys.exit("usage: make_golden.py <path of a ktir_cpu checkout> [--only=<case>] [--latency-only]")
    only = [a[len("--only="):] for a in sys.argv[1:] if a.startswith("--only=")]
    if "--lx-only" in sys.argv:
        lx_main(root)
        sys.exit(0)
    if "--latency-only" not in sys.argv:
        main(root, only)
    latency_main(root)
    lx_main(root)

"""Benchmark of the KTIR execution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
                    [--no-extras] [--no-cpu]

Headline workload (the one the metric is quoted on): row softmax over f16[8192, 4096] with f32
statistics, 32 KTIR cores x 256 contiguous rows.  One "step" is one pass of the hot path over the
whole workload.  Prints ONE JSON line (rank 0):

* ``value``     elements/s with the tensors resident in HBM, each step timed by CUDA events on the
                launch stream, L2 flushed between steps;
* ``roofline``  algorithmic bytes (or FLOP) / mean launch time against the measured peak; for the
                HBM-bound kernels also ``frac_sustained``: eight back-to-back launches over eight
                distinct buffer sets (together far larger than L2), one event pair, no flush, so
                the write-back of each launch's output is paid inside the window;
* ``e2e``       the same metric through ``KTIRInterpreter.execute_function`` with host arrays in
                and fresh host arrays out every step (page-locked caller arrays; ``pageable`` is the
                same with ordinary NumPy arrays);
* ``cpu_baseline``  the reference interpreter itself (``baseline/_ref``, else the oracle port) on
                the host cores, on a bounded sample of the same workload;
* ``extras``    the same report for the other configurations (vector add, gather + ordered scatter,
                tiled matmul, causal attention, the 512-variant candidate sweep).

With N > 1 (one process per GPU, launched by torchrun) ONE instance of N times the rows is split by
core range: rank r runs cores [32 r, 32 r + 32), uploads only the rows they read and reads back
only the rows they wrote; nothing is exchanged (``scaling: weak``).  ``extras.strong`` is the
fixed 8192-row instance split the same way, ``extras.candidates`` the sweep with candidate i on
rank i mod N.  ``--impl reference`` times the reference interpreter on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


# ---------------------------------------------------------------------------
# Workloads: KTIR source, seeded synthetic inputs, algorithmic work per step
# ---------------------------------------------------------------------------
class Workload:
    name = func = kernel = describe = metric = ""
    unit = "elem/s"
    bound = "hbm"
    dtype = "f32"
    units_per_step = 0          # elements (or FLOP) one step processes
    algo_per_step = 0           # algorithmic bytes (hbm) or FLOP (tensor) of the dominant kernel
    cpu_ladder = ()             # (size, rough seconds on one core of the reference) for CPU samples

    def source(self): ...
    def inputs(self, rank=0): ...
    def check(self, kw, res): return None
    def cpu_case(self, size, seed): ...     # (source, func, kwargs, units) of a bounded CPU sample


def _rows_fix(rows, cores, r):
    cores = max(1, min(cores, rows // r))
    while rows % (cores * r):
        cores -= 1
    return cores


class Softmax(Workload):
    name, func, kernel = "softmax", "softmax_kernel", "ktb_row_softmax_fast_kernel"
    C, RPI = 4096, 8
    metric = "KTIR exec throughput (row softmax 8192x4096 f16, f32 stats)"
    cpu_ladder = ((512, 0.3), (2048, 1.4), (4096, 6.0), (8192, 24.0))

    def __init__(self, scale=1):
        self.R, self.CORES = 8192 * scale, 32 * scale
        self.units_per_step = self.R * self.C
        self.algo_per_step = 2 * self.R * self.C * 2
        self.describe = (f"row_softmax f16[{self.R},4096], grid {self.CORES} cores x 256 rows, 8 rows/iteration, "
                         "f32 stats")

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.softmax_rows(self.R, self.C, self.CORES, self.RPI, True)

    def _x(self, rows, seed):
        return (np.random.default_rng(seed).standard_normal((rows, self.C), dtype=np.float32) * 2).astype(np.float16)

    def inputs(self, rank=0, rows=None):
        """``rows = (lo, hi)``: only these rows carry data (a rank's share of a split instance)."""
        if rows is None:
            x = self._x(self.R, 2 + rank)
        else:
            x = np.zeros((self.R, self.C), np.float16)
            x[rows[0]:rows[1]] = self._x(rows[1] - rows[0], 2 + rank)
        return dict(output_ptr=np.zeros_like(x), input_ptr=x)

    def check(self, kw, res, rows=None):
        x, y = kw["input_ptr"], res["output_ptr"]
        lo, hi = rows or (0, self.R)
        pick = np.arange(lo, hi, 257)
        xf = np.asarray(x[pick], dtype=np.float32)
        e = np.exp(xf - xf.max(1, keepdims=True))
        return float(np.abs(y[pick].astype(np.float32) - e / e.sum(1, keepdims=True)).max())

    def cpu_case(self, rows, seed=2):
        from ktir_cpu_b200 import kernels as K
        cores = _rows_fix(rows, 32, self.RPI)
        x = self._x(rows, seed)
        return (K.softmax_rows(rows, self.C, cores, self.RPI, True), self.func,
                dict(output_ptr=np.zeros_like(x), input_ptr=x), rows * self.C)


class VectorAdd(Workload):
    name, func, kernel = "vector_add", "add_kernel", "ktb_ew_f16_kernel"
    N, BLOCK, CORES = 1 << 26, 131072, 32
    units_per_step = N
    algo_per_step = 3 * N * 2
    describe = "vector_add f16[2^26], 32 cores x 16 blocks of 131072 (scaled twin of the 4096-element example)"
    metric = "KTIR exec throughput (vector_add 2^26 f16)"
    dtype = "f16"
    cpu_ladder = ((1 << 22, 0.3), (1 << 24, 3.0), (1 << 26, 23.0))

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.vector_add(self.N, self.BLOCK, self.CORES)

    def inputs(self, rank=0):
        rng = np.random.default_rng(1 + rank)
        x = rng.standard_normal(self.N, dtype=np.float32).astype(np.float16)
        y = rng.standard_normal(self.N, dtype=np.float32).astype(np.float16)
        return dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(self.N, np.float16), BLOCK_SIZE=self.BLOCK)

    def check(self, kw, res):
        return float(np.abs((kw["x_ptr"][:65536] + kw["y_ptr"][:65536]).astype(np.float32)
                            - res["output_ptr"][:65536].astype(np.float32)).max())

    def cpu_case(self, n, seed=1):
        from ktir_cpu_b200 import kernels as K
        rng = np.random.default_rng(seed)
        x = rng.standard_normal(n, dtype=np.float32).astype(np.float16)
        y = rng.standard_normal(n, dtype=np.float32).astype(np.float16)
        blk = min(self.BLOCK, n // 32)
        return (K.vector_add(n, blk, 32), self.func,
                dict(x_ptr=x, y_ptr=y, output_ptr=np.zeros(n, np.float16), BLOCK_SIZE=blk), n)


class GatherScatter(Workload):
    name, func, kernel = "gather_scatter", "gather_scale_scatter", "ktb_scatter_apply_axpy128h_kernel"
    ROWS, COLS, NIDX, TILE, CORES = 65536, 128, 262144, 64, 64
    units_per_step = NIDX * COLS
    algo_per_step = NIDX * (4 + 3 * COLS * 2)
    describe = ("gather + x0.5 + read-modify-write scatter: table f16[65536,128], 262144 int32 indices, "
                "64-row tiles with 6 duplicates per tile, 64 cores")
    metric = "KTIR exec throughput (indirect gather+scatter, gathered elements)"
    dtype = "f16"
    accumulates = "out_ptr"       # the kernel adds into this tensor: re-uploaded before the timed region
    cpu_ladder = ((2048, 2.6), (4096, 5.1), (8192, 10.7))

    def _idx(self, rng, rows, n):
        idx = rng.integers(0, rows, n)
        for t in range(n // self.TILE):
            pos = rng.choice(self.TILE, 12, replace=False)
            idx[t * self.TILE + pos[:6]] = idx[t * self.TILE + pos[6:]]
        return idx.astype(np.int32)

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.gather_scale_scatter(self.ROWS, self.COLS, self.NIDX, self.TILE, self.CORES)

    def inputs(self, rank=0):
        rng = np.random.default_rng(3 + rank)
        table = rng.standard_normal((self.ROWS, self.COLS), dtype=np.float32).astype(np.float16)
        return dict(table_ptr=table, idx_ptr=self._idx(rng, self.ROWS, self.NIDX), out_ptr=np.zeros_like(table))

    def check(self, kw, res):
        idx = kw["idx_ptr"].reshape(-1, self.TILE)[:64]
        rows = np.unique(idx)
        counts = np.zeros(self.ROWS, np.int64)
        for t in kw["idx_ptr"].reshape(-1, self.TILE):
            counts[np.unique(t)] += 1
        h = (kw["table_ptr"][rows] * np.float16(0.5)).astype(np.float16)
        acc = np.zeros_like(h)
        for n in range(1, int(counts[rows].max()) + 1):
            m = counts[rows] >= n
            acc[m] = acc[m] + h[m]
        return float(np.abs(res["out_ptr"][rows].astype(np.float32) - acc.astype(np.float32)).max())

    def cpu_case(self, n, seed=3):
        from ktir_cpu_b200 import kernels as K
        rng = np.random.default_rng(seed)
        rows = max(64, n // 4)
        table = rng.standard_normal((rows, self.COLS), dtype=np.float32).astype(np.float16)
        cores = max(1, min(self.CORES, n // self.TILE))
        return (K.gather_scale_scatter(rows, self.COLS, n, self.TILE, cores), self.func,
                dict(table_ptr=table, idx_ptr=self._idx(rng, rows, n), out_ptr=np.zeros_like(table)),
                n * self.COLS)


class Matmul(Workload):
    name, func, kernel = "matmul", "matmul_kernel", "ktb_gemm_f16_pair_kernel"
    M = N = KK = 4096
    unit, bound = "FLOP/s", "tensor"
    units_per_step = 2 * M * N * KK
    algo_per_step = units_per_step
    describe = "tiled matmul f16 4096^3, 64x64 tiles, K-step 64, 32 cores x 128 tiles, f32 accumulate"
    metric = "KTIR exec throughput (tiled matmul 4096^3 f16, f32 accumulate)"
    cpu_ladder = ((512, 0.2), (1024, 1.5), (2048, 12.0))

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.tiled_matmul(self.M, self.N, self.KK, 64, 64, 64, 32, True)

    def inputs(self, rank=0):
        rng = np.random.default_rng(4 + rank)
        a = rng.uniform(-1, 1, (self.M, self.KK)).astype(np.float16)
        b = rng.uniform(-1, 1, (self.KK, self.N)).astype(np.float16)
        return dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((self.M, self.N), np.float16))

    def check(self, kw, res):
        rows = np.arange(0, self.M, 409)
        want = kw["a_ptr"][rows].astype(np.float32) @ kw["b_ptr"].astype(np.float32)
        return float(np.abs(res["c_ptr"][rows].astype(np.float32) - want).max())

    def cpu_case(self, n, seed=4):
        from ktir_cpu_b200 import kernels as K
        rng = np.random.default_rng(seed)
        a = rng.uniform(-1, 1, (n, n)).astype(np.float16)
        b = rng.uniform(-1, 1, (n, n)).astype(np.float16)
        cores = min(32, (n // 64) ** 2)
        return (K.tiled_matmul(n, n, n, 64, 64, 64, cores, True), self.func,
                dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((n, n), np.float16)), 2 * n ** 3)


def attention_kwargs(rng, S, H, D, tn):
    """Inputs of a ``paged_attention_kernel`` call that is dense causal attention: identity block
    table, no context before the queries."""
    q, k, v = (rng.standard_normal((S, H, D), dtype=np.float32).astype(np.float16) for _ in range(3))
    nt = S // tn
    return dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k.reshape(nt, tn, H, D),
                value_cache_ptr=v.reshape(nt, tn, H, D), block_tables_ptr=np.arange(nt, dtype=np.int32).reshape(1, -1),
                cur_batch_start_index=0, block_table_offset=0, num_tiles=nt, context_len=0,
                scale=np.float32(1.0 / np.sqrt(D)))


def attention_check(kw, out, h):
    S, D = kw["query_ptr"].shape[0], kw["query_ptr"].shape[2]
    q = kw["query_ptr"][:, h].astype(np.float64)
    k = kw["key_cache_ptr"][:, :, h].reshape(S, D).astype(np.float64)
    v = kw["value_cache_ptr"][:, :, h].reshape(S, D).astype(np.float64)
    sc = np.where(np.tril(np.ones((S, S), bool)), q @ k.T / np.sqrt(D), -np.inf)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    return float(np.abs(out[:, h].astype(np.float64) - (p / p.sum(-1, keepdims=True)) @ v).max())


class Attention(Workload):
    name, func, kernel = "attention", "paged_attention_kernel", "ktb_attention_fwd_kernel"
    S, H, D, TM, TN = 2048, 256, 128, 128, 128
    unit, bound = "FLOP/s", "tensor"
    units_per_step = 4 * H * D * (S * (S + 1) // 2)
    algo_per_step = units_per_step
    describe = ("causal attention f16 B8 H32 (batch folded into 256 heads) S2048 D128: the paged-attention kernel "
                "shape of the reference's generator, identity block table, tiles 128x128, f32 online softmax")
    metric = "KTIR exec throughput (causal attention B8 H32 S2048 D128, causal FLOP)"
    cpu_ladder = ((256, 0.8), (512, 3.0), (1024, 12.0), (2048, 49.0))

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.paged_attention(self.S, self.S, self.H, self.H, self.D, self.TN, self.TM)

    def inputs(self, rank=0):
        return attention_kwargs(np.random.default_rng(5 + rank), self.S, self.H, self.D, self.TN)

    def check(self, kw, res):
        return attention_check(kw, res["output_ptr"], 3)

    def cpu_case(self, S, seed=5):
        from ktir_cpu_b200 import kernels as K
        return (K.paged_attention(S, S, 1, 1, self.D, self.TN, self.TM), self.func,
                attention_kwargs(np.random.default_rng(seed), S, 1, self.D, self.TN),
                4 * self.D * (S * (S + 1) // 2))


class LayerNorm(Workload):
    """The reference's layer-norm example (examples/triton-ktir/layernorm_fwd_ktir.mlir: f16 throughout, rows
    walked in column blocks, Mean and Rstd kept per row) at 4096 rows of its 8192 columns."""
    name, func, kernel = "layernorm", "_layer_norm_fwd_fused", "ktb_row_norm_h_kernel"
    ROWS, COLS, BLOCK, CORES = 4096, 8192, 1024, 32
    units_per_step = ROWS * COLS
    algo_per_step = 4 * ROWS * COLS * 2 + 2 * ROWS * 2          # X, W, B read, Y written; Mean and Rstd
    describe = ("layer norm f16[4096,8192] in 8 column blocks of 1024 with per-element weight and bias tiles, Mean and "
                "Rstd per row, 32 cores (row-scaled twin of the reference's 1151x8192 example)")
    metric = "KTIR exec throughput (layer norm 4096x8192 f16, column-blocked)"
    dtype = "f16"
    cpu_ladder = ((128, 0.8), (512, 3.1), (2048, 12.6), (4096, 25.0))

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.layernorm_blocked(self.ROWS, self.COLS, self.BLOCK, self.CORES)

    def _kw(self, rows, seed):
        rng = np.random.default_rng(seed)
        t = lambda: rng.standard_normal((rows, self.COLS), dtype=np.float32).astype(np.float16)     # noqa: E731
        return dict(X=t(), Y=np.zeros((rows, self.COLS), np.float16), W=t(), B=t(), Mean=np.zeros(rows, np.float16),
                    Rstd=np.zeros(rows, np.float16), N=self.COLS, eps=np.float16(1e-5), BLOCK_SIZE=self.BLOCK)

    def inputs(self, rank=0):
        return self._kw(self.ROWS, 6 + rank)

    def check(self, kw, res):
        pick = np.arange(0, self.ROWS, 131)
        x = kw["X"][pick].astype(np.float64)
        mean = x.mean(1, keepdims=True)
        y = (x - mean) / np.sqrt(x.var(1, keepdims=True) + 1e-5) * kw["W"][pick].astype(np.float64) + kw["B"][pick].astype(np.float64)
        return float(max(np.abs(res["Y"][pick].astype(np.float64) - y).max(),
                         np.abs(res["Mean"][pick].astype(np.float64) - mean[:, 0]).max()))

    def cpu_case(self, rows, seed=6):
        from ktir_cpu_b200 import kernels as K
        return (K.layernorm_blocked(rows, self.COLS, self.BLOCK, min(self.CORES, rows)), self.func, self._kw(rows, seed),
                rows * self.COLS)


WORKLOADS = {w.name: w for w in (Softmax(), VectorAdd(), GatherScatter(), Matmul(), Attention(), LayerNorm())}


def measured_peak(bound):
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return (float(d["hbm_gbs"]), "GB/s", "measured (MEASURED_PEAKS.json)") if bound == "hbm" else \
            (float(d["bf16_tflops"]), "TFLOP/s", "measured burst (MEASURED_PEAKS.json)")
    except Exception:
        return (6650.0, "GB/s", "fallback") if bound == "hbm" else (1590.0, "TFLOP/s", "fallback")


def dram_traffic(name):
    """DRAM read + write bytes of one launch of the dominant kernel, from the ncu capture summarised
    under profiles/."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "traffic.json"))).get(name)
        return t["dram_read_bytes"] + t["dram_write_bytes"] if t else None
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx, self.first = [], None, gpu_index, 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 5.0:      # first sample = the sampler is live
                time.sleep(0.02)
            self.first = len(self.rows)
        except Exception:
            self.proc = None

    def under_load(self):
        return len(self.rows) - self.first

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        rows = self.rows[self.first:]

        def num(s):
            try:
                return float(s)
            except ValueError:
                return None
        sm = [num(r[1]) for r in rows if len(r) > 8 and num(r[1]) is not None]
        mx = [num(r[2]) for r in rows if len(r) > 8 and num(r[2]) is not None]
        reasons = set()
        for r in rows:
            if len(r) > 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU side: the reference interpreter (baseline/_ref) or, without it, the oracle port
# ---------------------------------------------------------------------------
def reference_available():
    return os.path.isdir(os.path.join(REF_DIR, "ktir_cpu"))


def _cpu_interpreter():
    if reference_available():
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from ktir_cpu import KTIRInterpreter
        return KTIRInterpreter()
    from oracle.numpy_interp import OracleInterpreter
    return OracleInterpreter()


def _cpu_worker(args):
    name, size, seed = args
    src, fn, kw, units = WORKLOADS[name].cpu_case(size, seed)
    it = _cpu_interpreter()
    it.load(src)
    t0 = time.perf_counter()
    it.execute_function(fn, **kw)
    return time.perf_counter() - t0, units


def _cpu_import(_):
    _cpu_interpreter()
    import ktir_cpu_b200.kernels  # noqa: F401
    return 0


def host_cores():
    try:
        return max(1, min(len(os.sched_getaffinity(0)), 32))
    except AttributeError:
        return max(1, min(os.cpu_count() or 1, 32))


def ladder_size(w, per_step_s):
    """Largest sample of ``w`` the reference finishes in about ``per_step_s`` on one core (the port is
    roughly ten times faster, so it gets the largest)."""
    if not reference_available():
        return w.cpu_ladder[-1][0]
    ok = [s for s, t in w.cpu_ladder if t <= per_step_s]
    return ok[-1] if ok else w.cpu_ladder[0][0]


def cpu_sample(w, procs, size, pool=None):
    """units/s of the CPU interpreter on ``procs`` host processes, each running its own instance
    of the kernel at ``size`` (seeds differ).  Returns (units/s, seconds)."""
    import multiprocessing as mp
    own = pool is None
    if own:
        pool = mp.get_context("spawn").Pool(procs)
        pool.map(_cpu_import, range(procs))       # interpreter start-up stays outside the timing
    try:
        t0 = time.perf_counter()
        out = pool.map(_cpu_worker, [(w.name, size, 2 + i) for i in range(procs)])
        dt = time.perf_counter() - t0
    finally:
        if own:
            pool.close()
    return sum(u for _, u in out) / dt, dt


def cpu_baseline(w, per_step_s=20.0):
    procs = host_cores()
    size = ladder_size(w, per_step_s)
    v, dt = cpu_sample(w, procs, size)
    kind = "reference" if reference_available() else "port"
    what = "the reference interpreter (baseline/_ref)" if kind == "reference" else "oracle/numpy_interp.py"
    return {"value": v, "unit": w.unit, "cores": procs, "kind": kind,
            "sample": f"{procs} processes, each the same KTIR kernel at size {size} (full size "
                      f"{w.cpu_ladder[-1][0]}) through {what}, NumPy {np.__version__}, {dt:.1f} s"}


def run_reference(args, w):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import multiprocessing as mp
    procs = host_cores()
    size = ladder_size(w, 150.0 / max(1, args.steps + args.warmup))
    kind = "reference" if reference_available() else "port"
    res = []
    with mp.get_context("spawn").Pool(procs) as pool:
        pool.map(_cpu_import, range(procs))
        for i in range(args.warmup + args.steps):
            v, dt = cpu_sample(w, procs, size, pool)
            if i >= args.warmup:
                res.append((v, dt))
    value = float(np.mean([v for v, _ in res]))
    what = "the unmodified reference package (baseline/_ref)" if kind == "reference" else "oracle/numpy_interp.py"
    sample = (f"{procs} processes, each the same KTIR kernel at size {size} (full size {w.cpu_ladder[-1][0]}) "
              f"through {what}, NumPy {np.__version__}")
    line = {"impl": "reference", "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean([dt for _, dt in res])) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
            "data": "synthetic", "config": {"workload": w.describe, "units_per_step_per_gpu": w.units_per_step},
            "cpu_baseline": {"value": value, "unit": w.unit, "cores": procs, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------
class Dist:
    """torch.distributed when there is more than one rank, no-ops otherwise."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.d = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.d, self.torch = dist, torch

    def barrier(self):
        if self.d is not None:
            self.d.barrier()

    def max(self, *vals):
        if self.d is None:
            return [float(v) for v in vals]
        t = self.torch.tensor(list(vals), device="cuda", dtype=self.torch.float64)
        self.d.all_reduce(t, op=self.d.ReduceOp.MAX)
        return [float(x) for x in t]

    def close(self):
        if self.d is not None:
            self.d.destroy_process_group()


def pin_near_gpu(local):
    """Keep this process (and its copy threads) on the CPUs of the GPU's NUMA node, so that eight
    ranks do not all stage through one node's memory.  Read-only look-ups; nothing is changed on
    the GPU."""
    try:
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(local)],
                             capture_output=True, text=True, timeout=10).stdout.strip().lower()
        if bus.startswith("00000000:"):
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    return None


def pinned_copy(dev, kw):
    from ktir_cpu_b200.pinned import pinned_empty
    out = {}
    for k, v in kw.items():
        if isinstance(v, np.ndarray):
            p = pinned_empty(dev, v.shape, v.dtype)
            p[...] = v
            out[k] = p
        else:
            out[k] = v
    return out


def time_device(dev, run, steps, warm):
    """Per-step milliseconds of ``run()``: CUDA events on the launch stream, L2 flushed before each."""
    for _ in range(warm):
        run()
    dev.sync()
    per_step = []
    l0 = dev.launch_count()
    for _ in range(steps):
        dev.flush_l2()
        dev.record(0)
        run()
        dev.record(1)
        dev.sync()
        per_step.append(dev.elapsed_ms(0, 1))
    return per_step, dev.launch_count() - l0


def time_sustained(dev, sess, sets=8, reps=3):
    """Milliseconds per launch when ``sets`` launches over distinct copies of the arena run back to
    back inside one event pair (no flush): steady-state streaming, deferred write-back included."""
    size = sess.arena_bytes + 256
    arenas = [sess.arena] + [dev.alloc(size) for _ in range(sets - 1)]
    try:
        for a in arenas[1:]:
            dev.check(dev.lib.ktb_d2d(dev.h, a, sess.arena, sess.arena_bytes))
        dev.sync()
        best = None
        for _ in range(reps + 1):
            dev.flush_l2()
            dev.record(2)
            for a in arenas:
                sess.plan.launch(dev, a)
            dev.record(3)
            dev.sync()
            ms = dev.elapsed_ms(2, 3) / sets
            best = ms if best is None else min(best, ms)
        return best
    finally:
        for a in arenas[1:]:
            dev.free(a)


def time_e2e(call, steps, warm=3):
    """Seconds per call of ``call()`` (host arrays in, fresh host arrays out), results of the previous
    call still alive while the next one runs, as in a caller's loop."""
    res = None
    for _ in range(warm):
        res = call()
    t0 = time.perf_counter()
    for _ in range(steps):
        res = call()
    return (time.perf_counter() - t0) / steps, res


def report(w, interp, kw_host, steps, warm, dist, clocks_for=None, shard=None, world_units=1, cpu=True,
           sustained=True, check_rows=None):
    """Device-timed throughput, roofline, end-to-end and CPU baseline of one workload."""
    dev = interp.device
    kw = pinned_copy(dev, kw_host)
    sess, _ = interp.session(w.func, _shard=shard, **kw)
    tp = sess.transfer_plan()
    for k, v in kw.items():
        if isinstance(v, np.ndarray) and k not in sess.no_upload:
            sess.upload(k, v)
    dev.sync()
    sampler = None
    if clocks_for is not None:
        sampler = ClockSampler(clocks_for)
        sampler.start()
    for _ in range(warm):
        sess.run()
    if getattr(w, "accumulates", None):
        sess.upload(w.accumulates, kw[w.accumulates])
    dev.sync()
    dist.barrier()
    per_step, launches = time_device(dev, sess.run, steps, 0)
    if sampler is not None:
        # a timed region shorter than the sampling period: keep the same load running (untimed) until
        # the sampler has seen it a few times
        t_extra = time.time()
        while sampler.proc is not None and sampler.under_load() < 4 and time.time() - t_extra < 3.0:
            sess.run()
            dev.sync()
    dist.barrier()
    clocks = sampler.stop() if sampler is not None else None
    total_ms = float(sum(per_step))

    if shard is None:
        call_pinned = lambda: interp.execute_function(w.func, **kw)             # noqa: E731
        call_pageable = lambda: interp.execute_function(w.func, **kw_host)      # noqa: E731
    else:
        call_pinned = lambda: interp.execute_shard(w.func, shard[0], shard[1], **kw)          # noqa: E731
        call_pageable = lambda: interp.execute_shard(w.func, shard[0], shard[1], **kw_host)   # noqa: E731
    e2e_steps = max(3, min(steps, 10))
    dist.barrier()
    e2e_s, res = time_e2e(call_pinned, e2e_steps)
    if check_rows is not None:
        err = w.check(kw, res, check_rows)
    else:
        err = w.check(kw, res) if shard is None else None      # a rank holds only its slabs
    dist.barrier()
    e2e_pg, _ = time_e2e(call_pageable, e2e_steps)
    del res
    total_ms, e2e_s, e2e_pg = dist.max(total_ms, e2e_s, e2e_pg)
    ms = total_ms / steps
    peak, punit, peak_src = measured_peak(w.bound)
    scale = 1e9 if w.bound == "hbm" else 1e12
    units = w.units_per_step * world_units
    algo = w.algo_per_step // (shard[1] if shard else 1)        # one rank's launch covers its share of the instance
    achieved = algo / (ms * 1e-3) / scale
    out = {"metric": w.metric, "workload": w.describe, "value": units / (ms * 1e-3), "unit": w.unit, "ms_per_step": ms,
           "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": punit, "frac": achieved / peak,
                        "traffic": dram_traffic(w.name), "peak_source": peak_src, "algorithmic_per_launch": algo,
                        "kernel": w.kernel},
           "e2e": {"value": units / e2e_s, "unit": w.unit, "h2d_bytes_per_step": int(tp.h2d_bytes),
                   "d2h_bytes_per_step": int(tp.d2h_bytes), "ms_per_step": e2e_s * 1e3,
                   "parts": len(tp.chunks), "pageable": {"value": units / e2e_pg, "ms_per_step": e2e_pg * 1e3}},
           "gpu_launches": int(launches), "max_abs_err_spot_check": err}
    if clocks is not None:
        out["clocks"] = clocks
    if sustained and w.bound == "hbm" and shard is None:
        if getattr(w, "accumulates", None):
            sess.upload(w.accumulates, kw[w.accumulates])
        sms = time_sustained(dev, sess)
        ach = algo / (sms * 1e-3) / scale
        out["roofline"]["frac_sustained"] = ach / peak
        out["roofline"]["sustained"] = {"achieved": ach, "ms_per_launch": sms,
                                        "how": "8 back-to-back launches over 8 distinct arenas, one event pair, no L2 flush"}
        if algo // 2 <= (2 << 30):
            cms = time_copy_sustained(dev, algo // 2)
            cach = algo / (cms * 1e-3) / scale
            out["roofline"]["sustained"]["device_copy_same_bytes"] = {
                "achieved": cach, "ms_per_copy": cms, "kernel_over_copy": ach / cach,
                "how": "cudaMemcpyAsync device to device moving the same bytes (half read, half written), timed the same way"}
    if cpu and dist.rank == 0:
        out["cpu_baseline"] = cpu_baseline(w)
    return out


def time_copy_sustained(dev, nbytes, sets=8, reps=3):
    """Milliseconds per plain device-to-device copy of ``nbytes`` (read ``nbytes``, write ``nbytes``), measured like
    ``time_sustained``: ``sets`` copies over distinct buffers back to back inside one event pair.  What the
    memory system gives a kernel-free stream of this size — the measured peak is quoted on far larger buffers."""
    bufs = [dev.alloc(2 * nbytes + 256) for _ in range(sets)]
    try:
        for b in bufs:
            dev.check(dev.lib.ktb_memset(dev.h, b, 1, 2 * nbytes))
        dev.sync()
        best = None
        for _ in range(reps + 1):
            dev.flush_l2()
            dev.record(2)
            for b in bufs:
                dev.check(dev.lib.ktb_d2d(dev.h, b + nbytes, b, nbytes))
            dev.record(3)
            dev.sync()
            ms = dev.elapsed_ms(2, 3) / sets
            best = ms if best is None else min(best, ms)
        return best
    finally:
        for b in bufs:
            dev.free(b)


def host_link_probe(dev, dist, mib=64, reps=8):
    """GB/s this rank moves when every rank copies ``mib`` MiB up and ``mib`` MiB down at once between
    page-locked memory and its GPU (plain DMA, no kernels, no host copies), and the sum over ranks:
    what the host gives N GPUs together, the ceiling of any end-to-end number."""
    from ktir_cpu_b200.pinned import pinned_empty
    n = mib << 20
    a, b = pinned_empty(dev, (n,), np.uint8), pinned_empty(dev, (n,), np.uint8)
    a[:] = 1
    from ktir_cpu_b200 import runtime as R
    up = (R.PipeRegion * 1)(R.PipeRegion(0, 0, 0, 0, n, 1, n))
    down = (R.PipeRegion * 1)(R.PipeRegion(1, 0, n, 0, n, 1, n))
    import ctypes as C
    chunk = (R.PipeChunk * 1)()
    chunk[0].n_up, chunk[0].n_down, chunk[0].up, chunk[0].down = 1, 1, up, down
    ptrs = (C.c_void_p * 2)(a.ctypes.data, b.ctypes.data)
    arena = dev.alloc(2 * n)

    def once():
        dev.run_pipeline(arena, chunk, 1, ptrs, ptrs, 2)        # source already page-locked: DMA only, both lanes
        dev.sync()
    once()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        once()
    dt = (time.perf_counter() - t0) / reps
    (dt,) = dist.max(dt)
    dev.free(arena)
    per_rank = 2 * n / dt / 1e9
    return {"per_rank_gbs": per_rank, "aggregate_gbs": per_rank * dist.world,
            "what": f"{mib} MiB up + {mib} MiB down per rank at the same time, page-locked memory, max time over ranks"}


def candidate_sweep(n=512, B=1, H=4, D=128):
    """The 512-variant attention sweep: variant i has tile_m = (32,64,128)[i%3],
    tile_n = (32,64,128)[(i//3)%3], S = (512,1024,2048)[(i//9)%3], inputs seeded 1000+i.
    B and H are not fixed by the configuration; B=1, H=4 keeps the CPU interpreter able to finish a sample."""
    from ktir_cpu_b200 import kernels as K
    from ktir_cpu_b200.batch import Candidate
    out, flops = [], 0
    for i in range(n):
        tm, tn, S = (32, 64, 128)[i % 3], (32, 64, 128)[(i // 3) % 3], (512, 1024, 2048)[(i // 9) % 3]
        kw = attention_kwargs(np.random.default_rng(1000 + i), S, B * H, D, tn)
        out.append(Candidate(K.paged_attention(S, S, B * H, B * H, D, tn, tm), "paged_attention_kernel", kw, tag=(tm, tn, S)))
        flops += 4 * B * H * D * (S * (S + 1) // 2)
    return out, flops


def _candidate_cpu_worker(i):
    from ktir_cpu_b200 import kernels as K
    tm, tn, S = (32, 64, 128)[i % 3], (32, 64, 128)[(i // 3) % 3], (512, 1024, 2048)[(i // 9) % 3]
    kw = attention_kwargs(np.random.default_rng(1000 + i), S, 4, 128, tn)
    it = _cpu_interpreter()
    it.load(K.paged_attention(S, S, 4, 4, 128, tn, tm))
    t0 = time.perf_counter()
    it.execute_function("paged_attention_kernel", **kw)
    return time.perf_counter() - t0


def candidates_report(dist, sweeps=2, cpu=True):
    """kernels/s over the candidate sweep, host arrays in and out for every candidate (there is no
    device-resident variant of this metric: a candidate arrives as text + host tensors)."""
    from ktir_cpu_b200.batch import BatchRunner
    n = 512
    cands, flops = candidate_sweep(n)
    runner = BatchRunner(dist.local)
    checks = {}

    def score(i, c, out):
        if i % 27 == (7 * dist.rank + i // 27) % 27:       # one head of a few variants of every kernel, against f64 math
            checks[i] = attention_check(c.kwargs, out["output_ptr"], 1)
        return True
    warm = runner.run(cands[:54 * dist.world], dist.rank, dist.world, score=score, keep_outputs=False)
    res = runner.run(cands, dist.rank, dist.world, keep_outputs=True)   # one untimed sweep: result buffers exist
    dist.barrier()
    t0 = time.perf_counter()
    launches = 0
    for _ in range(sweeps):
        res = None                            # the consumer is done with the previous sweep's results
        res = runner.run(cands, dist.rank, dist.world, keep_outputs=True)
        launches += res.launches
    dt = time.perf_counter() - t0
    errs = len(res.errors) + len(warm.errors)
    dt, errs, worst = dist.max(dt, float(errs), max(checks.values()) if checks else 0.0)
    h2d = sum(v.nbytes for c in cands for k, v in c.kwargs.items() if isinstance(v, np.ndarray) and k != "output_ptr")
    d2h = sum(c.kwargs["output_ptr"].nbytes for c in cands)
    out = {"metric": "candidate kernels evaluated per second (512-variant causal attention sweep)",
           "value": n * sweeps / dt, "unit": "kernels/s", "ms_per_step": dt / sweeps * 1e3,
           "workload": "512 variants: tile_m, tile_n in {32,64,128}, S in {512,1024,2048}, B=1, H=4, D=128; variant i on "
                       "rank i % world; 27 distinct kernels parsed and planned once",
           "roofline": {"bound": "tensor", "achieved": flops * sweeps / dt / 1e12, "unit": "TFLOP/s",
                        "peak": measured_peak("tensor")[0], "frac": flops * sweeps / dt / 1e12 / measured_peak("tensor")[0],
                        "traffic": None, "note": "whole sweep including host transfers; the sweep is transfer-bound"},
           "e2e": {"value": n * sweeps / dt, "unit": "kernels/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "gpu_launches": int(launches), "failed_candidates": int(errs), "max_abs_err_spot_check": worst}
    runner.close()
    if cpu and dist.rank == 0:
        import multiprocessing as mp
        procs = host_cores()
        picks = list(range(9))                   # the nine S = 512 variants: the cheapest third of the sweep
        with mp.get_context("spawn").Pool(min(procs, len(picks))) as pool:
            pool.map(_cpu_import, range(min(procs, len(picks))))
            t1 = time.perf_counter()
            pool.map(_candidate_cpu_worker, picks)
            d1 = time.perf_counter() - t1
        kind = "reference" if reference_available() else "port"
        out["cpu_baseline"] = {"value": len(picks) / d1, "unit": "kernels/s", "cores": min(procs, len(picks)), "kind": kind,
                               "sample": f"variants 0-8 (S = 512, every tile pair; the cheapest third of the sweep) one per "
                                         f"process, {d1:.1f} s"}
    return out


# The block gathers of the reference's indirect-load benchmark (benchmarks/configs/load_path_compare.toml):
# label -> (source shape, rows selected per indirect dim).  Leading dims are looked up, the rest taken whole.
GATHER_WORKLOADS = {
    "moe-262K": ((128, 256, 128), (8,)), "moe-1M": ((128, 1024, 128), (8,)),
    "paged-attn-256K": ((1024, 16, 128, 128), (16,)),
    "sparse-attn-32K": ((1024, 512, 64), (4, 16)), "sparse-attn-128K": ((4096, 512, 256), (4, 16)),
    "retro-attn-16K": ((1024, 128, 128), (32, 4)), "multi-head-4M": ((128, 64, 256, 256), (8, 8)),
}


def _bit_pattern(n, seed):
    """n pseudo-random f16 bit patterns (finite values), generated in pieces: these sources reach 1 GiB."""
    out = np.empty(n, np.uint16)
    step = 1 << 24
    for i in range(0, n, step):
        j = min(n, i + step)
        x = (np.arange(i, j, dtype=np.uint64) + seed) * np.uint64(0x9E3779B97F4A7C15)
        out[i:j] = ((x >> np.uint64(40)) & np.uint64(0x7BFF)).astype(np.uint16)       # exponent < 31: no inf / NaN
    return out.view(np.float16)


def gathers_report(device, steps=10, cpu=True):
    """The seven block gathers as KTIR kernels (one indirect tile load + store), device-timed with the
    tensors resident: result bytes moved (read + written) per second against the HBM roofline, and — for
    the sizes the reference finishes in seconds — the reference interpreter on the same kernel."""
    from ktir_cpu_b200 import HardwareConfig, KTIRInterpreter, kernels as K
    peak, _, src_peak = measured_peak("hbm")
    rows = {}
    for label, (shape, sel) in GATHER_WORKLOADS.items():
        rshape = tuple(sel) + tuple(shape[len(sel):])
        rng = np.random.default_rng(17)
        kw = {"src_ptr": _bit_pattern(int(np.prod(shape)), 17).reshape(shape)}
        for i, n_ in enumerate(sel):
            kw[f"idx{i}_ptr"] = rng.choice(shape[i], n_, replace=False).astype(np.int32)
        kw["out_ptr"] = np.zeros(rshape, np.float16)
        it = KTIRInterpreter(device=device, latency_config=HardwareConfig(lx_size_mb=64))
        it.load(K.blocked_gather(shape, sel))
        try:
            sess, _ = it.session("blocked_gather", **kw)
            for k, v in kw.items():
                sess.upload(k, v)
            dev = it.device
            dev.sync()
            per_step, launches = time_device(dev, sess.run, steps, 3)
            got = sess.download("out_ptr")
            dev.sync()
            want = kw["src_ptr"][np.ix_(*[kw[f"idx{i}_ptr"] for i in range(len(sel))])]
            ok = bool(np.array_equal(got.view(np.uint16), want.view(np.uint16)))
            ms = float(np.mean(per_step))
            moved = 2 * want.nbytes + sum(kw[f"idx{i}_ptr"].nbytes for i in range(len(sel)))
            rows[label] = {"source_shape": list(shape), "result_shape": list(rshape), "kernels": [s_.kind for s_ in sess.plan.statements],
                           "t_indirect_load_us": ms * 1e3, "launches_per_step": launches // max(steps, 1),
                           "roofline": {"bound": "hbm", "achieved": moved / ms / 1e6, "peak": peak, "unit": "GB/s",
                                        "frac": moved / ms / 1e6 / peak, "peak_source": src_peak,
                                        "algorithmic_per_launch": moved},
                           "bit_exact": ok}
            if cpu and want.nbytes <= (4 << 20) and int(np.prod(shape)) <= (1 << 26):
                ref = _cpu_interpreter()
                if reference_available():
                    from ktir_cpu import HardwareConfig as RefConfig
                    ref = type(ref)(latency_config=RefConfig(lx_size_mb=64))
                ref.load(K.blocked_gather(shape, sel))
                t0 = time.perf_counter()
                r = ref.execute_function("blocked_gather", **kw)
                rows[label]["reference_ms"] = (time.perf_counter() - t0) * 1e3
                rows[label]["reference_equal"] = bool(np.array_equal(r["out_ptr"].view(np.uint16), want.view(np.uint16)))
        except Exception as e:                               # noqa: BLE001
            rows[label] = {"error": f"{type(e).__name__}: {e}"}
        it.close()
    return {"metric": "block gathers of the reference's indirect-load benchmark, tensors resident", "workloads": rows,
            "reference_kind": "reference" if reference_available() else "port",
            "note": "reference_ms is one execute_function call of the reference interpreter, host copies included"}


def run_gpu(args, w):
    dist = Dist()
    from ktir_cpu_b200.interpreter import KTIRInterpreter
    numa = None
    if dist.world > 1:
        from ktir_cpu_b200 import runtime as R
        R.lib().ktb_set_copy_threads(max(2, min(8, host_cores() // dist.world)))     # the ranks share the host cores
        numa = pin_near_gpu(dist.local)
    interp = KTIRInterpreter(device=dist.local)
    warm = max(args.warmup, 3)
    cpu = not args.no_cpu
    if dist.world == 1:
        interp.load(w.source())
        head = report(w, interp, w.inputs(0), args.steps, warm, dist, clocks_for=dist.local, cpu=cpu,
                      sustained=not args.no_sustained)
        sharding = "single GPU"
        scaling = "weak"
    else:
        # ONE instance of world x the rows, split by core range: this rank's cores own rows [lo, hi)
        big = Softmax(dist.world) if w.name == "softmax" else w
        interp.load(big.source())
        if w.name == "softmax":
            rows = (8192 * dist.rank, 8192 * (dist.rank + 1))
            kw = big.inputs(dist.rank, rows)
            head = report(big, interp, kw, args.steps, warm, dist, clocks_for=dist.local, shard=(dist.rank, dist.world),
                          cpu=False, sustained=False, check_rows=rows)
            head["metric"] = w.metric
            sharding = (f"one instance of {big.R} rows split over {dist.world} GPUs by core range (32 cores = 8192 rows per "
                        "rank); a rank uploads the rows its cores read and reads back the rows they wrote; no collective")
            scaling = "weak"
        else:
            kw = big.inputs(0)
            head = report(big, interp, kw, args.steps, warm, dist, clocks_for=dist.local, shard=(dist.rank, dist.world),
                          cpu=False, sustained=False)
            sharding = f"one instance split over {dist.world} GPUs (core ranges / destination-row ownership); no collective"
            scaling = "strong"
    line = {"metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": dist.world,
            "steps": args.steps, "warmup": warm, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": head["workload"], "units_per_step_per_gpu": w.units_per_step, "sharding": sharding,
                       "l2": "flushed (256 MiB written, 256 MiB read) between timed steps; each step timed by CUDA "
                             "events on the launch stream", "numa_node": numa},
            "roofline": head["roofline"], "e2e": head["e2e"], "gpu_launches": head["gpu_launches"],
            "clocks": head.get("clocks"), "max_abs_err_spot_check": head["max_abs_err_spot_check"]}
    if "cpu_baseline" in head:
        line["cpu_baseline"] = head["cpu_baseline"]
    interp.close()

    if not args.no_extras:
        extras = {}
        if dist.world == 1 and w.name == "softmax":
            for name in ("vector_add", "gather_scatter", "matmul", "attention", "layernorm"):
                x = WORKLOADS[name]
                it = KTIRInterpreter(device=dist.local)
                it.load(x.source())
                try:
                    extras[name] = report(x, it, x.inputs(0), max(5, args.steps // 2), warm, dist, cpu=cpu)
                except Exception as e:                       # noqa: BLE001 - an extra must not lose the headline
                    extras[name] = {"error": f"{type(e).__name__}: {e}"}
                it.close()
        elif dist.world > 1 and w.name == "softmax":
            x = WORKLOADS["softmax"]                         # the fixed-size instance, split the same way
            it = KTIRInterpreter(device=dist.local)
            it.load(x.source())
            try:
                s = report(x, it, x.inputs(0), args.steps, warm, dist, shard=(dist.rank, dist.world), cpu=False,
                           sustained=False, check_rows=(256 * 32 * dist.rank // dist.world, 256 * 32 * (dist.rank + 1) // dist.world))
                s["scaling"] = "strong"
                extras["strong"] = s
            except Exception as e:                           # noqa: BLE001
                extras["strong"] = {"error": f"{type(e).__name__}: {e}"}
            it.close()
        if w.name == "softmax":
            try:
                from ktir_cpu_b200 import runtime as R
                extras["host_link"] = host_link_probe(R.get_device(dist.local), dist)
            except Exception as e:                           # noqa: BLE001
                extras["host_link"] = {"error": f"{type(e).__name__}: {e}"}
            try:
                extras["candidates"] = candidates_report(dist, cpu=cpu and dist.world == 1)
            except Exception as e:                           # noqa: BLE001
                extras["candidates"] = {"error": f"{type(e).__name__}: {e}"}
            if dist.world == 1:
                try:
                    extras["indirect_gathers"] = gathers_report(dist.local, cpu=cpu)
                except Exception as e:                       # noqa: BLE001
                    extras["indirect_gathers"] = {"error": f"{type(e).__name__}: {e}"}
        line["extras"] = extras
    if dist.rank == 0:
        print(json.dumps(line))
    dist.close()


def run_candidates(args):
    dist = Dist()
    out = candidates_report(dist, sweeps=max(1, args.steps // 10), cpu=not args.no_cpu)
    if dist.rank == 0:
        line = {"metric": out["metric"], "value": out["value"], "unit": out["unit"], "n_gpus": dist.world,
                "steps": max(1, args.steps // 10), "warmup": 2, "ms_per_step": out["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": out["workload"]}, **{k: out[k] for k in out if k not in ("metric", "value", "unit",
                                                                                             "ms_per_step", "workload")}}
        print(json.dumps(line))
    dist.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="softmax", choices=sorted(WORKLOADS) + ["candidates", "gathers"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline samples")
    ap.add_argument("--no-extras", action="store_true", help="only the headline workload")
    ap.add_argument("--no-sustained", action="store_true", help="skip the eight-arena steady-state measurement")
    args = ap.parse_args()
    if args.workload == "candidates":
        return run_candidates(args)
    if args.workload == "gathers":
        print(json.dumps(gathers_report(0, max(3, args.steps // 2), cpu=not args.no_cpu)))
        return
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_gpu(args, w)


if __name__ == "__main__":
    main()

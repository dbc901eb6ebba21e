"""Benchmark of the KTIR execution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload (the one the headline metric is quoted on): row softmax over
f16[8192, 4096] with f32 statistics, 32 KTIR cores x 256 contiguous rows.  One
"step" is one pass of the hot path over the whole workload: the launch plan of
the KTIR function on tensors resident in HBM.  Prints ONE JSON line (rank 0).
``--impl reference`` times the CPU restatement of the reference interpreter
(oracle/) on the host cores instead.  Other workloads (vector_add,
gather_scatter, matmul, attention) report the same fields for the other
benchmark configurations.
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


# ---------------------------------------------------------------------------
# Workloads: KTIR source, seeded synthetic inputs, algorithmic work per step
# ---------------------------------------------------------------------------
class Workload:
    name = ""
    func = ""
    unit = "elem/s"
    bound = "hbm"
    kernel = ""
    dtype = "f32"
    units_per_step = 0          # elements (or FLOP) one step processes
    algo_per_step = 0           # algorithmic bytes (hbm) or FLOP (tensor) of the dominant kernel
    describe = ""

    def source(self): ...
    def inputs(self, rank=0): ...
    def check(self, kw, res): return None
    def cpu_case(self, procs): ...     # (source, func, kwargs, units) of a bounded CPU sample


def _rows_fix(rows, cores, r):
    cores = max(1, min(cores, rows // r))
    while rows % (cores * r):
        cores -= 1
    return cores


class Softmax(Workload):
    name, func, kernel = "softmax", "softmax_kernel", "ktb_row_softmax_fast_kernel"
    R, C, CORES, RPI = 8192, 4096, 32, 8
    units_per_step = R * C
    algo_per_step = 2 * R * C * 2
    describe = "row_softmax f16[8192,4096], grid 32 cores x 256 rows, 8 rows/iteration, f32 stats"
    metric = "KTIR exec throughput (row softmax 8192x4096 f16, f32 stats)"

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.softmax_rows(self.R, self.C, self.CORES, self.RPI, True)

    def _x(self, rows, seed):
        return (np.random.default_rng(seed).standard_normal((rows, self.C), dtype=np.float32) * 2).astype(np.float16)

    def inputs(self, rank=0):
        x = self._x(self.R, 2 + rank)
        return dict(output_ptr=np.zeros_like(x), input_ptr=x)

    def check(self, kw, res):
        x, y = kw["input_ptr"], res["output_ptr"]
        rows = np.arange(0, self.R, 257)
        xf = np.asarray(x[rows], dtype=np.float32)
        e = np.exp(xf - xf.max(1, keepdims=True))
        return float(np.abs(y[rows].astype(np.float32) - e / e.sum(1, keepdims=True)).max())

    def cpu_case(self, rows, seed=2):
        from ktir_cpu_b200 import kernels as K
        cores = _rows_fix(rows, self.CORES, self.RPI)
        x = self._x(rows, seed)
        return (K.softmax_rows(rows, self.C, cores, self.RPI, True), self.func,
                dict(output_ptr=np.zeros_like(x), input_ptr=x), rows * self.C)

    cpu_full, cpu_small = 8192, 8192


class VectorAdd(Workload):
    name, func, kernel = "vector_add", "add_kernel", "ktb_ew_stream_kernel"
    N, BLOCK, CORES = 1 << 26, 131072, 32
    units_per_step = N
    algo_per_step = 3 * N * 2
    describe = "vector_add f16[2^26], 32 cores x 16 blocks of 131072 (scaled twin of the 4096-element example)"
    metric = "KTIR exec throughput (vector_add 2^26 f16)"
    dtype = "f16"

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

    cpu_full, cpu_small = 1 << 26, 1 << 26


class GatherScatter(Workload):
    name, func, kernel = "gather_scatter", "gather_scale_scatter", "ktb_scatter_apply_axpy128_kernel"
    ROWS, COLS, NIDX, TILE, CORES = 65536, 128, 262144, 64, 64
    units_per_step = NIDX * COLS
    algo_per_step = NIDX * (4 + 3 * COLS * 2)
    describe = ("gather + x0.5 + read-modify-write scatter: table f16[65536,128], 262144 int32 indices, "
                "64-row tiles with 6 duplicates per tile, 64 cores")
    metric = "KTIR exec throughput (indirect gather+scatter, gathered elements)"
    dtype = "f16"

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

    def reset(self, sess, kw):
        sess.upload("out_ptr", kw["out_ptr"])      # the kernel accumulates into out

    def cpu_case(self, n, seed=3):
        from ktir_cpu_b200 import kernels as K
        rng = np.random.default_rng(seed)
        rows = max(64, n // 4)
        table = rng.standard_normal((rows, self.COLS), dtype=np.float32).astype(np.float16)
        cores = max(1, min(self.CORES, n // self.TILE))
        return (K.gather_scale_scatter(rows, self.COLS, n, self.TILE, cores), self.func,
                dict(table_ptr=table, idx_ptr=self._idx(rng, rows, n), out_ptr=np.zeros_like(table)),
                n * self.COLS)

    cpu_full, cpu_small = 262144, 131072


class Matmul(Workload):
    name, func, kernel = "matmul", "matmul_kernel", "ktb_gemm_f16_kernel"
    M = N = KK = 4096
    unit, bound = "FLOP/s", "tensor"
    units_per_step = 2 * M * N * KK
    algo_per_step = units_per_step
    describe = "tiled matmul f16 4096^3, 64x64 tiles, K-step 64, 32 cores x 128 tiles, f32 accumulate"
    metric = "KTIR exec throughput (tiled matmul 4096^3 f16, f32 accumulate)"

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
        tiles = (n // 64) ** 2
        cores = min(32, tiles)
        return (K.tiled_matmul(n, n, n, 64, 64, 64, cores, True), self.func,
                dict(a_ptr=a, b_ptr=b, c_ptr=np.zeros((n, n), np.float16)), 2 * n ** 3)

    cpu_full, cpu_small = 2048, 2048


class Attention(Workload):
    name, func, kernel = "attention", "attention_kernel", "ktb_attention_fwd_kernel"
    S, H, D, TM, TN = 2048, 256, 128, 128, 128
    unit, bound = "FLOP/s", "tensor"
    units_per_step = 4 * H * D * (S * (S + 1) // 2)
    algo_per_step = units_per_step
    describe = ("causal attention f16 B8 H32 (batch folded into 256 heads) S2048 D128, paged K/V with identity "
                "block table, tiles 128x128, f32 online softmax")
    metric = "KTIR exec throughput (causal attention B8 H32 S2048 D128, causal FLOP)"

    def source(self):
        from ktir_cpu_b200 import kernels as K
        return K.causal_attention(self.S, self.H, self.D, self.TM, self.TN)

    def _kw(self, rng, S, H):
        D, tn = self.D, self.TN
        q, k, v = (rng.standard_normal((S, H, D), dtype=np.float32).astype(np.float16) for _ in range(3))
        return dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k.reshape(S // tn, tn, H, D),
                    value_cache_ptr=v.reshape(S // tn, tn, H, D),
                    block_tables_ptr=np.arange(S // tn, dtype=np.int32).reshape(1, -1),
                    num_tiles=S // tn, context_len=0, scale=float(1.0 / np.sqrt(D)))

    def inputs(self, rank=0):
        return self._kw(np.random.default_rng(5 + rank), self.S, self.H)

    def check(self, kw, res):
        h = 3
        q = kw["query_ptr"][:, h].astype(np.float64)
        k = kw["key_cache_ptr"][:, :, h].reshape(self.S, self.D).astype(np.float64)
        v = kw["value_cache_ptr"][:, :, h].reshape(self.S, self.D).astype(np.float64)
        sc = q @ k.T / np.sqrt(self.D)
        sc = np.where(np.tril(np.ones((self.S, self.S), bool)), sc, -np.inf)
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        return float(np.abs(res["output_ptr"][:, h].astype(np.float64) - p @ v).max())

    def cpu_case(self, S, seed=5):
        from ktir_cpu_b200 import kernels as K
        H = 1
        return (K.causal_attention(S, H, self.D, self.TM, self.TN), self.func,
                self._kw(np.random.default_rng(seed), S, H), 4 * H * self.D * (S * (S + 1) // 2))

    cpu_full, cpu_small = 2048, 2048


WORKLOADS = {w.name: w for w in (Softmax(), VectorAdd(), GatherScatter(), Matmul(), Attention())}


def workload_config(w, n_gpus):
    return {"workload": w.describe, "units_per_step_per_gpu": w.units_per_step,
            "sharding": f"one independent replica of the workload per GPU (x{n_gpus}), no collective",
            "l2": "flushed (256 MiB memset) between timed steps; each step timed by CUDA events on the launch stream"}


def measured_peak(bound):
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return (float(d["hbm_gbs"]), "GB/s", "measured (MEASURED_PEAKS.json)") if bound == "hbm" else \
            (float(d["bf16_tflops"]), "TFLOP/s", "measured burst (MEASURED_PEAKS.json)")
    except Exception:
        return (6650.0, "GB/s", "fallback") if bound == "hbm" else (1590.0, "TFLOP/s", "fallback")


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

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
        """Samples taken since start() returned."""
        return len(self.rows) - getattr(self, "first", 0)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.rows = self.rows[getattr(self, "first", 0):]

        def num(s):
            try:
                return float(s)
            except ValueError:
                return None
        sm = [num(r[1]) for r in self.rows if len(r) > 8 and num(r[1]) is not None]
        mx = [num(r[2]) for r in self.rows if len(r) > 8 and num(r[2]) is not None]
        reasons = set()
        for r in self.rows:
            if len(r) > 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU side: the oracle port of the reference interpreter
# ---------------------------------------------------------------------------
def _cpu_worker(args):
    name, size, seed = args
    from oracle.numpy_interp import OracleInterpreter
    src, fn, kw, units = WORKLOADS[name].cpu_case(size, seed)
    it = OracleInterpreter()
    it.load(src)
    t0 = time.perf_counter()
    it.execute_function(fn, **kw)
    return time.perf_counter() - t0, units


def _cpu_import(_):
    import oracle.numpy_interp  # noqa: F401
    import ktir_cpu_b200.kernels  # noqa: F401
    return 0


def cpu_sample(w, procs, size):
    """units/s of the oracle on `procs` host processes, each running its own instance."""
    import multiprocessing as mp
    if procs == 1:
        dt, units = _cpu_worker((w.name, size, 2))
        return units / dt, dt
    with mp.get_context("spawn").Pool(procs) as pool:
        pool.map(_cpu_import, range(procs))       # interpreter start-up stays outside the timing
        t0 = time.perf_counter()
        out = pool.map(_cpu_worker, [(w.name, size, 2 + i) for i in range(procs)])
        dt = time.perf_counter() - t0
    return sum(u for _, u in out) / dt, dt


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    procs = max(1, min(os.cpu_count() or 1, 32))
    size = w.cpu_small
    res = []
    for i in range(args.warmup + args.steps):
        v, dt = cpu_sample(w, procs, size)
        if i >= args.warmup:
            res.append((v, dt))
    value = float(np.mean([v for v, _ in res]))
    sample = (f"{procs} processes, each the same KTIR kernel at size {size} "
              f"(oracle/numpy_interp.py, NumPy {np.__version__})")
    line = {"impl": "reference", "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean([dt for _, dt in res])) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
            "data": "synthetic", "config": workload_config(w, args.gpus),
            "cpu_baseline": {"value": value, "unit": w.unit, "cores": procs, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------
def run_gpu(args, w):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from ktir_cpu_b200.interpreter import KTIRInterpreter
    from ktir_cpu_b200.pinned import pinned_empty

    interp = KTIRInterpreter(device=local)
    interp.load(w.source())
    dev = interp.device
    kw = {}
    for k, v in w.inputs(rank).items():
        if isinstance(v, np.ndarray):
            p = pinned_empty(dev, v.shape, v.dtype)
            p[...] = v
            kw[k] = p
        else:
            kw[k] = v
    sess, _ = interp.session(w.func, **kw)
    for k, v in kw.items():
        if isinstance(v, np.ndarray):
            sess.upload(k, v)
    dev.sync()

    def barrier():
        if dist is not None:
            dist.barrier()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        sess.run()
    dev.sync()
    if hasattr(w, "reset"):
        w.reset(sess, kw)
        dev.sync()

    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    dev.sync()
    l0 = dev.launch_count()
    per_step = []
    for _ in range(args.steps):
        dev.flush_l2()
        dev.record(0)
        sess.run()
        dev.record(1)
        dev.sync()
        per_step.append(dev.elapsed_ms(0, 1))
    launches = dev.launch_count() - l0
    dev.sync()
    # a timed region shorter than the sampling period: keep the same load running (untimed) until
    # the sampler has seen it a few times
    t_extra = time.time()
    while sampler.proc is not None and sampler.under_load() < 4 and time.time() - t_extra < 3.0:
        sess.run()
        dev.sync()
    barrier()
    clocks = sampler.stop()
    total_ms = float(sum(per_step))

    # end to end through the public API: host (pinned) buffers in, fresh host arrays out, every step
    for _ in range(2):
        interp.execute_function(w.func, **kw)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        res = interp.execute_function(w.func, **kw)
    e2e_s = time.perf_counter() - t0
    h2d, d2h = int(sess.last_h2d_bytes), int(sess.last_d2h_bytes)
    err = w.check(kw, res) if not hasattr(w, "reset") else None

    if dist is not None:
        import torch
        t = torch.tensor([total_ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_s = float(t[0]), float(t[1])
    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = world * w.units_per_step / (ms_per_step * 1e-3)
        peak, punit, peak_src = measured_peak(w.bound)
        achieved = w.algo_per_step / (ms_per_step * 1e-3) / (1e9 if w.bound == "hbm" else 1e12)
        traffic = None
        tp = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tp):
            t = json.load(open(tp)).get(w.name)
            if t:        # DRAM bytes of one launch of the dominant kernel, from the ncu capture summarised in profiles/
                traffic = t["dram_read_bytes"] + t["dram_write_bytes"]
        line = {"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": world, "steps": args.steps,
                "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": w.dtype, "data": "synthetic", "config": workload_config(w, world),
                "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": punit,
                             "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                             "algorithmic_per_launch": w.algo_per_step, "kernel": w.kernel},
                "e2e": {"value": world * w.units_per_step * args.steps / e2e_s, "unit": w.unit,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s / args.steps * 1e3},
                "gpu_launches": int(launches), "clocks": clocks, "max_abs_err_spot_check": err}
        if world == 1 and not args.no_cpu:
            v, dt = cpu_sample(w, 1, w.cpu_small)
            line["cpu_baseline"] = {"value": v, "unit": w.unit, "cores": 1, "kind": "port",
                                    "sample": f"same KTIR kernel at size {w.cpu_small} through "
                                              f"oracle/numpy_interp.py on 1 core, {dt:.2f} s"}
        print(json.dumps(line))
    interp.close()
    if dist is not None:
        dist.destroy_process_group()


def run_sharded(args, w):
    """Strong scaling: ONE instance of the workload split over the ranks (core ranges, or
    destination-row ownership for the ordered scatter), each step = this rank's launches + the
    exchange of the written slabs over NCCL, so every rank ends with the full result."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ktir_cpu_b200.interpreter import KTIRInterpreter
    from ktir_cpu_b200.sharded import ShardedRun
    interp = KTIRInterpreter(device=local)
    interp.load(w.source())
    kw = w.inputs(0)                                   # the same instance on every rank
    run = ShardedRun(interp, w.func, rank, world, dist, **kw)
    dev = interp.device
    arrays = {k: v for k, v in kw.items() if isinstance(v, np.ndarray)}
    run.upload(**arrays)

    def barrier():
        if world > 1:
            dist.barrier()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        if hasattr(w, "reset"):
            run.upload(**arrays)
        run.step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms = 0.0
    l0 = dev.launch_count()
    for _ in range(args.steps):
        if hasattr(w, "reset"):
            run.upload(**arrays)
        dev.flush_l2()
        torch.cuda.synchronize()
        barrier()
        ev0.record()
        run.step()
        ev1.record()
        torch.cuda.synchronize()
        total_ms += ev0.elapsed_time(ev1)
    launches = dev.launch_count() - l0
    for _ in range(200 if sampler.proc is not None else 0):   # same load, untimed, until the sampler has seen it
        run.step()
        torch.cuda.synchronize()
        if world == 1 and sampler.under_load() >= 4:
            break
    barrier()
    clocks = sampler.stop()
    res = {k: run.download(k) for k in arrays}
    err = w.check(kw, res) if not hasattr(w, "reset") else None
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    if rank == 0:
        ms = total_ms / args.steps
        slabs = sum(hi - lo for lo, hi in run.my_ranges)
        cfg = workload_config(w, 1)
        cfg["sharding"] = (f"one instance split over {world} GPUs "
                           f"({'destination-row ownership' if w.name == 'gather_scatter' else 'core ranges'}); "
                           f"inputs replicated; per step each rank broadcasts its {slabs} B of results (NCCL)")
        print(json.dumps({"metric": w.metric + " [one instance, sharded]", "value": w.units_per_step / (ms * 1e-3),
                          "unit": w.unit, "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w.dtype,
                          "data": "synthetic", "config": cfg, "gpu_launches": int(launches), "clocks": clocks,
                          "max_abs_err_spot_check": err}))
    run.close()
    interp.close()
    if world > 1:
        dist.destroy_process_group()


def candidate_sweep(n=512, B=1, H=4, D=128):
    """The 512-variant attention sweep: variant i has tile_m = (32,64,128)[i%3],
    tile_n = (32,64,128)[(i//3)%3], S = (512,1024,2048)[(i//9)%3], inputs seeded 1000+i.
    B and H are not fixed by the configuration; B=1, H=4 keeps the CPU interpreter able to finish a sample."""
    from ktir_cpu_b200 import kernels as K
    from ktir_cpu_b200.batch import Candidate
    out, flops = [], 0
    for i in range(n):
        tm, tn, S = (32, 64, 128)[i % 3], (32, 64, 128)[(i // 3) % 3], (512, 1024, 2048)[(i // 9) % 3]
        rng = np.random.default_rng(1000 + i)
        q, k, v = (rng.standard_normal((S, B * H, D), dtype=np.float32).astype(np.float16) for _ in range(3))
        kw = dict(output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=k.reshape(S // tn, tn, B * H, D),
                  value_cache_ptr=v.reshape(S // tn, tn, B * H, D),
                  block_tables_ptr=np.arange(S // tn, dtype=np.int32).reshape(1, -1),
                  num_tiles=S // tn, context_len=0, scale=float(1.0 / np.sqrt(D)))
        out.append(Candidate(K.causal_attention(S, B * H, D, tm, tn), "attention_kernel", kw, tag=(tm, tn, S)))
        flops += 4 * B * H * D * (S * (S + 1) // 2)
    return out, flops


def run_candidates(args):
    """kernels/s over the candidate sweep, host arrays in and out for every candidate (there is
    no device-resident variant of this metric: a candidate arrives as text + host tensors)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ktir_cpu_b200.batch import BatchRunner
    n = 512
    cands, flops = candidate_sweep(n)
    runner = BatchRunner(local)
    checks = {}

    def score(i, c, out):
        if i % 9 == rank % 9:                  # spot-check one head of a few variants against f64 math (warm-up pass only)
            S, h = c.tag[2], 1
            q = c.kwargs["query_ptr"][:, h].astype(np.float64)
            k = c.kwargs["key_cache_ptr"][:, :, h].reshape(S, -1).astype(np.float64)
            v = c.kwargs["value_cache_ptr"][:, :, h].reshape(S, -1).astype(np.float64)
            sc = np.where(np.tril(np.ones((S, S), bool)), q @ k.T / np.sqrt(q.shape[1]), -np.inf)
            p = np.exp(sc - sc.max(-1, keepdims=True))
            checks[i] = float(np.abs(out["output_ptr"][:, h].astype(np.float64) - (p / p.sum(-1, keepdims=True)) @ v).max())
        return True
    warm = runner.run(cands[:27 * world], rank, world, score=score, keep_outputs=False)  # every distinct kernel planned once
    res = runner.run(cands, rank, world, score=None, keep_outputs=True)   # one untimed sweep: the pinned result buffers exist
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    steps = max(1, args.steps // 10)
    launches = 0
    for _ in range(steps):
        res = None                            # the consumer is done with the previous sweep's results: their buffers are reused
        res = runner.run(cands, rank, world, score=None, keep_outputs=True)
        launches += res.launches
    dt = time.perf_counter() - t0
    clocks = sampler.stop()
    errs = len(res.errors) + len(warm.errors)
    if dist is not None:
        import torch
        t = torch.tensor([dt, float(errs)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt, errs = float(t[0]), int(t[1])
    if rank == 0:
        h2d = sum(v.nbytes for c in cands for v in c.kwargs.values() if isinstance(v, np.ndarray)) // n
        line = {"metric": "candidate kernels evaluated per second (512-variant causal attention sweep)",
                "value": n * steps / dt, "unit": "kernels/s", "n_gpus": world, "steps": steps, "warmup": 2,
                "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": "512 variants: tile_m,tile_n in {32,64,128}, S in {512,1024,2048}, B=1, H=4, D=128; "
                                       "variant i on rank i % world; 27 distinct kernels parsed and planned once",
                           "flops_per_sweep": flops},
                "e2e": {"value": n * steps / dt, "unit": "kernels/s", "h2d_bytes_per_step": h2d * n,
                        "d2h_bytes_per_step": h2d * n},
                "tflops": flops * steps / dt / 1e12, "gpu_launches": int(launches), "clocks": clocks,
                "failed_candidates": errs, "max_abs_err_spot_check": max(checks.values()) if checks else None}
        if world == 1 and not args.no_cpu:
            sys.path.insert(0, ROOT)
            from oracle.numpy_interp import OracleInterpreter
            t1 = time.perf_counter()
            c = cands[0]                          # smallest variant: tile 32x32, S = 512
            o = OracleInterpreter()
            o.load(c.source)
            o.execute_function(c.function, **c.kwargs)
            d1 = time.perf_counter() - t1
            line["cpu_baseline"] = {"value": 1.0 / d1, "unit": "kernels/s", "cores": 1, "kind": "port",
                                    "sample": f"variant 0 (tile 32x32, S=512, the cheapest) through oracle/numpy_interp.py on 1 core, {d1:.1f} s"}
        print(json.dumps(line))
    runner.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="softmax", choices=sorted(WORKLOADS) + ["candidates"])
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--shard", action="store_true",
                    help="split ONE instance of the workload over the ranks (strong scaling) instead of one replica per rank")
    args = ap.parse_args()
    if args.workload == "candidates":
        return run_candidates(args)
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    elif args.shard:
        run_sharded(args, w)
    else:
        run_gpu(args, w)


if __name__ == "__main__":
    main()

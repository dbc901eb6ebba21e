"""Benchmark: KTIR execution throughput on the row-softmax workload (8192 x 4096 f16, f32 stats).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass of the hot path over the whole workload: the launch plan
of ``softmax_kernel`` (32 KTIR cores x 256 rows each) on tensors resident in
HBM.  Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU
restatement of the reference interpreter (oracle/) on the host cores instead.
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

N_ROWS, N_COLS, CORES, ROWS_PER_ITER = 8192, 4096, 32, 8
ELEMS = N_ROWS * N_COLS
ALGO_BYTES = 2 * ELEMS * 2          # read f16 once + write f16 once
METRIC = "KTIR exec throughput (row softmax 8192x4096 f16, f32 stats)"
UNIT = "elem/s"


def workload_config(n_gpus):
    return {"workload": "row_softmax f16[8192,4096], grid 32 cores x 256 rows, 8 rows/iteration, f32 stats",
            "elements_per_step_per_gpu": ELEMS, "sharding": f"replica per GPU x{n_gpus} (independent shards)",
            "l2": "flushed (256 MiB memset) between timed steps; step timed by CUDA events on the launch stream"}


def make_input(seed=2):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((N_ROWS, N_COLS), dtype=np.float32) * 2).astype(np.float16)


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback"


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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
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
    rows, seed = args
    from ktir_cpu_b200 import kernels as K
    from oracle.numpy_interp import OracleInterpreter
    cores = max(1, min(CORES, rows // ROWS_PER_ITER))
    while rows % (cores * ROWS_PER_ITER):
        cores -= 1
    x = (np.random.default_rng(seed).standard_normal((rows, N_COLS), dtype=np.float32) * 2).astype(np.float16)
    it = OracleInterpreter()
    it.load(K.softmax_rows(rows, N_COLS, cores, ROWS_PER_ITER, True))
    t0 = time.perf_counter()
    it.execute_function("softmax_kernel", output_ptr=np.zeros_like(x), input_ptr=x)
    return time.perf_counter() - t0


def cpu_sample(procs: int, rows_per_proc: int):
    """elements/s of the oracle on `procs` host processes, each on its own shard of rows."""
    import multiprocessing as mp
    if procs == 1:
        dt = _cpu_worker((rows_per_proc, 2))
    else:
        with mp.get_context("spawn").Pool(procs) as pool:
            t0 = time.perf_counter()
            pool.map(_cpu_worker, [(rows_per_proc, 2 + i) for i in range(procs)])
            dt = time.perf_counter() - t0
    return procs * rows_per_proc * N_COLS / dt, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    procs = max(1, min(os.cpu_count() or 1, 32))
    rows_per_proc = max(ROWS_PER_ITER * 8, (N_ROWS // procs) // ROWS_PER_ITER * ROWS_PER_ITER)
    times = []
    for i in range(args.warmup + args.steps):
        v, dt = cpu_sample(procs, rows_per_proc)
        if i >= args.warmup:
            times.append((v, dt))
    value = float(np.mean([v for v, _ in times]))
    sample = (f"{procs} processes x {rows_per_proc} rows x {N_COLS} cols per step "
              f"(oracle/numpy_interp.py, NumPy {np.__version__})")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": float(np.mean([dt for _, dt in times])) * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": procs, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------
def run_gpu(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from ktir_cpu_b200 import kernels as K
    from ktir_cpu_b200.interpreter import KTIRInterpreter
    from ktir_cpu_b200.pinned import pinned_empty

    interp = KTIRInterpreter(device=local)
    interp.load(K.softmax_rows(N_ROWS, N_COLS, CORES, ROWS_PER_ITER, True))
    dev = interp.device
    x = pinned_empty(dev, (N_ROWS, N_COLS), np.float16)
    x[...] = make_input(2 + rank)
    out0 = pinned_empty(dev, (N_ROWS, N_COLS), np.float16)
    out0[...] = 0
    sess, _ = interp.session("softmax_kernel", output_ptr=out0, input_ptr=x)
    sess.upload("input_ptr", x)
    sess.upload("output_ptr", out0)
    dev.sync()

    def barrier():
        if dist is not None:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        sess.run()
    dev.sync()

    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    dev.sync()
    l0 = dev.launch_count()
    per_step = []
    for i in range(args.steps):
        dev.flush_l2()
        dev.record(0)
        sess.run()
        dev.record(1)
        dev.sync()
        per_step.append(dev.elapsed_ms(0, 1))
    launches = dev.launch_count() - l0
    dev.sync()
    barrier()
    clocks = sampler.stop()
    total_ms = float(sum(per_step))

    # end to end through the public API: host (pinned) buffers in, host arrays out, every step
    for _ in range(2):
        interp.execute_function("softmax_kernel", output_ptr=out0, input_ptr=x)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        res = interp.execute_function("softmax_kernel", output_ptr=out0, input_ptr=x)
    e2e_s = time.perf_counter() - t0
    h2d = int(sess.last_h2d_bytes)
    d2h = int(sess.last_d2h_bytes)

    # spot check of the timed result against a float32 softmax of the same rows
    y = res["output_ptr"]
    rows = np.arange(0, N_ROWS, 257)
    xf = np.asarray(x[rows], dtype=np.float32)
    e = np.exp(xf - xf.max(1, keepdims=True))
    err = float(np.abs(y[rows].astype(np.float32) - e / e.sum(1, keepdims=True)).max())

    if dist is not None:
        import torch
        t = torch.tensor([total_ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_s = float(t[0]), float(t[1])
    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = world * ELEMS / (ms_per_step * 1e-3)
        peak, peak_src = measured_peak_gbs()
        achieved = ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
        traffic = None
        tp = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tp):
            traffic = json.load(open(tp)).get("row_softmax_8192x4096_dram_bytes_per_launch")
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(world),
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": ALGO_BYTES, "kernel": "ktb_row_softmax_kernel"},
                "e2e": {"value": world * ELEMS * args.steps / e2e_s, "unit": UNIT,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_s / args.steps * 1e3},
                "gpu_launches": int(launches), "clocks": clocks, "max_abs_err_vs_f32_softmax": err}
        if world == 1 and not args.no_cpu:
            procs = 1
            rows = 1024
            v, dt = cpu_sample(procs, rows)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": procs, "kind": "port",
                                    "sample": f"{rows} rows x {N_COLS} cols of the same kernel, "
                                              f"oracle/numpy_interp.py on 1 core, {dt:.2f} s"}
        print(json.dumps(line))
    interp.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

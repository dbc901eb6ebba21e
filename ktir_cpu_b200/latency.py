"""Analytical latency / roofline model of the modelled accelerator (host side).

Same public surface as the reference's model (ktir_cpu/latency.py:41-846):
``HardwareConfig``, ``ExecutionModel``, ``LatencyCategory``, ``CoreLatencyCounters``,
``LatencyTracker`` and ``LatencyReport`` with ``kernel_cycles``, ``kernel_time_us``,
``bottleneck``, ``per_core_summary()``, ``chip_roofline()``, ``core_roofline()``,
``roofline()``, ``summary_dict()`` and ``counters[core_id]``.

The reference charges every op as it is dispatched on every core
(ktir_cpu/interpreter.py:268-279).  Here nothing is dispatched op by op: the
whole-grid tracer visits each op once and knows how many times each core would have
executed it, so the tracker is fed *weighted* records — (op, per-core execution
count, cost of one execution) — and the per-core counters are the weighted sums.
The cost rules themselves are the reference's (ktir_cpu/latency.py:311-393):

* ``zero``      metadata ops, casts, views, control flow: nothing;
* ``memory``    ``ktdp.load`` / ``ktdp.store``: bytes = distinct 128-byte sticks touched x 128,
                cycles = bytes / (chip HBM bytes per cycle / active cores);
* ``compute_matmul``  2*M*N*K flops at ``2 * simd_elements_per_cycle * systolic_rows`` per cycle;
* ``compute_float`` / ``compute_int``  one element per SIMD lane per cycle (scalar index
                arithmetic is free);
* ``compute_transcendental``  the same times ``transcendental_penalty``;
* ``comm``      ring bytes / ring bytes per cycle.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np

STICK_BYTES = 128


class LatencyCategory(str):
    """String constants naming the cost classes (ktir_cpu/latency.py:41-49)."""
    ZERO = "zero"
    MEMORY = "memory"
    COMPUTE_FLOAT = "compute_float"
    COMPUTE_TRANSCENDENTAL = "compute_transcendental"
    COMPUTE_INT = "compute_int"
    COMPUTE_MATMUL = "compute_matmul"
    COMM = "comm"


_FLOAT_OPS = ("arith.absf arith.addf arith.cmpf arith.divf arith.maxf arith.maximumf arith.maxnumf arith.minf "
              "arith.minimumf arith.minnumf arith.mulf arith.negf arith.remf arith.select arith.subf linalg.add "
              "linalg.generic linalg.max math.absf math.absi math.ceil math.floor math.fma").split()
_INT_OPS = ("arith.addi arith.andi arith.ceildivsi arith.ceildivui arith.cmpi arith.divsi arith.divui "
            "arith.floordivsi arith.maxsi arith.maxui arith.minsi arith.minui arith.muli arith.ori arith.remsi "
            "arith.remui arith.shli arith.shrsi arith.shrui arith.subi arith.xori").split()
_TRANS_OPS = ("math.cos math.erf math.exp math.log math.log1p math.log2 math.powf math.rsqrt math.sin math.sqrt "
              "math.tanh").split()

CATEGORY_OF: Dict[str, str] = {}
CATEGORY_OF.update({n: LatencyCategory.COMPUTE_FLOAT for n in _FLOAT_OPS})
CATEGORY_OF.update({n: LatencyCategory.COMPUTE_INT for n in _INT_OPS})
CATEGORY_OF.update({n: LatencyCategory.COMPUTE_TRANSCENDENTAL for n in _TRANS_OPS})
CATEGORY_OF.update({"ktdp.load": LatencyCategory.MEMORY, "ktdp.store": LatencyCategory.MEMORY,
                    "linalg.matmul": LatencyCategory.COMPUTE_MATMUL,
                    "linalg.batch_matmul": LatencyCategory.COMPUTE_MATMUL,
                    "ktdp.inter_tile_reduce": LatencyCategory.COMM})


def get_latency_category(op_type: str) -> str:
    """Cost class of an op; anything not listed is free (ktir_cpu/dialects/registry.py)."""
    return CATEGORY_OF.get(op_type, LatencyCategory.ZERO)


@dataclass
class ExecutionModel:
    """How compute, memory and communication time combine (ktir_cpu/latency.py:57-102)."""
    unit_categories: Dict[str, set] = field(default_factory=lambda: {
        "systolic": {"compute_matmul"},
        "simd": {"compute_float", "compute_transcendental", "compute_int"},
    })
    pipeline: str = "serial"          # serial | overlapped | overlapped_3way
    bw_sharing: str = "contended"
    fallback_unit: str = "simd"

    def __post_init__(self):
        if self.bw_sharing == "static":
            raise NotImplementedError("bw_sharing='static' (fixed per-core partition) is reserved "
                                      "and not yet implemented; only 'contended' is available.")
        if self.bw_sharing != "contended":
            raise ValueError(f"bw_sharing must be 'contended' (got {self.bw_sharing!r})")


@dataclass
class HardwareConfig:
    """Parameters of the modelled chip (ktir_cpu/latency.py:105-185); defaults as in the reference."""
    num_cores: int = 32
    clock_ghz: float = 1.0
    hbm_bandwidth_tb_s: float = 0.128
    ring_bandwidth_tb_s: float = 0.064
    simd_elements_per_cycle: int = 64
    systolic_rows: int = 8
    transcendental_penalty: int = 4
    lx_size_mb: int = 2

    @property
    def clock_hz(self) -> float:
        return self.clock_ghz * 1e9

    @property
    def hbm_bw_chip(self) -> float:
        return self.hbm_bandwidth_tb_s * 1e12

    @property
    def systolic_flops_per_cycle(self) -> int:
        return 2 * self.simd_elements_per_cycle * self.systolic_rows

    @property
    def systolic_peak(self) -> float:
        return self.systolic_flops_per_cycle * self.clock_hz

    @property
    def simd_peak(self) -> float:
        return self.simd_elements_per_cycle * self.clock_hz

    def lx_bytes_per_cycle(self) -> float:
        return self.ring_bandwidth_tb_s * 1e12 / (self.clock_ghz * 1e9)

    def lx_bytes_per_cycle_per_core(self) -> float:
        return self.lx_bytes_per_cycle()

    @property
    def ring_bytes_per_cycle(self) -> float:
        return self.ring_bandwidth_tb_s * 1e12 / self.clock_hz


@dataclass
class _TraceEntry:
    """One charged op; ``count`` is how many times this core executed it."""
    op_type: str
    cycles: float
    category: str
    count: int = 1


@dataclass
class CoreLatencyCounters:
    """Cycle / flop / byte totals of one core (ktir_cpu/latency.py:195-264)."""
    memory_cycles: float = 0.0
    comm_cycles: float = 0.0
    flops_by_category: Dict[str, float] = field(default_factory=dict)
    cycles_by_category: Dict[str, float] = field(default_factory=dict)
    bytes_by_category: Dict[str, int] = field(default_factory=dict)
    trace: Optional[List[_TraceEntry]] = None

    @property
    def compute_cycles(self) -> float:
        return sum(self.cycles_by_category.values())

    @property
    def total_cycles(self) -> float:
        return self.compute_cycles + self.memory_cycles + self.comm_cycles

    @property
    def total_flops(self) -> float:
        return sum(self.flops_by_category.values())

    @property
    def total_bytes(self) -> int:
        return sum(self.bytes_by_category.values())

    @property
    def comm_bytes(self) -> int:
        return self.bytes_by_category.get("comm", 0)

    @property
    def dram_bytes(self) -> int:
        return self.bytes_by_category.get("memory", 0)

    def record(self, category: str, cycles: float, op_type: str = "", flops: float = 0.0, nbytes: int = 0,
               count: int = 1):
        """Add ``count`` executions of an op whose totals over those executions are given."""
        if category.startswith("compute_"):
            self.cycles_by_category[category] = self.cycles_by_category.get(category, 0.0) + cycles
            self.flops_by_category[category] = self.flops_by_category.get(category, 0.0) + flops
        elif category == "memory":
            self.memory_cycles += cycles
        elif category == "comm":
            self.comm_cycles += cycles
        if nbytes:
            self.bytes_by_category[category] = self.bytes_by_category.get(category, 0) + int(nbytes)
        if self.trace is not None:
            self.trace.append(_TraceEntry(op_type, cycles, category, count))


# ---------------------------------------------------------------------------
# Weighted op records produced by the tracer
# ---------------------------------------------------------------------------

@dataclass
class OpRecord:
    """One traced op: how often each core executes it and what one execution costs.

    ``kind`` selects the cost rule: ``elems`` (n_elems), ``matmul`` (m, n, k), ``bytes``
    (per-core byte totals already summed over the executions) or ``indirect`` (bytes that
    depend on index *values*; ``resolve(tensors)`` yields the per-core byte totals).
    """
    op_type: str
    category: str
    count: np.ndarray                      # [n_cores] executions per core
    kind: str = "zero"
    n_elems: int = 0
    mnk: tuple = (1, 1, 1)
    nbytes: Optional[np.ndarray] = None    # [n_cores]
    resolve: Any = None


class LatencyTracker:
    """Accumulates per-core cost from weighted op records (ktir_cpu/latency.py:267-308)."""

    def __init__(self, config: HardwareConfig, trace: bool = False):
        self.config = config
        self._trace = trace
        self.counters: Dict[int, CoreLatencyCounters] = {}
        self._cores_active: int = config.num_cores

    def set_cores_active(self, cores_active: int):
        self._cores_active = cores_active

    def reset(self):
        self.counters.clear()

    def _core(self, core_id: int) -> CoreLatencyCounters:
        c = self.counters.get(core_id)
        if c is None:
            c = self.counters[core_id] = CoreLatencyCounters(trace=[] if self._trace else None)
        return c

    def record_weighted(self, core_id: int, op_type: str, category: str, count: int, cycles_each: float,
                        flops_each: float, nbytes_total: int = 0, cycles_total: Optional[float] = None):
        cyc = cycles_each * count if cycles_total is None else cycles_total
        self._core(core_id).record(category, cyc, op_type, flops=flops_each * count, nbytes=nbytes_total,
                                   count=int(count))

    def feed(self, records: List[OpRecord], tensors: Optional[Dict[str, np.ndarray]] = None):
        """Charge every record to the cores that execute it."""
        cfg = self.config
        hbm_bw = cfg.hbm_bw_chip / cfg.clock_hz / self._cores_active     # bytes per cycle per core
        for r in records:
            cores = np.nonzero(r.count)[0]
            if r.kind == "zero":
                for c in cores:
                    self._core(int(c))
                continue
            if r.kind == "elems":
                n = r.n_elems
                if r.category == LatencyCategory.COMPUTE_INT and n <= 1:
                    each, fl = 0.0, 0.0          # scalar index arithmetic is resolved at compile time
                else:
                    each = n / cfg.simd_elements_per_cycle
                    if r.category == LatencyCategory.COMPUTE_TRANSCENDENTAL:
                        each *= cfg.transcendental_penalty
                    fl = float(n)
                for c in cores:
                    self.record_weighted(int(c), r.op_type, r.category, int(r.count[c]), each, fl)
            elif r.kind == "matmul":
                m, n, k = r.mnk
                fl = 2.0 * m * n * k
                each = fl / cfg.systolic_flops_per_cycle
                for c in cores:
                    self.record_weighted(int(c), r.op_type, r.category, int(r.count[c]), each, fl)
            elif r.kind == "comm":
                # bytes each core sends over the ring (ktir_cpu/latency.py:380-390)
                bw = cfg.ring_bytes_per_cycle
                for c in cores:
                    b = int(r.nbytes[c])
                    self.record_weighted(int(c), r.op_type, "comm", int(r.count[c]), 0.0, 0.0, b,
                                         cycles_total=(b / bw if bw > 0 else 0.0))
            elif r.kind in ("bytes", "indirect"):
                nb = r.nbytes if r.kind == "bytes" else r.resolve(tensors or {})
                for c in cores:
                    b = int(nb[c])
                    self.record_weighted(int(c), r.op_type, "memory", int(r.count[c]), 0.0, 0.0, b,
                                         cycles_total=(b / hbm_bw if hbm_bw > 0 else 0.0))
            else:
                raise NotImplementedError(f"Unknown category {r.category}")

    def report(self) -> "LatencyReport":
        return LatencyReport(config=self.config, counters=dict(self.counters))


# ---------------------------------------------------------------------------
# Report
# ---------------------------------------------------------------------------

@dataclass
class LatencyReport:
    """Kernel latency = slowest core; rooflines at chip and core scope (ktir_cpu/latency.py:566-846)."""
    config: HardwareConfig
    counters: Dict[int, CoreLatencyCounters]
    model: ExecutionModel = field(default_factory=ExecutionModel)

    def _effective_cycles(self, core: CoreLatencyCounters) -> float:
        p = self.model.pipeline
        if p == "overlapped":
            return max(core.compute_cycles, core.memory_cycles + core.comm_cycles)
        if p == "overlapped_3way":
            return max(core.compute_cycles, core.memory_cycles, core.comm_cycles)
        return core.compute_cycles + core.memory_cycles + core.comm_cycles

    @property
    def critical_core(self) -> CoreLatencyCounters:
        return max(self.counters.values(), key=self._effective_cycles)

    @property
    def kernel_cycles(self) -> float:
        return self._effective_cycles(self.critical_core) if self.counters else 0.0

    @property
    def kernel_time_us(self) -> float:
        return self.kernel_cycles / (self.config.clock_hz / 1e6)

    @property
    def bottleneck(self) -> str:
        if not self.counters:
            return "none"
        c = self.critical_core
        parts = {"compute": c.compute_cycles, "memory": c.memory_cycles, "comm": c.comm_cycles}
        return max(parts, key=parts.get)

    def per_core_summary(self) -> List[Dict[str, Any]]:
        return [{"core_id": cid, "compute_cycles": c.compute_cycles, "memory_cycles": c.memory_cycles,
                 "comm_cycles": c.comm_cycles, "total_cycles": self._effective_cycles(c)}
                for cid, c in sorted(self.counters.items())]

    @staticmethod
    def _roofline_at(flops: float, nbytes: float, peak_compute: float, peak_bw: float,
                     elapsed_s: float) -> Dict[str, Any]:
        inf = float("inf")
        ai = flops / nbytes if nbytes > 0 else inf
        achieved = flops / elapsed_s if elapsed_s > 0 else 0.0
        ceiling = peak_compute if ai == inf else min(peak_compute, peak_bw * ai)
        return {
            "AI": ai,
            "compute_throughput": achieved / peak_compute if peak_compute > 0 else 0.0,
            "dram_throughput": nbytes / (peak_bw * elapsed_s) if elapsed_s > 0 and peak_bw > 0 else 0.0,
            "achieved_gflops": achieved / 1e9,
            "ceiling_gflops": ceiling / 1e9,
            "attainment": achieved / ceiling if ceiling > 0 else 0.0,
            "ridge": peak_compute / peak_bw if peak_bw > 0 else inf,
            "peak_gflops": peak_compute / 1e9,
        }

    def _dominant_unit(self) -> str:
        chip: Dict[str, float] = {}
        for c in self.counters.values():
            for cat, cyc in c.cycles_by_category.items():
                chip[cat] = chip.get(cat, 0.0) + cyc
        totals = {u: sum(chip.get(cat, 0.0) for cat in cats) for u, cats in self.model.unit_categories.items()}
        return max(totals, key=totals.get) if any(totals.values()) else self.model.fallback_unit

    def _cores_active(self) -> int:
        return sum(1 for c in self.counters.values() if self._effective_cycles(c) > 0)

    def _unit_peaks(self) -> Dict[str, float]:
        return {"systolic": self.config.systolic_peak, "simd": self.config.simd_peak}

    def chip_roofline(self) -> Dict[str, Any]:
        if not self.counters:
            return {}
        dom = self._dominant_unit()
        cats = self.model.unit_categories[dom]
        n = self.config.num_cores
        elapsed_cycles = self.kernel_cycles
        elapsed_s = elapsed_cycles / self.config.clock_hz
        flops = sum(c.flops_by_category.get(cat, 0.0) for c in self.counters.values() for cat in cats)
        dram = sum(c.dram_bytes for c in self.counters.values())
        busy = sum(self._effective_cycles(c) for c in self.counters.values())
        active = self._cores_active()
        rf = self._roofline_at(flops, dram, self._unit_peaks()[dom] * n, self.config.hbm_bw_chip, elapsed_s)
        rf.update({
            "mean_core_active_frac": busy / (n * elapsed_cycles) if n > 0 and elapsed_cycles > 0 else 0.0,
            "grid_coverage": active / n if n > 0 else 0.0,
            "dominant_unit": dom,
            "num_cores": n,
            "cores_active": active,
        })
        return rf

    def core_roofline(self) -> Dict[str, Any]:
        if not self.counters:
            return {}
        dom = self._dominant_unit()
        crit = self.critical_core
        elapsed_s = self.kernel_cycles / self.config.clock_hz
        peak_bw = self.config.hbm_bw_chip / self._cores_active()
        units = {}
        for unit, peak in self._unit_peaks().items():
            fl = sum(crit.flops_by_category.get(cat, 0.0) for cat in self.model.unit_categories[unit])
            units[unit] = self._roofline_at(fl, crit.dram_bytes, peak, peak_bw, elapsed_s)
        return {"core_AI": units[dom]["AI"], "core_attainment": units[dom]["attainment"],
                "core_dominant_unit": dom, "peak_bw_gb_s": peak_bw / 1e9, "ridge": units[dom]["ridge"],
                "units": units}

    def roofline(self) -> Dict[str, Any]:
        if not self.counters:
            return {}
        return {**self.core_roofline(), **self.chip_roofline()}

    def summary_dict(self) -> Dict[str, Any]:
        return {"kernel_cycles": self.kernel_cycles, "kernel_time_us": self.kernel_time_us,
                "bottleneck": self.bottleneck, "grid_cores": len(self.counters),
                "num_cores": self.config.num_cores, "per_core": self.per_core_summary()}

    def __str__(self) -> str:
        bar = "=" * 60
        out = [bar, "KTIR Latency Estimation Report", bar,
               f"  Kernel cycles : {self.kernel_cycles:,.1f}",
               f"  Kernel time   : {self.kernel_time_us:.3f} us",
               f"  Bottleneck    : {self.bottleneck}",
               f"  Cores         : {len(self.counters)}", "-" * 60,
               f"  {'Core':>4}  {'Compute':>12}  {'Memory':>12}  {'Comm':>12}  {'Total':>12}", "-" * 60]
        for row in self.per_core_summary():
            out.append(f"  {row['core_id']:>4}  {row['compute_cycles']:>12.1f}  {row['memory_cycles']:>12.1f}  "
                       f"{row['comm_cycles']:>12.1f}  {row['total_cycles']:>12.1f}")
        out.append(bar)
        if self.counters and (self.critical_core.total_flops > 0 or self.critical_core.total_bytes > 0):
            chip, core = self.chip_roofline(), self.core_roofline()

            def ai(v):
                return f"{v:.2f} FLOP/B" if v != float("inf") else "inf (no HBM traffic)"
            out += ["", "Roofline: CHIP-LEVEL  (whole chip as one unit)", "-" * 60,
                    f"  AI                    : {ai(chip['AI'])}",
                    f"  compute_throughput    : {chip['compute_throughput']:.1%}",
                    f"  dram_throughput       : {chip['dram_throughput']:.1%}",
                    f"  attainment            : {chip['attainment']:.1%}",
                    f"  mean_core_active_frac : {chip['mean_core_active_frac']:.1%}",
                    f"  grid_coverage         : {chip['cores_active']}/{chip['num_cores']}  ({chip['grid_coverage']:.1%})",
                    f"  dominant_unit         : {chip['dominant_unit']}",
                    "", "Roofline: PER-CORE  (critical-path core)", "-" * 60,
                    f"  core_AI               : {ai(core['core_AI'])}",
                    f"  core_attainment       : {core['core_attainment']:.1%}",
                    f"  core_dominant_unit    : {core['core_dominant_unit']}",
                    f"  peak_bw (per-core)    : {core['peak_bw_gb_s']:.2f} GB/s", ""]
            for unit, u in core["units"].items():
                mark = " *" if unit == core["core_dominant_unit"] else "  "
                out.append(f"{mark} {unit:>10}  {u['achieved_gflops']:>10.2f} G  {u['ceiling_gflops']:>10.2f} G  "
                           f"{u['ridge']:>8.1f} F/B  {u['attainment']:>6.1%}")
            out.append(bar)
        return "\n".join(out)

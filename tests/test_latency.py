"""Latency model against the reference's reports (tests/golden/latency.json) — host only, no GPU."""
import json
import math
import os

import numpy as np
import pytest

from conftest import golden_names, load_golden
from ktir_cpu_b200 import ExecutionModel, HardwareConfig, KTIRInterpreter, LatencyReport
from ktir_cpu_b200.latency import CoreLatencyCounters, LatencyTracker, OpRecord

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "latency.json")))


def _same(a, b, path=""):
    if isinstance(a, dict):
        assert set(a) == set(b), path
        for k in a:
            _same(a[k], b[k], f"{path}/{k}")
    elif isinstance(a, (list, tuple)):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, f"{path}/{i}")
    elif isinstance(a, float) or isinstance(b, float):
        assert (a == b) or math.isclose(a, b, rel_tol=1e-9), f"{path}: {a} vs {b}"
    else:
        assert a == b, f"{path}: {a} vs {b}"


@pytest.mark.parametrize("name", sorted(GOLD))
def test_report_matches_reference(name):
    assert name in golden_names()
    src, fn, kwargs, _ = load_golden(name)
    interp = KTIRInterpreter(latency_config=HardwareConfig())
    interp.load(src)
    rep = interp.estimate_latency(fn, **kwargs)
    assert isinstance(rep, LatencyReport)
    want = GOLD[name]
    _same(want["summary"], json.loads(json.dumps(rep.summary_dict())), "summary")
    _same(want["roofline"], json.loads(json.dumps(rep.roofline())), "roofline")
    _same(want["flops"], {str(c): dict(v.flops_by_category) for c, v in rep.counters.items()}, "flops")
    _same(want["bytes"], {str(c): dict(v.bytes_by_category) for c, v in rep.counters.items()}, "bytes")
    assert interp.get_latency_report().kernel_cycles == rep.kernel_cycles


def test_no_config_means_no_report():
    src, fn, kwargs, _ = load_golden("vector_add_4096")
    interp = KTIRInterpreter()
    interp.load(src)
    assert interp.get_latency_report() is None
    assert interp.estimate_latency(fn, **kwargs) is None


def test_closed_forms():
    """Memory: bytes / (chip bandwidth / active cores); matmul: 2MNK / (2 * simd * rows)."""
    cfg = HardwareConfig(num_cores=4, hbm_bandwidth_tb_s=0.256, clock_ghz=2.0, simd_elements_per_cycle=32,
                         systolic_rows=4, transcendental_penalty=3)
    tr = LatencyTracker(cfg)
    tr.set_cores_active(2)
    one = np.array([1, 0], np.int64)
    tr.feed([OpRecord("ktdp.load", "memory", one, "bytes", nbytes=np.array([1280, 0])),
             OpRecord("linalg.matmul", "compute_matmul", np.array([2, 1]), "matmul", mnk=(8, 16, 32)),
             OpRecord("math.exp", "compute_transcendental", one, "elems", n_elems=64),
             OpRecord("arith.addi", "compute_int", one, "elems", n_elems=1)])
    rep = tr.report()
    c0, c1 = rep.counters[0], rep.counters[1]
    assert c0.memory_cycles == 1280 / (0.256e12 / 2.0e9 / 2)
    assert c0.cycles_by_category["compute_matmul"] == 2 * (2 * 8 * 16 * 32) / (2 * 32 * 4)
    assert c1.cycles_by_category["compute_matmul"] == (2 * 8 * 16 * 32) / (2 * 32 * 4)
    assert c0.cycles_by_category["compute_transcendental"] == 64 / 32 * 3
    assert c0.cycles_by_category["compute_int"] == 0.0
    assert c0.dram_bytes == 1280 and c1.dram_bytes == 0
    assert rep.kernel_cycles == c0.total_cycles and rep.bottleneck == "compute"


def test_pipeline_models():
    c = CoreLatencyCounters(memory_cycles=10.0, comm_cycles=4.0, cycles_by_category={"compute_float": 12.0})
    cfg = HardwareConfig()
    assert LatencyReport(cfg, {0: c}).kernel_cycles == 26.0
    assert LatencyReport(cfg, {0: c}, ExecutionModel(pipeline="overlapped")).kernel_cycles == 14.0
    assert LatencyReport(cfg, {0: c}, ExecutionModel(pipeline="overlapped_3way")).kernel_cycles == 12.0
    with pytest.raises(NotImplementedError):
        ExecutionModel(bw_sharing="static")
    with pytest.raises(ValueError):
        ExecutionModel(bw_sharing="other")
    assert LatencyReport(cfg, {}).kernel_cycles == 0.0 and LatencyReport(cfg, {}).bottleneck == "none"
    assert "KTIR Latency Estimation Report" in str(LatencyReport(cfg, {0: c}))

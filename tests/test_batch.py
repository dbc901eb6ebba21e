"""Candidate batches: shared parse / plan per kernel text, several candidates in flight, failures
isolated.  The CPU part drives the runner with a device stand-in that accepts every call; the GPU
part checks results bit for bit against one-at-a-time ``execute_function``."""
import ctypes

import numpy as np
import pytest

from ktir_cpu_b200 import kernels as K
from ktir_cpu_b200 import runtime as R
from ktir_cpu_b200.batch import BatchRunner, Candidate, evaluate_many


_OK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p)(lambda ctx, args: 0)


class _AnyCall:
    """Every entry point is a C-callable that returns success."""

    def __getattr__(self, name):
        return _OK


class FakeDevice(R.PlanOnlyDevice):
    """Accepts uploads, launches and events without doing anything; host buffers are NumPy memory."""
    lib = _AnyCall()
    h = 1
    device = index = 0

    def __init__(self):
        self._host = {}
        self.next_ptr = 0
        self.launches = 0
        self.pipeline_calls = []

    def check(self, rc):
        assert rc == 0

    def alloc(self, nbytes):
        self.next_ptr += 1 << 20
        return self.next_ptr

    def alloc_host(self, nbytes):
        buf = np.zeros(max(nbytes, 1), np.uint8)
        self._host[buf.ctypes.data] = buf
        return buf.ctypes.data

    def free_host(self, ptr):
        self._host.pop(ptr, None)

    def launch_count(self):
        return self.launches

    def run_pipeline(self, arena, chunks, n_chunks, pinned, src, n_tensors):
        self.pipeline_calls.append((arena, n_chunks, n_tensors))

    def submit_pipeline(self, arena, chunks, n_chunks, pinned, src, n_tensors, snapshot_ptr, event_slot):
        self.pipeline_calls.append((arena, n_chunks, n_tensors))
        return len(self.pipeline_calls)

    def wait_submitted(self, seq): pass
    def fence(self, a, b): pass
    def lane_d2h(self, *a): pass
    def record_on(self, slot, lane): pass
    def event_sync(self, slot): pass
    def status_snapshot(self, ptr): pass


def _vadd(n, seed):
    rng = np.random.default_rng(seed)
    return dict(x_ptr=rng.standard_normal(n).astype(np.float16), y_ptr=rng.standard_normal(n).astype(np.float16),
                output_ptr=np.zeros(n, np.float16), BLOCK_SIZE=128)


def test_runner_shares_parses_and_plans_and_isolates_bad_candidates(monkeypatch):
    fake = FakeDevice()
    monkeypatch.setattr(R, "get_device", lambda index=0: fake)
    add, soft = K.vector_add(4096, 128, 32), K.softmax_rows(64, 256, 4, 4, True)
    x = np.ones((64, 256), np.float16)
    cands = [Candidate(add, "add_kernel", _vadd(4096, s)) for s in range(3)]
    cands.insert(1, Candidate("module { this is not KTIR", "f", {}))
    cands.insert(3, Candidate(add, "no_such_function", _vadd(4096, 9)))
    cands.append(Candidate(soft, "softmax_kernel", dict(output_ptr=np.zeros_like(x), input_ptr=x)))
    cands.append(Candidate(add, "add_kernel", dict(_vadd(4096, 5), x_ptr=np.zeros(4096, np.int8))))   # unsupported dtype
    runner = BatchRunner(0, depth=2)
    seen = []
    res = runner.run(cands, score=lambda i, c, out: seen.append((i, sorted(out))) or i)
    assert sorted(res.errors) == [1, 3, 6]
    assert "not found" in res.errors[3] and "ValueError" in res.errors[6]
    assert res.outputs == {0: 0, 2: 2, 4: 4, 5: 5}
    assert seen == [(0, ["output_ptr"]), (2, ["output_ptr"]), (4, ["output_ptr"]), (5, ["output_ptr"])]
    assert runner.parses == 2                                   # the unparsable text never became an interpreter
    add_interp = runner._interps[add]
    assert len(add_interp._sessions) == 1                       # three seeds, one plan
    # two flight slots: the add plan ran on two arenas in turn
    assert len({a for a, _, _ in fake.pipeline_calls[:3]}) == 2
    runner.close()


def test_ranks_take_every_world_th_candidate(monkeypatch):
    fake = FakeDevice()
    monkeypatch.setattr(R, "get_device", lambda index=0: fake)
    cands = [Candidate(K.vector_add(4096, 128, 32), "add_kernel", _vadd(4096, s)) for s in range(7)]
    got = [sorted(BatchRunner(0).run(cands, r, 3, score=lambda i, c, o: i).outputs) for r in range(3)]
    assert got == [[0, 3, 6], [1, 4], [2, 5]]


@pytest.mark.gpu
def test_evaluate_many_equals_one_at_a_time(build_lib):
    from ktir_cpu_b200.interpreter import KTIRInterpreter
    rng = np.random.default_rng(0)
    cands = []
    for i in range(12):
        S, tm, tn = (256, 512)[i % 2], (32, 64, 128)[i % 3], (32, 64, 128)[(i // 3) % 3]
        q = rng.standard_normal((S, 4, 128), dtype=np.float32).astype(np.float16)
        nt = S // tn
        kc, vc = (rng.standard_normal((nt, tn, 4, 128), dtype=np.float32).astype(np.float16) for _ in range(2))
        cands.append(Candidate(K.paged_attention(S, S, 4, 4, 128, tn, tm), "paged_attention_kernel", dict(
            output_ptr=np.zeros_like(q), query_ptr=q, key_cache_ptr=kc, value_cache_ptr=vc,
            block_tables_ptr=rng.permutation(nt).astype(np.int32).reshape(1, -1), cur_batch_start_index=0,
            block_table_offset=0, num_tiles=nt, context_len=0, scale=np.float32(0.088))))
    table = rng.standard_normal((512, 128), dtype=np.float32).astype(np.float16)
    idx = rng.integers(0, 512, 4096).astype(np.int32)
    gs = K.gather_scale_scatter(512, 128, 4096, 64, 4)
    good = dict(table_ptr=table, idx_ptr=idx, out_ptr=rng.standard_normal((512, 128), dtype=np.float32).astype(np.float16))
    bad_idx = idx.copy()
    bad_idx[777] = -3
    cands.insert(4, Candidate(gs, "gather_scale_scatter", good))
    cands.insert(7, Candidate(gs, "gather_scale_scatter", dict(good, idx_ptr=bad_idx)))        # fails in the middle
    cands.insert(9, Candidate(gs, "gather_scale_scatter", good))
    res = evaluate_many(cands)
    assert list(res.errors) == [7] and "-3 is negative" in res.errors[7]
    assert sorted(res.outputs) == [i for i in range(len(cands)) if i != 7]
    for i, c in enumerate(cands):
        if i == 7:
            continue
        it = KTIRInterpreter()
        it.load(c.source)
        want = it.execute_function(c.function, **c.kwargs)
        it.close()
        assert set(res.outputs[i]) == {"output_ptr"} or set(res.outputs[i]) == {"out_ptr"}
        for k, v in res.outputs[i].items():
            assert v.tobytes() == want[k].tobytes(), (i, k)

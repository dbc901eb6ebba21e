"""Batches of candidate kernels — the reward-loop use of the interpreter.

The reference evaluates one candidate at a time: parse, run over the grid, compare
(README.md:13-15, notebooks/demo_helpers.py:32-46).  Here a batch is a list of
``Candidate(source, function, kwargs)``; candidates that share their KTIR text share one
parsed module and, when tensor shapes and scalars also agree, one cached launch plan, so a
sweep over seeds costs one parse + plan per distinct kernel.  Several candidates are in flight
at once: while one candidate's kernels run, the next one's tensors are staged into page-locked
memory and uploaded, and the previous one's results come back; each has its own arena, staging
buffers, completion event and status word, so a bad candidate (negative index, unsupported
KTIR) is an entry in ``errors`` and nothing else.  With several GPUs candidate ``i`` belongs
to rank ``i % world`` — nothing is exchanged on the data path; the caller gathers the
per-rank result dictionaries (e.g. ``torch.distributed.all_gather_object``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np

from . import runtime as R
from .interpreter import KTIRInterpreter


@dataclass
class Candidate:
    source: str
    function: str
    kwargs: Dict[str, Any]
    tag: Any = None


@dataclass
class BatchResult:
    outputs: Dict[int, Dict[str, np.ndarray]] = field(default_factory=dict)
    errors: Dict[int, str] = field(default_factory=dict)
    parses: int = 0
    launches: int = 0


class _Flight:
    """One candidate between submission and retirement."""
    __slots__ = ("index", "cand", "out", "slot", "seq", "keep")

    def __init__(self, index, cand, out, slot, seq, keep):
        self.index, self.cand, self.out, self.slot, self.seq, self.keep = index, cand, out, slot, seq, keep


class BatchRunner:
    """Runs candidates on one GPU, keeping one interpreter (parsed module + plans) per KTIR text."""

    EVENT0 = 32          # event slots EVENT0 .. EVENT0 + depth - 1 of the context mark completion

    def __init__(self, device: int = 0, max_kernels: int = 64, latency_config=None, depth: int = 3):
        self.device = device
        self.max_kernels = max_kernels
        self.latency_config = latency_config
        self.depth = max(1, min(depth, 16))
        self._interps: Dict[str, KTIRInterpreter] = {}
        self.parses = 0
        self._pool = None                                   # pinned buffers behind the result arrays
        self._staging: Dict[Any, np.ndarray] = {}           # (flight slot, argument) -> pinned staging buffer
        self._arenas: Dict[int, List[int]] = {}             # id(session) -> one arena per flight slot
        self._sessions: Dict[int, Any] = {}
        self._status: List[np.ndarray] = []                 # per flight slot: pinned copy of the device status word
        self._plans: Dict[int, Any] = {}

    def _interp(self, source: str) -> KTIRInterpreter:
        it = self._interps.get(source)
        if it is None:
            if len(self._interps) >= self.max_kernels:
                old = self._interps.pop(next(iter(self._interps)))
                self._forget(old)
                old.close()
            it = KTIRInterpreter(device=self.device, latency_config=self.latency_config, max_sessions=4)
            it.load(source)
            self._interps[source] = it
            self.parses += 1
        return it

    def _forget(self, it: KTIRInterpreter):
        for sess in list(it._sessions.values()):
            self._release_session(sess)

    def _release_session(self, sess):
        for a in self._arenas.pop(id(sess), [])[1:]:
            sess.dev.free(a)
        for key in [k for k in self._plans if k[0] == id(sess)]:
            del self._plans[key]
        self._sessions.pop(id(sess), None)

    # -- per-session resources ---------------------------------------------------------------
    def _transfer(self, sess, slot: int):
        """Transfer plan of a candidate on the arena of flight slot ``slot``: what the plan reads goes
        up, what it writes comes back; a scorer has the inputs already, so no copies of them are
        made.  A plan of one statement that launches through the C ABI runs as one part that the
        submission thread can issue on its own."""
        b = self._plans.get((id(sess), slot))
        if b is None:
            from .pipeline import BoundPipeline, TransferPlan
            tensors = {k: (off, nbytes) for k, (off, nbytes, _, _) in sess.layout.items()}
            chunks = sess.plan.statements[0].split(1 << 62) if len(sess.plan.statements) == 1 else None
            tp = TransferPlan(tensors, sess.written, sess.no_upload, chunks, None, partial=True)
            b = BoundPipeline(sess.dev, self._arena(sess, slot), tp)
            self._plans[(id(sess), slot)] = b
            self._sessions[id(sess)] = sess
        return b

    def _arena(self, sess, slot: int) -> int:
        arenas = self._arenas.setdefault(id(sess), [sess.arena])
        while len(arenas) <= slot:
            arenas.append(sess.dev.alloc(sess.arena_bytes + 256))
        return arenas[slot]

    def _stage_buffer(self, dev, slot: int, name: str, arr: np.ndarray) -> np.ndarray:
        from .pinned import pinned_empty
        buf = self._staging.get((slot, name))
        if buf is None or buf.nbytes < arr.nbytes:
            buf = pinned_empty(dev, (max(arr.nbytes, 1) * 5 // 4,), np.uint8)
            self._staging[(slot, name)] = buf
        return buf[:arr.nbytes].view(arr.dtype).reshape(arr.shape)

    # -- submission / retirement -----------------------------------------------------------------
    def _submit(self, index: int, c: Candidate, slot: int, res: BatchResult) -> _Flight:
        it = self._interp(c.source)
        sess, kwargs = it.session(c.function, **c.kwargs)
        for gone in [s for s in list(self._sessions.values()) if s.arena is None]:
            self._release_session(gone)                   # evicted from the interpreter's plan cache
        dev = sess.dev
        if self._pool is None:
            from .pinned import PinnedPool
            self._pool = PinnedPool(dev)
        while len(self._status) <= slot:
            from .pinned import pinned_empty
            self._status.append(pinned_empty(dev, (C.sizeof(R.Status),), np.uint8))
        pipe = self._transfer(sess, slot)
        arena = self._arena(sess, slot)
        host, pinned, out = {}, {}, {}
        for k, v in kwargs.items():
            if not isinstance(v, np.ndarray):
                continue
            v = np.ascontiguousarray(v)
            host[k] = v
            if k in sess.written:
                pinned[k] = out[k] = self._pool.empty(v.shape, v.dtype)
                if k not in sess.no_upload:
                    np.copyto(out[k], v)                  # read and written: goes up from (and comes back into) the result array
                    host[k] = out[k]
            elif k in sess.no_upload:
                pinned[k] = v
            else:
                pinned[k] = self._stage_buffer(dev, slot, k, v)
        status_ptr = self._status[slot].ctypes.data
        if pipe.tp.split:
            seq = pipe.submit(dev, arena, host, pinned, status_ptr, self.EVENT0 + slot)
        else:
            dev.wait_submitted(0)              # this plan's launches go out from here: nothing may be pending
            seq = None
            pipe.run(dev, arena, host, pinned, lambda: sess.plan.launch(dev, arena),
                     after_launch=lambda: dev.status_snapshot(status_ptr))
            dev.record_on(self.EVENT0 + slot, 2 if sess.written else 0)
        return _Flight(index, c, out, slot, seq, (host, pinned))

    def _retire(self, f: _Flight, res: BatchResult, score, keep_outputs: bool):
        dev = R.get_device(self.device)
        if f.seq is not None:
            dev.wait_submitted(f.seq)
        dev.event_sync(self.EVENT0 + f.slot)
        f.keep = None
        st = R.Status.from_buffer_copy(self._status[f.slot].tobytes())
        if st.negative_index:
            res.errors[f.index] = f"IndexError: indirect index {st.bad_index_value} is negative"
            return
        if st.wait_timeout:
            res.errors[f.index] = f"DeviceError: a bounded device-side wait ran out (site {st.wait_site})"
            return
        out = f.out
        try:
            if score is not None:
                out = score(f.index, f.cand, out)
            if keep_outputs or score is not None:
                res.outputs[f.index] = out
        except Exception as e:               # noqa: BLE001
            res.errors[f.index] = f"{type(e).__name__}: {e}"

    def run(self, candidates: Sequence[Candidate], rank: int = 0, world: int = 1,
            score: Optional[Callable[[int, Candidate, Dict[str, np.ndarray]], Any]] = None,
            keep_outputs: bool = True) -> BatchResult:
        """Evaluate the candidates this rank owns.  A candidate that fails (unsupported KTIR, bad
        index, ...) is recorded in ``errors`` and does not stop the batch.  ``score`` may reduce each
        result to what the caller keeps (its return value replaces the output dictionary).  Outputs
        hold the tensors the kernel writes."""
        res = BatchResult()
        flights: List[_Flight] = []
        n = 0
        l0 = None
        for i in range(rank, len(candidates), world):
            slot = n % self.depth
            if len(flights) == self.depth:                 # the flight that used this slot before
                self._retire(flights.pop(0), res, score, keep_outputs)
            try:
                if l0 is None and self._interps:
                    l0 = R.get_device(self.device).launch_count()
                flights.append(self._submit(i, candidates[i], slot, res))
                n += 1
            except Exception as e:           # noqa: BLE001 - a bad candidate is a result, not a crash
                res.errors[i] = f"{type(e).__name__}: {e}"
        for f in flights:
            self._retire(f, res, score, keep_outputs)
        if n:
            res.launches = R.get_device(self.device).launch_count() - (l0 or 0)
        res.parses = self.parses
        return res

    def close(self):
        for it in self._interps.values():
            try:
                it.device.sync()
            except Exception:                # noqa: BLE001
                pass
            self._forget(it)
            it.close()
        self._interps.clear()
        self._staging.clear()
        self._status.clear()
        if self._pool is not None:
            self._pool.close()
            self._pool = None


def evaluate_many(candidates: Sequence[Candidate], device: int = 0, rank: int = 0, world: int = 1,
                  **kw) -> BatchResult:
    runner = BatchRunner(device)
    try:
        return runner.run(candidates, rank, world, **kw)
    finally:
        runner.close()

"""Batches of candidate kernels — the reward-loop use of the interpreter.

The reference evaluates one candidate at a time: parse, run over the grid, compare
(README.md:13-15, notebooks/demo_helpers.py:32-46).  Here a batch is a list of
``Candidate(source, function, kwargs)``; candidates that share their KTIR text share one
parsed module and, when tensor shapes and scalars also agree, one cached launch plan, so a
sweep over seeds costs one parse + plan per distinct kernel.  With several GPUs candidate
``i`` belongs to rank ``i % world`` — nothing is exchanged on the data path; the caller
gathers the per-rank result dictionaries (e.g. ``torch.distributed.all_gather_object``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np

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


class BatchRunner:
    """Runs candidates on one GPU, keeping one interpreter (parsed module + plans) per KTIR text."""

    def __init__(self, device: int = 0, max_kernels: int = 64, latency_config=None):
        self.device = device
        self.max_kernels = max_kernels
        self.latency_config = latency_config
        self._interps: Dict[str, KTIRInterpreter] = {}
        self.parses = 0
        self._pool = None                     # pinned buffers behind the result arrays
        self._staging: Dict[int, np.ndarray] = {}     # pinned staging buffers for uploads, one per argument slot

    def _interp(self, source: str) -> KTIRInterpreter:
        it = self._interps.get(source)
        if it is None:
            if len(self._interps) >= self.max_kernels:
                self._interps.pop(next(iter(self._interps))).close()
            it = KTIRInterpreter(device=self.device, latency_config=self.latency_config, max_sessions=4)
            it.load(source)
            self._interps[source] = it
            self.parses += 1
        return it

    def run(self, candidates: Sequence[Candidate], rank: int = 0, world: int = 1,
            score: Optional[Callable[[int, Candidate, Dict[str, np.ndarray]], Any]] = None,
            keep_outputs: bool = True) -> BatchResult:
        """Evaluate the candidates this rank owns.  A candidate that fails (unsupported KTIR, bad
        index, ...) is recorded in ``errors`` and does not stop the batch.  ``score`` may reduce each
        result to what the caller keeps (its return value replaces the output dictionary)."""
        res = BatchResult()
        dev = None
        for i in range(rank, len(candidates), world):
            c = candidates[i]
            try:
                it = self._interp(c.source)
                dev = it.device
                l0 = dev.launch_count()
                out = self._execute(it, c)
                res.launches += dev.launch_count() - l0
                if score is not None:
                    out = score(i, c, out)
                if keep_outputs or score is not None:
                    res.outputs[i] = out
            except Exception as e:           # noqa: BLE001 - a bad candidate is a result, not a crash
                res.errors[i] = f"{type(e).__name__}: {e}"
        res.parses = self.parses
        return res

    def _stage(self, dev, slot: int, arr: np.ndarray) -> np.ndarray:
        """Copy ``arr`` into the pinned staging buffer of argument slot ``slot``: the DMA of one
        tensor then overlaps the host copy of the next.  The buffers are reused by the next
        candidate, which is safe because every candidate ends with a stream synchronisation."""
        from .pinned import pinned_empty
        buf = self._staging.get(slot)
        if buf is None or buf.nbytes < arr.nbytes:
            buf = pinned_empty(dev, (max(arr.nbytes, 1) * 5 // 4,), np.uint8)
            self._staging[slot] = buf
        view = buf[:arr.nbytes].view(arr.dtype).reshape(arr.shape)
        np.copyto(view, arr)
        return view

    def _execute(self, it: KTIRInterpreter, c: Candidate) -> Dict[str, np.ndarray]:
        """Upload, launch, and read back only the tensors the kernel writes (a scorer has the
        inputs already; ``execute_function`` would copy every tensor back).  Host copies go through
        page-locked memory on both sides, so the transfers run asynchronously at PCIe speed."""
        sess, kwargs = it.session(c.function, **c.kwargs)
        if self._pool is None:
            from .pinned import PinnedPool
            self._pool = PinnedPool(sess.dev)
        slot = 0
        for k, v in kwargs.items():
            if isinstance(v, np.ndarray) and k not in sess.no_upload:
                sess.upload(k, self._stage(sess.dev, slot, v) if v.nbytes >= 65536 else v)
                slot += 1
        sess.run()
        out = {k: sess.download(k, pool=self._pool) for k in kwargs if k in sess.written}
        st = sess.dev.sync()
        if st.negative_index:
            raise IndexError(f"indirect index {st.bad_index_value} is negative")
        return out

    def close(self):
        for it in self._interps.values():
            it.close()
        self._interps.clear()
        self._staging.clear()
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

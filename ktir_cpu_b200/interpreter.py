"""``KTIRInterpreter`` — drop-in for the reference class of the same name
(ktir_cpu/interpreter.py:40-194, 312-341), executing on a B200.

``load`` / ``arg_names`` / ``tensor_input_output_sizes`` / ``execute_function``
/ ``get_latency_report`` keep their signatures and error behaviour.  Instead of
interpreting op by op, ``execute_function`` traces the function once for the
whole grid, lowers it to a launch plan (cached per tensor layout and scalar
arguments) and runs the plan through ``libktir_b200``.

Memory layout: one device arena whose byte offset equals the KTIR byte address
(first tensor at 0x10000, each rounded up to a 128-byte stick, as
ktir_cpu/memory.py:330-352 allocates), so SSA pointer values — element indices
— mean the same thing on the device as in the reference.
"""
from __future__ import annotations


from typing import Sequence, Any, Dict, List, Optional, Tuple

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem, to_ktir_dtype
from .ir import IRModule
from .lower import Allocation, ArenaMap, Plan, lower, lower_core_groups
from .parser import KTIRParser, KTIRParserBase
from .trace import CoreOrderHazard, Tracer

STICK = 128
ARENA_BASE = 0x10000


def arena_layout(tensors):
    """name -> (byte offset, nbytes, shape, dtype) and name -> element pointer, in argument order.

    The first tensor sits at 0x10000 and each one starts on a 128-byte stick, like
    HBMSimulator.allocate (ktir_cpu/memory.py:330-352).
    """
    layout, ptrs = {}, {}
    nxt = ARENA_BASE
    for name, shape, dt in tensors:
        dt = np.dtype(dt)
        nbytes = int(np.prod(shape)) * dt.itemsize if len(shape) else dt.itemsize
        layout[name] = (nxt, nbytes, tuple(shape), dt)
        ptrs[name] = nxt // bytes_per_elem(to_ktir_dtype(dt))
        nxt = (nxt + nbytes + STICK - 1) & ~(STICK - 1)
    return layout, ptrs


def layout_of(sess) -> Dict[str, Tuple[int, int, Tuple[int, ...], np.dtype]]:
    return sess.layout


class HostTensors:
    """Read access to the caller's arrays by KTIR element index (for data-dependent accounting)."""

    def __init__(self, layout, kwargs):
        self.spans = [(off, off + nbytes, np.ascontiguousarray(kwargs[name]).reshape(-1))
                      for name, (off, nbytes, _, _) in layout.items() if isinstance(kwargs.get(name), np.ndarray)]

    def read(self, dtype: str, elems: np.ndarray) -> np.ndarray:
        bpe = bytes_per_elem(dtype)
        elems = np.asarray(elems, np.int64)
        if elems.size == 0:
            return np.zeros(0, np.int64)
        first = int(elems.min()) * bpe
        for lo, hi, flat in self.spans:
            if lo <= first < hi:
                rel = elems - lo // bpe
                ok = (rel >= 0) & (rel < flat.size)
                out = np.zeros(elems.shape, np.int64)
                out[ok] = flat[rel[ok]]
                return out
        raise ValueError(f"Read from unmapped address 0x{first:x}")


class Session:
    """One function bound to one tensor layout: the arena in HBM plus its launch plan."""

    PIPELINE_PIECE = 16 << 20        # bytes moved (both directions) per part of a pipelined call

    def __init__(self, dev: R.Device, func, tensors: List[Tuple[str, Tuple[int, ...], np.dtype]],
                 scalars: Dict[str, Any], latency: bool = False, shard: Optional[Tuple[int, int]] = None,
                 arena_ptr: Optional[int] = None, seeded: Sequence[Tuple[int, int, str]] = (), fused: bool = True,
                 lx_bytes: int = 2 << 20):
        """``shard = (rank, world)`` plans only this rank's part of the kernel (see ``sharded.py``);
        ``arena_ptr`` places the arena in caller-owned device memory of at least ``arena_size(tensors)`` bytes;
        ``seeded`` = (byte address, nbytes, dtype) of memory written through ``interp.memory.hbm`` at fixed
        addresses, which becomes part of the arena next to the argument tensors.  ``lx_bytes`` is the
        per-core scratchpad capacity the kernel is checked against while it is traced
        (``MemoryError("LX scratchpad overflow on core ...")``, ktir_cpu/grid.py:292-301)."""
        self.dev = dev
        self.func = func
        self.latency_records = None
        self.shard = shard
        self.own_arena = arena_ptr is None
        self.layout: Dict[str, Tuple[int, int, Tuple[int, ...], np.dtype]] = {}
        nxt = ARENA_BASE
        allocs = []
        ptrs = {}
        for name, shape, dt in tensors:
            nbytes = int(np.prod(shape)) * dt.itemsize if len(shape) else dt.itemsize
            kdt = to_ktir_dtype(dt)
            self.layout[name] = (nxt, nbytes, tuple(shape), dt)
            allocs.append(Allocation(name, nxt, nxt + nbytes, kdt))
            ptrs[name] = nxt // bytes_per_elem(kdt)
            nxt = (nxt + nbytes + STICK - 1) & ~(STICK - 1)
        for addr, nbytes, kdt in seeded:
            allocs.append(Allocation(f"hbm@0x{addr:x}", addr, addr + nbytes, kdt))
            nxt = max(nxt, (addr + nbytes + STICK - 1) & ~(STICK - 1))
        self.arena_bytes = nxt
        self.arena = dev.alloc(self.arena_bytes + 256) if arena_ptr is None else arena_ptr
        self.arena_map = ArenaMap(allocs)
        try:
            from .lx import LXModel, use_counts
            tracer = Tracer(func, scalars, ptrs)
            tracer.arena = self.arena_map
            tracer.lx = LXModel(tracer.ncores, 0, lx_bytes, use_counts(func.ops))
            if latency:
                from .trace_latency import LatencyRecorder
                tracer.latency = LatencyRecorder(tracer.ncores)
            stores = tracer.run()
            self.lx_peak_bytes = int(tracer.lx.peak.max()) if tracer.ncores else 0
            if latency:
                self.latency_records = tracer.latency.records
            self.n_cores = tracer.ncores
            row_shard = None
            if shard is not None and shard[1] > 1:
                from .sharded import core_slice, needs_row_ownership
                if needs_row_ownership(stores):
                    row_shard = shard          # every core runs; each rank applies the rows it owns
                else:
                    # a core of another rank may read or overlap what a core of this rank writes: the
                    # whole grid must pass the sequential-order check, not just this rank's slice
                    lower(R.PlanOnlyDevice(), stores, self.arena_map, fused=fused)
                    part = Tracer(func, scalars, ptrs, core_range=core_slice(tracer.ncores, *shard))
                    part.arena = self.arena_map
                    stores = part.run()
            try:
                self.plan: Plan = lower(dev, stores, self.arena_map, row_shard=row_shard, fused=fused)
            except CoreOrderHazard:
                if shard is not None and shard[1] > 1:
                    raise
                # some core touches bytes another core writes: groups of cores, one after the other

                def trace_cores(lo, hi, unroll):
                    part = Tracer(func, scalars, ptrs, core_range=(lo, hi))
                    part.arena, part.unroll_loops = self.arena_map, unroll
                    return part.run()
                self.plan = lower_core_groups(dev, trace_cores, tracer.ncores, self.arena_map, fused=fused)
        except Exception:
            if self.own_arena:
                dev.free(self.arena)
            self.arena = None
            raise
        self._graph = None
        self._runs = 0
        self.use_graph = arena_ptr is None
        self.written = set(self.plan.written)
        self.no_upload = set(self.plan.fully_overwritten)
        self.last_h2d_bytes = 0
        self.last_d2h_bytes = 0
        self._transfer = None
        self._pipeline = None

    def transfer_plan(self):
        """How a call moves its tensors (``pipeline.TransferPlan``): the plan's statement in
        independent parts when it has one statement that can be split, else as a whole."""
        if self._transfer is None:
            from .pipeline import TransferPlan
            chunks = None
            if len(self.plan.statements) == 1:
                chunks = self.plan.statements[0].split(self.PIPELINE_PIECE)
            tensors = {k: (off, nbytes) for k, (off, nbytes, _, _) in self.layout.items()}
            self._transfer = TransferPlan(tensors, self.written, self.no_upload, chunks, self.plan.written_ranges(),
                                          partial=self.shard is not None and self.shard[1] > 1)
        return self._transfer

    def pipeline(self):
        if self._pipeline is None:
            from .pipeline import BoundPipeline
            self._pipeline = BoundPipeline(self.dev, self.arena, self.transfer_plan())
        return self._pipeline

    def upload(self, name: str, arr: np.ndarray):
        off, nbytes, shape, dt = self.layout[name]
        if nbytes:
            return self.dev.h2d(self.arena + off, arr)
        return arr

    def run(self):
        """Launch the plan.  A plan of several launches is recorded as a CUDA graph on its second run
        and replayed from then on (arguments and the arena address are fixed for a session)."""
        if self._graph is not None:
            self.dev.graph_launch(self._graph)
            return
        self._runs += 1
        n = sum(getattr(s, "launches", 1) for s in self.plan.statements)
        if self._runs == 2 and n > 1 and self.use_graph and hasattr(self.dev, "graph_begin"):
            self.dev.graph_begin()
            try:
                self.plan.launch(self.dev, self.arena)
            finally:
                self._graph = self.dev.graph_end()
            if self._graph is not None:
                self.dev.graph_launch(self._graph)
                return
            self.use_graph = False
        self.plan.launch(self.dev, self.arena)

    def download(self, name: str, out: Optional[np.ndarray] = None, pool=None) -> np.ndarray:
        off, nbytes, shape, dt = self.layout[name]
        if out is None:
            out = pool.empty(shape, dt) if pool is not None else np.empty(shape, dtype=dt)
        if nbytes:
            self.dev.d2h(out, self.arena + off)
        return out

    def device_ptr(self, name: str) -> int:
        return self.arena + self.layout[name][0]

    def written_ranges(self) -> List[Tuple[int, int]]:
        """Merged arena byte ranges this session's launches write (this rank's slabs when sharded)."""
        return self.plan.written_ranges()

    def close(self):
        if self.arena is not None:
            self.dev.sync()
            if self._graph is not None:
                self.dev.graph_destroy(self._graph)
                self._graph = None
            self.plan.release(self.dev)
            if self.own_arena:
                self.dev.free(self.arena)
            self.arena = None


def _scalar_key(v):
    if isinstance(v, (np.floating, float)):
        return ("f", type(v).__name__, float(v))
    if isinstance(v, (bool, np.bool_)):
        return ("b", bool(v))
    if isinstance(v, (int, np.integer)):
        return ("i", int(v))
    return ("o", repr(v))


class _HBMFacade:
    """``interp.memory.hbm`` of the reference, as far as its tests use it: ``write(stick, data)`` before a
    run places data at byte address ``stick * 128`` (ktir_cpu/memory.py:354-398); ``read(stick, n, dtype)``
    afterwards returns what the kernels left there.  The data lives in the arena during the run."""

    def __init__(self):
        self.regions: Dict[int, np.ndarray] = {}         # byte address -> flat array

    def write(self, stick: int, data):
        arr = np.ascontiguousarray(np.asarray(data)).reshape(-1)
        to_ktir_dtype(arr.dtype)
        self.regions[int(stick) * STICK] = arr.copy()

    def read(self, stick: int, n_elements: int, dtype: str) -> np.ndarray:
        from .dtypes import to_np_dtype
        npdt = np.dtype(to_np_dtype(dtype))
        addr = int(stick) * STICK
        for base, arr in self.regions.items():
            end = base + arr.nbytes
            if base <= addr < end:
                raw = arr.view(np.uint8)[addr - base:addr - base + n_elements * npdt.itemsize]
                out = np.zeros(n_elements, npdt)                  # short reads are zero padded
                out.view(np.uint8)[:raw.size] = raw
                return out
        raise ValueError(f"Read from unmapped address 0x{addr:x} (n_elements={n_elements})")


class _MemoryFacade:
    def __init__(self):
        self.hbm = _HBMFacade()


class _GridFacade:
    def __init__(self, n_cores: int):
        self.cores = list(range(n_cores))


class KTIRInterpreter:
    """Executes KTIR functions on a B200 through ``libktir_b200`` (no CPU fallback)."""

    def __init__(self, latency_config=None, trace_latency: bool = False,
                 parser: Optional[KTIRParserBase] = None, device: int = 0, max_sessions: int = 8,
                 fused_kernels: bool = True):
        """The first three arguments are the reference's (ktir_cpu/interpreter.py:46-79).  ``device`` is the
        CUDA device index; ``fused_kernels=False`` runs every statement step by step on the device
        instead of through the fused kernels (slow; a cross-check)."""
        self.module: Optional[IRModule] = None
        self._parser = parser
        self._latency_config = latency_config
        self._trace_latency = trace_latency
        self._device_index = device
        self._fused = fused_kernels
        self._dev: Optional[R.Device] = None
        self._sessions: Dict[Any, Session] = {}
        self._max_sessions = max_sessions
        self._latency_report = None
        self._latency_tracker = None
        if latency_config is not None:
            from .latency import LatencyTracker
            self._latency_tracker = LatencyTracker(latency_config, trace=trace_latency)
        self._pool = None
        self.memory = _MemoryFacade()
        self.grid_executor = _GridFacade(0)

    # -- front end ------------------------------------------------------------
    def load(self, ktir_source: str):
        parser = self._parser if self._parser is not None else KTIRParser()
        if "\n" in ktir_source or ktir_source.lstrip().startswith("module"):
            self.module = parser.parse_module(ktir_source)
        else:
            with open(ktir_source) as f:
                self.module = parser.parse_module(f.read())
        self._drop_sessions()

    def _require_module(self) -> IRModule:
        if not self.module:
            raise RuntimeError("No module loaded. Call load() first.")
        return self.module

    def arg_names(self, func_name: str) -> List[str]:
        return self._require_module().get_function(func_name).arg_names

    def tensor_input_output_sizes(self, func_name: str) -> Dict[str, Dict[str, Any]]:
        return self._require_module().get_function(func_name).tensor_sizes

    def get_latency_report(self):
        """Report of the most recent call, or None without a ``latency_config``
        (ktir_cpu/interpreter.py:337-341)."""
        if self._latency_tracker is None:
            return None
        return self._latency_tracker.report()

    # -- device -----------------------------------------------------------------
    @property
    def device(self) -> R.Device:
        if self._dev is None:
            self._dev = R.get_device(self._device_index)
        return self._dev

    def _drop_sessions(self):
        for s in self._sessions.values():
            s.close()
        self._sessions = {}

    def close(self):
        self._drop_sessions()
        if self._pool is not None:
            self._pool.close()
            self._pool = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def session(self, func_name: str, _shard: Optional[Tuple[int, int]] = None, **kwargs) -> Session:
        """The cached (function, tensor layout, scalar arguments) session for these arguments."""
        func = self._require_module().get_function(func_name)
        declared = func.arg_names
        if kwargs and declared and not any(k in declared for k in kwargs):
            if len(kwargs) == len(declared):
                kwargs = dict(zip(declared, kwargs.values()))
        tensors, scalars = [], {}
        for k, v in kwargs.items():
            if isinstance(v, np.ndarray):
                to_ktir_dtype(v.dtype)           # ValueError for unsupported dtypes
                tensors.append((k, tuple(v.shape), v.dtype))
            else:
                scalars[k] = v
        seeded = tuple((addr, arr.nbytes, to_ktir_dtype(arr.dtype)) for addr, arr in
                       sorted(self.memory.hbm.regions.items()))
        key = (func_name, tuple(tensors),
               tuple((k, _scalar_key(v)) for k, v in scalars.items()), seeded, _shard)
        sess = self._sessions.get(key)
        if sess is None:
            if len(self._sessions) >= self._max_sessions:
                old = next(iter(self._sessions))
                self._sessions.pop(old).close()
            lx_mb = getattr(self._latency_config, "lx_size_mb", 2) if self._latency_config is not None else 2
            sess = Session(self.device, func, tensors, scalars, latency=self._latency_config is not None,
                           seeded=seeded, fused=self._fused, shard=_shard, lx_bytes=int(lx_mb * 1024 * 1024))
            self._sessions[key] = sess
        return sess, kwargs

    def _prepare_execution(self, grid_shape):
        """Fresh memory for a call (ktir_cpu/interpreter.py:95-120).  The reference's tests wrap this
        method to place data at fixed addresses through ``self.memory.hbm.write`` before the run."""
        self.memory = _MemoryFacade()
        n = int(np.prod(grid_shape)) if len(grid_shape) else 1
        self.grid_executor = _GridFacade(n)

    def execute_function(self, func_name: str, **kwargs) -> Dict[str, np.ndarray]:
        """Run ``func_name`` on the device.  As in the reference (ktir_cpu/interpreter.py:122-194)
        every ndarray argument comes back as a new array and the caller's arrays are not touched.

        Calls that move at least 1 MiB run pipelined (``pipeline.py``): the caller's arrays are copied
        once, by host threads, into page-locked result arrays that double as the DMA source; a plan
        whose statement splits into independent parts uploads, computes and reads back part by part
        on three streams."""
        self._prepare_execution(tuple(self._require_module().get_function(func_name).grid))
        sess, kwargs = self.session(func_name, **kwargs)
        if self._pool is None:
            from .pinned import PinnedPool
            self._pool = PinnedPool(self.device)
        arrays = {k: v for k, v in kwargs.items() if isinstance(v, np.ndarray)}
        seeded = self.memory.hbm.regions
        if not seeded and sum(v.nbytes for v in arrays.values()) >= (1 << 20):
            outputs = self._execute_pipelined(sess, arrays)
        else:
            outputs = self._execute_simple(sess, arrays, seeded)
        if self._latency_tracker is not None:
            self._charge_latency(sess.latency_records, sess.n_cores, layout_of(sess), kwargs)
        return outputs

    def execute_shard(self, func_name: str, rank: int, world: int, **kwargs) -> Dict[str, np.ndarray]:
        """This rank's share of one kernel split over ``world`` GPUs (one process per GPU, every rank
        calls with the same arguments): the cores ``[rank*C/world, (rank+1)*C/world)`` of the grid,
        or — for an ordered indirect store — all cores but only the destination rows this rank owns
        (``sharded.py``).  Only what these cores read is uploaded and only what they wrote is read
        back: the returned arrays are valid inside ``last_slabs`` (arena byte ranges; tensor ``k``
        starts at ``last_layout[k][0]``) and unspecified elsewhere.  Nothing is exchanged between
        ranks; the caller merges slabs where it needs the whole result."""
        if self.memory.hbm.regions:
            raise ValueError("execute_shard does not take memory seeded at fixed addresses")
        self._prepare_execution(tuple(self._require_module().get_function(func_name).grid))
        sess, kwargs = self.session(func_name, _shard=(rank, world), **kwargs)
        if self._pool is None:
            from .pinned import PinnedPool
            self._pool = PinnedPool(self.device)
        arrays = {k: v for k, v in kwargs.items() if isinstance(v, np.ndarray)}
        outputs = self._execute_pipelined(sess, arrays)
        self.last_slabs = sess.written_ranges()
        self.last_layout = dict(sess.layout)
        return outputs

    def _execute_pipelined(self, sess: Session, arrays: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        pipe = sess.pipeline()
        tp = pipe.tp
        host = {k: np.ascontiguousarray(v) for k, v in arrays.items()}
        outputs = {k: self._pool.empty(v.shape, v.dtype) for k, v in arrays.items()}
        pipe.run(sess.dev, sess.arena, host, outputs, sess.run)
        sess.dev.sync()
        sess.last_h2d_bytes, sess.last_d2h_bytes = tp.h2d_bytes, tp.d2h_bytes
        return outputs

    def _execute_simple(self, sess: Session, arrays, seeded) -> Dict[str, np.ndarray]:
        """Small calls, and calls with memory seeded at fixed addresses: upload, launch, read back
        what the kernels wrote, one after the other on the launch stream."""
        for addr, arr in seeded.items():
            sess.dev.h2d(sess.arena + addr, arr)
        keep = []
        h2d = d2h = 0
        for k, v in arrays.items():
            # a tensor the kernel overwrites completely and never reads needs no upload
            if k not in sess.no_upload:
                keep.append(sess.upload(k, v))
                h2d += v.nbytes
        sess.run()
        outputs: Dict[str, np.ndarray] = {}
        for k, v in arrays.items():
            if k in sess.written:
                outputs[k] = sess.download(k, pool=self._pool)
                d2h += v.nbytes
            else:
                outputs[k] = np.array(v, copy=True)
        for addr, arr in seeded.items():
            sess.dev.d2h(arr, sess.arena + addr)              # what the kernels left at the fixed addresses
        sess.dev.sync()
        sess.last_h2d_bytes, sess.last_d2h_bytes = h2d, d2h
        del keep
        return outputs

    def _charge_latency(self, records, n_cores, layout, kwargs):
        """Per-call latency accounting (reset + charge, interpreter.py:118-120 of the reference)."""
        self._latency_tracker.reset()
        self._latency_tracker.set_cores_active(n_cores)
        self._latency_tracker.feed(records, HostTensors(layout, kwargs))

    def estimate_latency(self, func_name: str, **kwargs):
        """The latency report of a call without running it: host-only, needs no device.

        Uses the same trace as ``execute_function``; index tensors are read from ``kwargs``
        for the data-dependent stick counts of indirect tiles.
        """
        if self._latency_tracker is None:
            return None
        func = self._require_module().get_function(func_name)
        declared = func.arg_names
        if kwargs and declared and not any(k in declared for k in kwargs) and len(kwargs) == len(declared):
            kwargs = dict(zip(declared, kwargs.values()))
        tensors = [(k, tuple(v.shape), v.dtype) for k, v in kwargs.items() if isinstance(v, np.ndarray)]
        scalars = {k: v for k, v in kwargs.items() if not isinstance(v, np.ndarray)}
        layout, ptrs = arena_layout(tensors)
        from .trace_latency import LatencyRecorder
        tracer = Tracer(func, scalars, ptrs)
        tracer.latency = LatencyRecorder(tracer.ncores)
        tracer.run()
        self._charge_latency(tracer.latency.records, tracer.ncores, layout, kwargs)
        return self._latency_tracker.report()

"""Whole-grid symbolic trace of a KTIR function.

The reference runs one core after another and one op at a time
(ktir_cpu/grid.py:595-613, ktir_cpu/interpreter.py:196-281).  Here the function
body is walked once for *all* cores: integer SSA scalars (core ids, offsets,
loop counters) become int64 arrays over the iteration space
``[core, loop0, loop1, ...]``, tiles become nodes of an expression DAG, and
every ``ktdp.store`` becomes a :class:`Store` record holding the DAG that
produces the stored tile plus the per-point destination offsets.  The lowering
pass (``lower.py``) turns these records into CUDA launches.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .affine import AffineMap, AffineSet
from .dtypes import bytes_per_elem, canon, to_np_dtype
from .ir import IRFunction, Op, Region

MAX_UNROLL = 512


class Unsupported(NotImplementedError):
    """Raised when a kernel uses something this backend has no device path for."""


class CoreOrderHazard(Unsupported):
    """The cores (or loop iterations) of a grid cannot all run at once: one touches bytes another
    writes, so the result depends on the reference's core-after-core order (ktir_cpu/grid.py:595-613)."""


# ---------------------------------------------------------------------------
# Integer values over the iteration space
# ---------------------------------------------------------------------------

def is_iv(v) -> bool:
    return isinstance(v, (int, np.integer, np.ndarray)) and not isinstance(v, (bool, np.bool_))


def iv_align(a, b):
    if isinstance(a, np.ndarray) and isinstance(b, np.ndarray) and a.ndim != b.ndim:
        n = max(a.ndim, b.ndim)
        a = a.reshape(a.shape + (1,) * (n - a.ndim))
        b = b.reshape(b.shape + (1,) * (n - b.ndim))
    return a, b


def iv_bin(fn, a, b):
    a, b = iv_align(a, b)
    r = fn(a, b)
    if isinstance(r, np.ndarray) and r.dtype != np.bool_:
        r = r.astype(np.int64, copy=False)
    elif isinstance(r, np.integer):
        r = int(r)
    return r


def iv_full(v, shape: Tuple[int, ...]) -> np.ndarray:
    """Broadcast an integer value to the full iteration-space shape."""
    if isinstance(v, np.ndarray):
        v = v.reshape(v.shape + (1,) * (len(shape) - v.ndim))
        return np.broadcast_to(v, shape)
    return np.broadcast_to(np.int64(v), shape)


def iv_uniform(v) -> Optional[int]:
    """The single value of ``v`` if it is the same at every point, else None."""
    if isinstance(v, np.ndarray):
        if v.size == 0:
            return 0
        f = v.reshape(-1)
        return int(f[0]) if (f == f[0]).all() else None
    return int(v)


# ---------------------------------------------------------------------------
# Tile expression DAG
# ---------------------------------------------------------------------------

@dataclass(eq=False)
class Node:
    kind: str
    shape: Tuple[int, ...]
    dtype: str
    args: Tuple["Node", ...] = ()
    attrs: Dict[str, Any] = field(default_factory=dict)

    def __repr__(self):
        return f"Node({self.kind}{'/' + str(self.attrs.get('op')) if 'op' in self.attrs else ''}, {self.shape}, {self.dtype})"


@dataclass
class View:
    base: Any                      # element index (integer value)
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    dtype: str
    space: str = "global"
    box: Optional[Tuple[Tuple[int, ...], Tuple[int, ...]]] = None   # coordinate_set as (lo, hi) in global coordinates
    points: Optional[np.ndarray] = None                             # ... or, when it is not a box, its points [n, ndim]
    cset: Optional[AffineSet] = None
    syms: Tuple[int, ...] = ()


@dataclass
class DistView:
    """``ktdp.construct_distributed_memory_view``: partitions that each cover part of one global
    coordinate space (ktir_cpu/ir_types.py:266-378)."""
    parts: List[View]
    shape: Tuple[int, ...]
    dtype: str


@dataclass
class TableAccess:
    """An access tile resolved element by element: ``addr`` holds, for every point of the iteration
    space (leading axes) and every element of the tile (last axis, row-major), the element address
    it lives at, or -1 where no memory backs it (reads give 0, writes are dropped)."""
    dtype: str
    shape: Tuple[int, ...]
    addr: np.ndarray
    multi: bool = False            # some element is backed by more than one partition
    part: Optional[np.ndarray] = None   # which partition backs each entry of ``addr`` (for the stick counts)


@dataclass
class Access:
    """Direct access tile: a strided box (``coords is None``) or a coordinate list."""
    view: View
    off: Any                       # element offset of the tile origin (integer value)
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    coords: Optional[np.ndarray] = None   # [n, ndim] relative coordinates


@dataclass
class IndirectAccess:
    view: View
    shape: Tuple[int, ...]
    subs: List[Dict[str, Any]]     # per view dim: direct expr or indirect (view, exprs)
    index_views: Dict[str, View]
    ssa: Dict[str, Any]            # SSA scalars referenced in subscripts (integer values)
    order: Optional[AffineMap]
    aset: AffineSet


@dataclass
class Store:
    value: Node
    target: Any                    # Access | IndirectAccess
    axes: Tuple[int, ...]          # iteration-space shape at the store
    active: Optional[np.ndarray]   # bool mask over the iteration space, None = all
    seq: int = 0
    loop_path: Tuple[int, ...] = ()


@dataclass
class LoopInfo:
    """A traced ``scf.for`` with tile iter_args (body traced once, symbolically)."""
    trips: int
    axis: int                      # index of the trip axis in the iteration space
    inits: List[Any]
    yields: List[Any]


class Tracer:
    def __init__(self, func: IRFunction, scalar_args: Dict[str, Any], ptr_args: Dict[str, int],
                 core_range: Optional[Tuple[int, int]] = None):
        """``core_range = (lo, hi)`` traces only the grid cores with linear id in [lo, hi) — the
        slice of a kernel one GPU runs when its cores are split over several GPUs."""
        self.func = func
        nx, ny, nz = func.grid
        total = nx * ny * nz
        lo, hi = core_range if core_range is not None else (0, total)
        if not (0 <= lo <= hi <= total):
            raise ValueError(f"core range [{lo}, {hi}) outside the grid of {total} cores")
        self.total_cores = total
        self.core_base = lo
        self.ncores = hi - lo
        cid = np.arange(lo, hi, dtype=np.int64)
        self.core_xyz = (cid % nx, (cid % (nx * ny)) // nx, cid // (nx * ny))
        self.axes: List[int] = [self.ncores]
        self.active: Optional[np.ndarray] = None
        self.stores: List[Store] = []
        self.unroll_loops = False       # trace every scf.for iteration by iteration (its stores become statements of their own)
        self.loop_path: List[int] = []
        self._loop_counter = 0
        self.latency = None            # a trace_latency.LatencyRecorder when the latency model is on
        self.lx = None                 # an lx.LXModel when scratchpad accounting is on
        self.arena = None              # a lower.ArenaMap: accesses are clipped to the allocation they start in
        self.scope: Dict[str, Any] = {}
        for n, _ in func.args:
            key = n[1:]
            if key in ptr_args:
                self.scope[n] = int(ptr_args[key])
            elif key in scalar_args:
                self.scope[n] = scalar_args[key]

    # -- helpers ---------------------------------------------------------
    def get(self, scope, name):
        try:
            return scope[name]
        except KeyError:
            raise KeyError(f"Value '{name}' not found")

    def run(self):
        self.trace_ops(self.func.ops, self.scope)
        return self.stores

    def cores_active(self) -> np.ndarray:
        """Per core: does it execute the op being traced (at any loop point)?"""
        if self.active is None:
            return np.ones(self.ncores, bool)
        return self.active.reshape(self.ncores, -1).any(axis=1)

    def trace_region(self, ops: Sequence[Op], scope: Dict[str, Any], bind: Sequence[Tuple[str, Any]] = ()):
        """Trace a nested region in its own scratchpad scope (CoreContext.push_scope / pop_scope,
        ktir_cpu/grid.py:210-236); ``bind`` = (name, tile) pairs the region starts with."""
        lx = self.lx
        if lx is None:
            return self.trace_ops(ops, scope)
        lx.push()
        try:
            cores = self.cores_active()
            for name, tile in bind:
                if hasattr(tile, "shape") and hasattr(tile, "dtype") and not isinstance(tile, np.ndarray):
                    lx.set_value(name, tile, cores)
            return self.trace_ops(ops, scope)
        finally:
            lx.pop()

    def trace_ops(self, ops: Sequence[Op], scope: Dict[str, Any]):
        for op in ops:
            r = self.trace_op(op, scope)
            if isinstance(r, _Yield):
                return r
        return None

    def bind(self, op: Op, scope, value):
        if not op.results:
            return
        pairs = [(op.results[0], value)] if len(op.results) == 1 else list(zip(op.results, value))
        for n, v in pairs:
            scope[n] = v
        if self.lx is not None:
            cores = self.cores_active()
            for n, v in pairs:
                if isinstance(v, Node):
                    # constants are compile-time literals: no scratchpad (registry no_lx_charge)
                    from .registry import NO_LX_CHARGE
                    self.lx.set_value(n, v, cores, charge=op.name not in NO_LX_CHARGE)

    def trace_op(self, op: Op, scope):
        from . import trace_comm, trace_mem, trace_ops2  # noqa: F401  (fill the rule table)
        from . import trace_ops as T
        fn = T.TABLE.get(op.name)
        if fn is None:
            if op.name.startswith("ktdp."):
                raise Unsupported(f"{op.name} (cross-core / distributed ops have no device path yet)")
            raise ValueError(f"Unknown operation: {op.name}")
        lat = self.latency
        pre = lat.before_op(self, op, scope) if lat is not None else None
        if self.lx is not None:
            # operands are fetched before the result exists; a last use frees its tile
            # (scf.for only peeks at its iter_args inits: they are copied, not consumed)
            for n in op.operands[:_FETCHED.get(op.name, len(op.operands))]:
                if isinstance(n, str):
                    self.lx.fetch(n)
        r = fn(self, op, scope)
        if isinstance(r, _Yield):
            return r
        if pre is not None:
            lat.after_op(self, op, scope, r, pre)
        self.bind(op, scope, r)
        return r


# How many leading operands a handler of the reference actually reads (the rest — an ``outs`` that only
# gives the shape, the inits an scf.for copies — is never fetched, hence never released by a last use):
# ktir_cpu/dialects/linalg_ops.py:254-303,600-608, ktir_cpu/dialects/scf_ops.py:57-66.
_FETCHED = {"linalg.transpose": 1, "linalg.add": 2, "linalg.max": 2, "scf.for": 3}


class _Yield:
    def __init__(self, values):
        self.values = values

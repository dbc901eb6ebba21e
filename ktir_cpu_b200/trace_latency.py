"""Feeds the latency model from the whole-grid trace.

The reference records one cost entry per op per core as it dispatches
(ktir_cpu/interpreter.py:268-279).  The tracer visits an op once for all cores, so
the recorder turns each visit into an :class:`OpRecord` — the op, how many times
each core executes it (active iteration points of that core) and what one
execution costs — following the reference's sizing rules:

* element count = size of the result tile, else of the first tile operand, else 1
  (ktir_cpu/latency.py:509-517);
* matmul dims from the first two tile operands (ktir_cpu/latency.py:520-531);
* ``ktdp.load`` / ``ktdp.store`` = distinct 128-byte sticks among the element addresses
  of the tile, plus the sticks of the index elements for indirect tiles
  (ktir_cpu/ops/memory_ops.py:84-107, 765-800, 895-964);
* ``linalg.reduce`` itself is free; its combiner ops are charged once per level of
  the pairwise halving fold, on tiles of the halved extent, and once more for the
  combine with ``outs`` (ktir_cpu/dialects/linalg_ops.py:61-246).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np

from .dtypes import bytes_per_elem
from .latency import STICK_BYTES, LatencyCategory as LC, OpRecord, get_latency_category
from .trace import Access, IndirectAccess, Node, TableAccess, iv_full


def _is_node(v) -> bool:
    return isinstance(v, Node)


class LatencyRecorder:
    def __init__(self, ncores: int):
        self.ncores = ncores
        # every core dispatches at least the function's free ops, so every core has a counter
        self.records: List[OpRecord] = [OpRecord("func.return", LC.ZERO, np.ones(ncores, np.int64), "zero")]

    # -- executions per core at the tracer's current position ---------------------------------
    repeat = None        # [n_cores] runs of the region being traced per execution (a ring reduce's combiner)

    def counts(self, tr) -> np.ndarray:
        axes = tuple(tr.axes)
        if tr.active is None:
            c = np.full(self.ncores, int(np.prod(axes[1:], dtype=np.int64)), np.int64)
        else:
            act = tr.active
            extra = int(np.prod(axes[act.ndim:], dtype=np.int64))        # axes of a symbolic loop
            c = act.reshape(self.ncores, -1).sum(1).astype(np.int64) * extra
        return c if self.repeat is None else c * self.repeat

    def _active_full(self, tr) -> np.ndarray:
        axes = tuple(tr.axes)
        if tr.active is None:
            return np.ones(axes, bool)
        act = tr.active
        return np.broadcast_to(act.reshape(act.shape + (1,) * (len(axes) - act.ndim)), axes)

    # -- hook -------------------------------------------------------------------------------
    def before_op(self, tr, op, scope):
        """Operand values as they are before the op runs (some ops rebind their ``outs`` name)."""
        if get_latency_category(op.name) == LC.ZERO and op.name != "linalg.reduce":
            return None
        return [scope.get(n) if isinstance(n, str) else None for n in op.operands]

    def after_op(self, tr, op, scope, result, operands):
        name = op.name
        if name == "linalg.reduce":
            return self._reduce(tr, op, operands)
        cat = get_latency_category(name)
        if cat == LC.ZERO:
            return
        if cat == LC.MEMORY:
            return self._memory(tr, op, operands, result)
        cnt = self.counts(tr)
        if not cnt.any():
            return
        if cat == LC.COMPUTE_MATMUL:
            tiles = [v for v in operands if _is_node(v)]
            m = n = k = 1
            if len(tiles) >= 2:
                a, b = tiles[0], tiles[1]
                m = a.shape[0] if len(a.shape) >= 2 else 1
                k = a.shape[1] if len(a.shape) >= 2 else a.shape[0]
                n = b.shape[1] if len(b.shape) >= 2 else 1
            self.records.append(OpRecord(name, cat, cnt, "matmul", mnk=(int(m), int(n), int(k))))
            return
        if cat == LC.COMM:
            # every core sends its tile n - 1 times around the ring, whatever its group
            # (RingReduceBackend.run, ktir_cpu/ops/comm_ops.py:294-345)
            if not _is_node(result):
                return
            from .dtypes import bytes_per_elem
            per_exec = (tr.total_cores - 1) * int(np.prod(result.shape, dtype=np.int64)) * bytes_per_elem(result.dtype)
            self.records.append(OpRecord(name, cat, cnt, "comm", nbytes=cnt * per_exec))
            return
        self.records.append(OpRecord(name, cat, cnt, "elems", n_elems=self._num_elements(result, operands)))

    @staticmethod
    def _num_elements(result, operands) -> int:
        if isinstance(result, tuple) and result and _is_node(result[0]):
            result = result[0]
        if _is_node(result):
            return int(np.prod(result.shape, dtype=np.int64))
        for v in operands:
            if _is_node(v):
                return int(np.prod(v.shape, dtype=np.int64))
        return 1

    # -- linalg.reduce: the combiner region, level by level -----------------------------------
    def _reduce(self, tr, op, operands):
        tile = operands[0] if operands else None
        if not _is_node(tile):
            return
        cnt = self.counts(tr)
        if not cnt.any():
            return
        if op.regions and op.regions[0].ops:
            body = [o.name for o in op.regions[0].ops if o.name != "linalg.yield"]
        else:
            body = [op.attrs.get("combiner") or "arith.addf"]
        outs_is_tile = len(operands) > 1 and _is_node(operands[1])
        dims = op.attrs.get("dimensions")
        shape = list(tile.shape)
        if dims is None:
            shape, fold_dims = [int(np.prod(shape, dtype=np.int64))], [0]
        else:
            fold_dims = sorted(dims, reverse=True)

        def charge(n_elems: int):
            for nm in body:
                cat = get_latency_category(nm)
                if cat != LC.ZERO:
                    self.records.append(OpRecord(nm, cat, cnt, "elems", n_elems=int(n_elems)))

        for d in fold_dims:
            n = shape[d]
            while n > 1:
                half = n // 2
                lvl = list(shape)
                lvl[d] = half
                charge(np.prod(lvl, dtype=np.int64))
                n = half + (n % 2)
            shape[d] = 1
        if outs_is_tile:
            red = [s for i, s in enumerate(shape) if dims is not None and i not in dims]
            charge(np.prod(red, dtype=np.int64) if red else 1)

    # -- ktdp.load / ktdp.store ------------------------------------------------------------------
    def _memory(self, tr, op, operands, result):
        if op.name == "ktdp.load":
            acc = result.attrs.get("access") if _is_node(result) else None
        else:
            acc = operands[1] if len(operands) > 1 else None
        cnt = self.counts(tr)
        if acc is None or not cnt.any():
            return
        axes = tuple(tr.axes)
        active = self._active_full(tr)
        if isinstance(acc, Access):
            sticks = direct_sticks(acc, axes)
            per_core = np.where(active, sticks, 0).reshape(self.ncores, -1).sum(1) * STICK_BYTES
            self.records.append(OpRecord(op.name, LC.MEMORY, cnt, "bytes", nbytes=per_core.astype(np.int64)))
        elif isinstance(acc, TableAccess):
            sticks = table_sticks(acc, axes)
            per_core = np.where(active, sticks, 0).reshape(self.ncores, -1).sum(1) * STICK_BYTES
            self.records.append(OpRecord(op.name, LC.MEMORY, cnt, "bytes", nbytes=per_core.astype(np.int64)))
        elif isinstance(acc, IndirectAccess):
            sel = np.nonzero(active.reshape(-1))[0]
            per_point = int(np.prod(axes[1:], dtype=np.int64))
            core_of = sel // per_point
            ncores = self.ncores

            def resolve(host, acc=acc, axes=axes, sel=sel, core_of=core_of):
                st = indirect_sticks(acc, axes, sel, host)
                return np.bincount(core_of, weights=st, minlength=ncores).astype(np.int64) * STICK_BYTES
            self.records.append(OpRecord(op.name, LC.MEMORY, cnt, "indirect", resolve=resolve))


def _rel_offsets(acc: Access) -> np.ndarray:
    """Element offsets of every element of the tile relative to its origin."""
    if acc.coords is not None:
        return (acc.coords * np.asarray(acc.strides, np.int64)[None, :]).sum(1)
    shape = tuple(acc.shape) or (1,)
    strides = tuple(acc.strides) or (1,)
    rel = np.zeros(shape, np.int64)
    for d, (n, s) in enumerate(zip(shape, strides)):
        rs = [1] * len(shape)
        rs[d] = n
        rel = rel + (np.arange(n, dtype=np.int64) * s).reshape(rs)
    return rel.reshape(-1)


def direct_sticks(acc: Access, axes) -> np.ndarray:
    """Distinct sticks per iteration point of a direct access tile, shape ``axes``.

    The element pattern is the same at every point, so the count depends only on the
    byte address of the origin modulo the stick size.
    """
    bpe = bytes_per_elem(acc.view.dtype)
    base = iv_full(acc.off, axes).astype(np.int64) * bpe
    res = base % STICK_BYTES
    rel = _rel_offsets(acc) * bpe
    out = np.zeros(axes, np.int64)
    for r in np.unique(res):
        n = int(np.unique((int(r) + rel) // STICK_BYTES).size)
        out[res == r] = n
    return out


def table_sticks(acc: TableAccess, axes) -> np.ndarray:
    """Sticks per iteration point of a tile resolved through a distributed view: the distinct sticks
    of each partition's share, summed over the partitions (MemoryOps.distributed_load adds up the
    counts of its per-partition loads, ktir_cpu/ops/memory_ops.py:1127-1195)."""
    E = acc.addr.shape[-1]
    addr = np.broadcast_to(acc.addr.reshape(acc.addr.shape[:-1] + (1,) * (len(axes) - acc.addr.ndim + 1) + (E,)),
                           tuple(axes) + (E,)).reshape(-1, E)
    part = np.broadcast_to(acc.part.reshape(acc.part.shape[:-1] + (1,) * (len(axes) - acc.part.ndim + 1) + (E,)),
                           tuple(axes) + (E,)).reshape(-1, E).astype(np.int64)
    valid = addr >= 0
    key = np.where(valid, (part << 44) + addr * bytes_per_elem(acc.dtype) // STICK_BYTES, -1)
    n = _unique_per_row(key) - (~valid).any(1)
    return n.reshape(axes).astype(np.int64)


def _union_count(first: np.ndarray, last: np.ndarray) -> np.ndarray:
    """Per row of ``first``/``last`` ([n, k] inclusive stick intervals): size of their union."""
    order = np.argsort(first, axis=1, kind="stable")
    f = np.take_along_axis(first, order, 1)
    l = np.take_along_axis(last, order, 1)
    run = np.maximum.accumulate(l, axis=1)
    prev = np.concatenate([np.full((f.shape[0], 1), -1, np.int64), run[:, :-1]], axis=1)
    return np.maximum(l - np.maximum(f, prev + 1) + 1, 0).sum(1)


def indirect_sticks(acc: IndirectAccess, axes, sel: np.ndarray, host) -> np.ndarray:
    """Data sticks + index sticks of an indirect tile at the points ``sel``; needs index values.

    ``host.read(dtype, element_indices)`` returns the caller's values at those element indices.
    """
    from .lower_scatter import row_form
    from .trace import Unsupported
    try:
        f = row_form(acc, axes, sel)
    except Unsupported:
        return _indirect_sticks_general(acc, axes, sel, host)
    n = len(sel)
    if n == 0:
        return np.zeros(0, np.int64)
    r = np.arange(f.rows, dtype=np.int64)[None, :]
    idx_elems = f.idx_off[:, None] + r * f.idx_stride                        # [n, rows]
    vals = host.read(f.idx_dtype, idx_elems.reshape(-1)).reshape(n, f.rows).astype(np.int64)
    if (vals < 0).any():
        bad = int(vals[vals < 0][0])
        raise IndexError(f"indirect index {bad} is negative")
    bpe = bytes_per_elem(f.dtype)
    start = (f.base[:, None] + vals * f.idx_mult + r * f.pos_stride) * bpe
    data = _union_count(start // STICK_BYTES, (start + f.cols * bpe - 1) // STICK_BYTES)
    ib = bytes_per_elem(f.idx_dtype)
    ia = idx_elems * ib
    idx = _union_count(ia // STICK_BYTES, (ia + ib - 1) // STICK_BYTES)
    return (data + idx).astype(np.int64)


def _unique_per_row(x: np.ndarray) -> np.ndarray:
    """Number of distinct values in each row of a 2-D integer array."""
    if x.shape[1] == 0:
        return np.zeros(x.shape[0], np.int64)
    y = np.sort(x, axis=1)
    return 1 + (np.diff(y, axis=1) != 0).sum(1)


def _indirect_sticks_general(ia: IndirectAccess, axes, sel: np.ndarray, host) -> np.ndarray:
    """Stick counts of an indirect tile of any rectangular form: one address per element, host side."""
    from .lower_scatter import sub_values
    from .trace import Unsupported
    from .lower_generic import variable_space_points
    vars_e = variable_space_points(ia)
    nv = vars_e.shape[0]

    def at(v):
        return np.ascontiguousarray(iv_full(v, axes).reshape(-1)[sel]).astype(np.int64)

    def ssa_at(name):
        return at(ia.ssa[name])

    addr = at(ia.view.base)[:, None] + np.zeros((1, vars_e.shape[1]), np.int64)
    idx_sticks = np.zeros(len(sel), np.int64)
    for sub, stride in zip(ia.subs, ia.view.strides):
        if sub["kind"] == "direct":
            addr = addr + stride * sub_values(sub["expr"], vars_e, ssa_at)
        else:
            iv = ia.index_views[sub["view"]]
            iaddr = at(iv.base)[:, None] + np.zeros((1, vars_e.shape[1]), np.int64)
            for e_, s_ in zip(sub["exprs"], iv.strides):
                iaddr = iaddr + s_ * sub_values(e_, vars_e, ssa_at)
            vals = host.read(iv.dtype, iaddr.reshape(-1)).reshape(iaddr.shape).astype(np.int64)
            if (vals < 0).any():
                raise IndexError(f"indirect index {int(vals[vals < 0][0])} is negative")
            addr = addr + vals * stride
            idx_sticks += _unique_per_row(iaddr * bytes_per_elem(iv.dtype) // STICK_BYTES)
    data = _unique_per_row(addr * bytes_per_elem(ia.view.dtype) // STICK_BYTES)
    return (data + idx_sticks).astype(np.int64)

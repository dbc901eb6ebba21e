"""Trace rules of the cross-core ops: ``ktdp.inter_tile_produce`` / ``ktdp.inter_tile_reduce``.

The reference runs a ring over the whole workgroup (ktir_cpu/ops/comm_ops.py:229-345): core ``c``
starts from its own partial and in round ``k`` folds in — through the combiner region, in the
tile's dtype — the partial that originated on core ``(c - k) mod n``, provided that core is a
producer of ``c``'s group.  A forwarded tile is never modified, so what core ``c`` computes is

    acc = partial[c];  for k = 1 .. n-1:  acc = combine(acc, partial[(c - k) mod n])   (group members only)

and every core has its own fold order.  The trace records exactly that as one DAG node
(``ringred``) with a per-core list of source cores; the device evaluates it with the group's
partials in the shared memory of a thread-block cluster (``g_ring_kernel`` in ``csrc/generic_ops.cu``).

A core that never reaches the reduce leaves its ring neighbours waiting for ever; the reference's
scheduler reports ``RuntimeError("Deadlock detected: ...")`` (ktir_cpu/grid.py:615-621), and so does
the trace when the op sits under a condition that only some cores take.
"""
from __future__ import annotations

import numpy as np

from .trace import Node, Tracer, Unsupported, _Yield, iv_full
from .trace_ops import is_node, rule


class TileFuture:
    """What ``inter_tile_produce`` binds: the local partial plus the sets that say who shares it
    (ktir_cpu/ir_types.py:480-521)."""

    def __init__(self, partial: Node, producer_set, groups_set, group_of_core: np.ndarray):
        self.partial = partial
        self.producer_set = producer_set
        self.groups_set = groups_set
        self.group_of_core = group_of_core


def _core_ids(tr: Tracer) -> np.ndarray:
    return tr.core_base + np.arange(tr.ncores, dtype=np.int64)


def _require_whole_workgroup(tr: Tracer, what: str):
    if tr.ncores != tr.total_cores:
        raise Unsupported(f"{what} in a kernel split over several GPUs (the ring spans every core of the grid)")
    if tr.active is not None:
        per_core = tr.active.reshape(tr.ncores, -1).all(axis=1)
        if not per_core.all():
            out = np.flatnonzero(~per_core)
            n = tr.total_cores
            waits = "; ".join(f"core {(int(c) + 1) % n} waiting on recv from core {int(c)}" for c in out[:4])
            raise RuntimeError(f"Deadlock detected: {waits}")


@rule("ktdp.inter_tile_produce")
def _produce(tr: Tracer, op, scope):
    _require_whole_workgroup(tr, "ktdp.inter_tile_produce")
    pset, gset = op.attrs["producer_tiles_per_group"], op.attrs["groups"]
    n = tr.total_cores
    groups = [g for g in range(n) if gset.contains([g])]
    gid = np.full(tr.ncores, -1, np.int64)
    for i, c in enumerate(_core_ids(tr)):
        hits = [g for g in groups if pset.contains([int(c)], [g])]
        if not hits:
            raise RuntimeError(f"tile {int(c)} is not contained in any producer group")
        if len(hits) > 1:
            raise RuntimeError(f"tile {int(c)} matched multiple groups {hits} — violates the disjointness invariant")
        gid[i] = hits[0]
    inner = dict(scope)
    reg = op.regions[0]
    if reg.arg_names:
        inner[reg.arg_names[0]] = gid.copy()
    y = tr.trace_ops(reg.ops, inner)
    if not isinstance(y, _Yield) or not y.values or not is_node(y.values[0]):
        raise TypeError("ktdp.inter_tile_produce: the region must yield a tile (ktdp.yield_partial)")
    if len(y.values) > 1:
        raise Unsupported("ktdp.inter_tile_produce yielding more than one partial")
    return TileFuture(y.values[0], pset, gset, gid)


def _combiner(tr: Tracer, op, partial: Node, folds: np.ndarray):
    """The combiner region as (elementwise op name, swapped): result = op(lhs, rhs), or op(rhs, lhs).
    ``folds`` = runs of the region per core, for the latency model (the reference charges every op of
    every fold like any other op)."""
    reg = op.regions[0] if op.regions else None
    if reg is None or len(reg.arg_names) < 2:
        raise ValueError("ktdp.inter_tile_reduce: combiner region needs >=2 block args (lhs, rhs)")
    lhs = Node("arg", partial.shape, partial.dtype, (), {"name": "lhs"})
    rhs = Node("arg", partial.shape, partial.dtype, (), {"name": "rhs"})
    inner = {reg.arg_names[0]: lhs, reg.arg_names[1]: rhs}
    if tr.latency is not None:
        tr.latency.repeat = folds
    try:
        y = tr.trace_region(reg.ops, inner, [(reg.arg_names[0], lhs), (reg.arg_names[1], rhs)])
    finally:
        if tr.latency is not None:
            tr.latency.repeat = None
    if not isinstance(y, _Yield) or not y.values or not is_node(y.values[0]):
        raise TypeError("ktdp.inter_tile_reduce: combiner did not yield a Tile")
    root = y.values[0]
    while root.kind == "reshape":
        root = root.args[0]
    if root.kind == "ew" and len(root.args) == 2:
        a, b = root.args
        if a is lhs and b is rhs:
            return root.attrs["op"], False
        if a is rhs and b is lhs:
            return root.attrs["op"], True
    raise Unsupported("ktdp.inter_tile_reduce whose combiner is more than one elementwise op of (lhs, rhs)")


@rule("ktdp.inter_tile_reduce")
def _reduce(tr: Tracer, op, scope):
    fut = tr.get(scope, op.operands[0])
    if not isinstance(fut, TileFuture):
        raise TypeError(f"ktdp.inter_tile_reduce: operand 0 must be a TileFuture, got {type(fut)}")
    _require_whole_workgroup(tr, "ktdp.inter_tile_reduce")
    tr.get(scope, op.operands[1])                    # identity: seeds non-producers; every core here produces
    n = tr.total_cores
    cset = op.attrs["consumer_tiles_per_group"]
    cores = _core_ids(tr)
    sources = np.full((tr.ncores, max(n - 1, 1)), -1, np.int64)
    counts = np.zeros(tr.ncores, np.int64)
    consumer = np.zeros(tr.ncores, bool)
    for i, c in enumerate(cores):
        g = int(fut.group_of_core[i])
        consumer[i] = cset.contains([int(c)], [g])
        for k in range(1, n):
            origin = (int(c) - k) % n
            if fut.producer_set.contains([origin], [g]):
                sources[i, counts[i]] = origin
                counts[i] += 1
    opname, swapped = _combiner(tr, op, fut.partial, counts)
    shape = tuple(op.result_types[0].shape) if op.result_types and op.result_types[0].shape is not None \
        else tuple(fut.partial.shape)
    if int(np.prod(shape)) != int(np.prod(fut.partial.shape)):
        raise ValueError("ktdp.inter_tile_reduce: result type does not hold the partial's elements")
    return Node("ringred", shape, fut.partial.dtype, (fut.partial,),
                {"op": opname, "swapped": swapped, "sources": sources[:, :max(int(counts.max()), 1)], "counts": counts,
                 "consumer": consumer, "groups": fut.group_of_core.copy()})


@rule("ktdp.yield_partial", "ktdp.yield_reduced")
def _yield(tr: Tracer, op, scope):
    return _Yield([tr.get(scope, n) for n in op.operands])

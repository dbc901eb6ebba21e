"""Trace rules for the ktdp dialect: grid ids, memory views, access tiles, load/store.

Address arithmetic follows MemoryOps.tile_access / _subtile_ref
(ktir_cpu/ops/memory_ops.py:610-646, 1100-1124): element offset = view base +
sum(index * stride) + sum(box_lo * stride); here each term is an int64 array
over the iteration space, so one evaluation yields the offsets of every core
and loop iteration.
"""
from __future__ import annotations

import numpy as np

from .affine import AffineMap, AffineSet
from .dtypes import canon
from .trace import (Access, IndirectAccess, Node, Store, Tracer, Unsupported, View, is_iv, iv_bin,
                    iv_uniform)
from .trace_ops import is_node, rule


@rule("ktdp.get_compute_tile_id")
def _tile_id(tr: Tracer, op, scope):
    n = len(op.results)
    if n == 1:
        return tr.core_xyz[0].copy()
    return tuple(tr.core_xyz[d].copy() for d in range(n))


@rule("ktdp.construct_memory_view")
def _memory_view(tr, op, scope):
    if not op.operands:
        raise ValueError("construct_memory_view: missing pointer operand")
    ptr = tr.get(scope, op.operands[0])
    if not is_iv(ptr):
        raise Unsupported("construct_memory_view: pointer must be an integer value")
    space = op.attrs.get("memory_space", "global")
    if space not in ("global", "HBM", "hbm"):
        raise Unsupported(f"memory space '{space}' (core-local scratchpad views)")

    def dims(key):
        out = []
        for s in op.attrs[key]:
            v = tr.get(scope, s) if isinstance(s, str) else s
            u = iv_uniform(v)
            if u is None:
                raise Unsupported(f"construct_memory_view: per-core {key}")
            out.append(u)
        return tuple(out)

    return View(ptr, dims("sizes"), dims("strides"), canon(op.attrs["dtype"]), "global")


@rule("ktdp.construct_access_tile")
def _access_tile(tr, op, scope):
    view = tr.get(scope, op.operands[0])
    if not isinstance(view, View):
        raise Unsupported("construct_access_tile on a distributed memory view")
    idx = [tr.get(scope, i) if isinstance(i, str) else i for i in op.attrs["indices"]]
    bm = op.attrs.get("base_map")
    coords = bm.eval(idx) if isinstance(bm, AffineMap) else idx
    off = view.base
    for c, s in zip(coords, view.strides):
        off = iv_bin(lambda a, b: a + b, off, iv_bin(lambda x, y: x * y, c, s))
    shape = tuple(op.attrs["shape"])
    aset: AffineSet = op.attrs.get("set")
    order: AffineMap = op.attrs.get("order")
    if aset is not None and aset.n_syms:
        raise NotImplementedError("construct_access_tile: symbolic access_tile_set is not yet supported")
    box = aset.box() if aset is not None else (tuple([0] * len(shape)), shape)
    ident = order is None or order.is_identity()
    if box is not None and ident:
        lo, hi = box
        off = iv_bin(lambda a, b: a + b, off, sum(l * s for l, s in zip(lo, view.strides)))
        return Access(view, off, tuple(h - l for l, h in zip(lo, hi)), tuple(view.strides))
    pts = aset.enumerate(shape)
    if order is not None:
        pts = [order.eval(pt) for pt in pts]
    coords_arr = np.asarray(pts, dtype=np.int64).reshape(len(pts), len(shape))
    return Access(view, off, shape, tuple(view.strides), coords_arr)


@rule("ktdp.construct_indirect_access_tile")
def _indirect_tile(tr, op, scope):
    view = tr.get(scope, op.operands[0])
    ivs = {}
    for s in op.attrs["subscripts"]:
        if s["kind"] == "indirect":
            iv = tr.get(scope, s["view"])
            if not isinstance(iv, View):
                raise Unsupported("indirect access through a non-view index operand")
            ivs[s["view"]] = iv
    ssa = {n: tr.get(scope, n) for n in op.attrs["ssa_refs"]}
    for n, v in ssa.items():
        if not is_iv(v):
            raise Unsupported(f"indirect subscript uses non-integer value {n}")
    return IndirectAccess(view, tuple(op.attrs["shape"]), op.attrs["subscripts"], ivs, ssa,
                          op.attrs.get("order"), op.attrs["set"])


@rule("ktdp.load")
def _load(tr, op, scope):
    at = tr.get(scope, op.operands[0])
    rshape = tuple(op.result_types[0].shape) if op.result_types else tuple(at.shape)
    if isinstance(at, IndirectAccess):
        if at.order is not None and not at.order.is_permutation():
            raise ValueError("indirect_load: variables_space_order must permute its input "
                             f"dimensions; got non-permutation map: {at.order.source}")
        return Node("iload", rshape, at.view.dtype, (), {"access": at, "axes": tuple(tr.axes)})
    if not isinstance(at, Access):
        raise Unsupported("ktdp.load from a distributed access tile")
    shape = tuple(at.shape) if at.coords is None else rshape
    return Node("load", shape, at.view.dtype, (), {"access": at, "axes": tuple(tr.axes)})


@rule("ktdp.store")
def _store(tr, op, scope):
    value = tr.get(scope, op.operands[0])
    at = tr.get(scope, op.operands[1])
    assert is_node(value), f"ktdp.store expects a Tile, got {type(value)}"
    if isinstance(at, IndirectAccess):
        if tuple(value.shape) != tuple(at.shape):
            raise ValueError(f"indirect_store: source tile shape {tuple(value.shape)} does not "
                             f"match IAT shape {tuple(at.shape)}")
        if at.order is not None and not at.order.is_permutation():
            raise ValueError("indirect_store: variables_space_order must permute its input "
                             f"dimensions; got non-permutation map: {at.order.source}")
    elif not isinstance(at, Access):
        raise Unsupported("ktdp.store to a distributed access tile")
    tr.stores.append(Store(value, at, tuple(tr.axes),
                           None if tr.active is None else tr.active.copy(),
                           len(tr.stores), tuple(tr.loop_path)))
    return None

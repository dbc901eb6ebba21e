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
from .dtypes import bytes_per_elem
from .trace import (Access, DistView, IndirectAccess, Node, Store, TableAccess, Tracer, Unsupported, View, is_iv,
                    iv_bin, iv_full, iv_uniform)
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

    view = View(ptr, dims("sizes"), dims("strides"), canon(op.attrs["dtype"]), "global")
    cset = op.attrs.get("coordinate_set")
    if isinstance(cset, AffineSet):
        # symbols of the set are bound, left to right, to the dynamic entries of ``sizes``
        # (ktir_cpu/dialects/ktdp_ops.py:88-110)
        syms = [iv_uniform(tr.get(scope, s_)) for s_ in op.attrs["sizes"] if isinstance(s_, str)]
        if cset.n_syms and len(syms) < cset.n_syms:
            raise ValueError(f"construct_memory_view: coordinate_set has {cset.n_syms} symbol(s) but sizes has "
                             f"{len(syms)} dynamic entries")
        view.box = cset.box_with(syms)
        view.cset, view.syms = cset, tuple(syms)
    return view


@rule("ktdp.construct_distributed_memory_view")
def _dist_view(tr, op, scope):
    """Partitions composed into one global coordinate space
    (ktir_cpu/dialects/ktdp_ops.py:114-150, ktir_cpu/ir_types.py:176-316)."""
    parts = [tr.get(scope, n) for n in op.operands]
    if not parts:
        raise ValueError("DistributedMemRef requires at least one partition")
    dtype = canon(op.attrs["dtype"])
    for i, pv in enumerate(parts):
        if not isinstance(pv, View):
            raise ValueError(f"construct_distributed_memory_view: operand {i} is {type(pv).__name__}, expected MemRef")
        if getattr(pv, "cset", None) is None:
            raise ValueError(f"DistributedMemRef partition {i} must have a coordinate_set")
        if pv.dtype != dtype:
            raise ValueError(f"DistributedMemRef partition {i} dtype {pv.dtype!r} does not match view dtype {dtype!r}")
    ndim = len(op.attrs["shape"])
    extent = [None] * ndim
    for pv in parts:
        if pv.box is not None:
            if len(pv.box[1]) != ndim:
                raise ValueError("construct_distributed_memory_view: partition rank does not match the view's rank")
            for d in range(ndim):
                extent[d] = pv.box[1][d] if extent[d] is None else max(extent[d], pv.box[1][d])
    shape = []
    for d, declared in enumerate(op.attrs["shape"]):
        if declared is None:
            if any(pv.box is None for pv in parts):
                raise ValueError("construct_distributed_memory_view: a dynamic result shape needs box-shaped partitions")
            declared = extent[d]
        elif extent[d] is not None and declared != extent[d]:
            raise ValueError(f"construct_distributed_memory_view: declared shape axis {d} = {declared} does not match "
                             f"the partition extent (max(hi)) = {extent[d]}; the view's declared shape must equal the "
                             "global coordinate extent covered by its partitions")
        shape.append(int(declared))
    for pv in parts:
        if pv.box is None and pv.points is None:
            pts = pv.cset.enumerate(shape, pv.syms)
            pv.points = np.asarray(pts, np.int64).reshape(len(pts), ndim)
    return DistView(parts, tuple(shape), dtype)


def _distributed_access(tr, dv: DistView, coords, shape, aset, order) -> TableAccess:
    """Which partition backs every element of the access tile, for every point of the iteration
    space (MemoryOps.distributed_tile_access / distributed_load, ktir_cpu/ops/memory_ops.py:985-1259):
    element ``a`` of the tile sits at global coordinate ``x + a``; partition i holds it when that
    coordinate is in its coordinate set B_i, at ``base_i + sum((x + a - p_i) * stride_i)`` with
    ``p_i = min(B_i)``.  Partitions are visited in order, so where they overlap a load sees the last."""
    if order is not None and not order.is_identity():
        raise Unsupported("access_tile_order other than the identity on a distributed memory view")
    ndim = len(dv.shape)
    if len(shape) != ndim or len(coords) != ndim:
        raise ValueError("construct_access_tile: rank of the access tile does not match the distributed view")
    axes = tuple(tr.axes)
    x = [np.ascontiguousarray(iv_full(c, axes)).reshape(-1) for c in coords]          # [P] per dim
    P = x[0].size if x else 1
    local = np.stack(np.meshgrid(*[np.arange(n_, dtype=np.int64) for n_ in shape], indexing="ij"), -1).reshape(-1, ndim)
    E = local.shape[0]
    in_tile = np.ones(E, bool)
    if aset is not None:
        b = aset.box()
        if b is not None:
            in_tile = ((local >= np.asarray(b[0])) & (local < np.asarray(b[1]))).all(1)
        else:
            in_tile = np.fromiter((aset.contains(tuple(int(v) for v in pt)) for pt in local), bool, E)
    addr = np.full((P, E), -1, np.int64)
    part = np.full((P, E), -1, np.int16)
    hits = np.zeros((P, E), np.int8)
    bpe = bytes_per_elem(dv.dtype)
    for pi, pv in enumerate(dv.parts):
        g = [x[d][:, None] + local[None, :, d] for d in range(ndim)]                  # global coordinates [P, E]
        if pv.box is not None:
            lo, hi = pv.box
            inside = np.ones((P, E), bool)
            for d in range(ndim):
                inside &= (g[d] >= lo[d]) & (g[d] < hi[d])
            origin = lo
        else:
            if pv.points.size == 0:
                continue
            origin = tuple(int(v) for v in pv.points.min(0))
            span = [int(pv.points[:, d].max()) - origin[d] + 1 for d in range(ndim)]
            member = np.zeros(span, bool)
            member[tuple((pv.points - np.asarray(origin)).T)] = True
            ok = np.ones((P, E), bool)
            idx = []
            for d in range(ndim):
                r = g[d] - origin[d]
                ok &= (r >= 0) & (r < span[d])
                idx.append(np.clip(r, 0, span[d] - 1))
            inside = ok & member[tuple(idx)]
        inside &= in_tile[None, :]
        if not inside.any():
            continue
        base = np.ascontiguousarray(iv_full(pv.base, axes)).reshape(-1)               # element index of the partition
        a = np.broadcast_to(base[:, None], (P, E)).copy()
        for d in range(ndim):
            a += (g[d] - origin[d]) * int(pv.strides[d])
        if tr.arena is not None:
            # as in a direct access, what lies past the end of the allocation the partition starts in
            # reads as zero and is not written (ktir_cpu/memory.py:218-300)
            for b0 in np.unique(base[inside.any(1)]):
                al = tr.arena.find(int(b0) * bpe)
                if al is None:
                    raise ValueError(f"Read from unmapped address 0x{int(b0) * bpe:x}")
                rows = base == b0
                inside[rows] &= (a[rows] >= al.byte_lo // bpe) & (a[rows] < al.byte_hi // bpe)
        hits += inside
        addr = np.where(inside, a, addr)
        part = np.where(inside, pi, part)
    if not (hits > 0).any(1).all():
        p0 = int(np.flatnonzero(~(hits > 0).any(1))[0])
        gb = tuple(int(x[d][p0]) for d in range(ndim))
        raise ValueError(f"distributed_tile_access: no partition covers access region global_base={gb} shape={tuple(shape)}")
    multi = bool((hits > 1).any())
    plain = _as_strided_box(tr, dv, addr, local, tuple(shape), axes, multi)
    if plain is not None:
        return plain
    return TableAccess(dv.dtype, tuple(shape), addr.reshape(axes + (E,)), multi, part.reshape(axes + (E,)))


def _as_strided_box(tr, dv: DistView, addr: np.ndarray, local: np.ndarray, shape, axes, multi: bool):
    """The common case — every point's tile lies whole inside one partition, all with the same layout,
    in one allocation — is an ordinary strided access tile, which the fused kernels understand."""
    if multi or addr.size == 0 or (addr < 0).any():
        return None
    rel = addr - addr[:, :1]
    if not (rel == rel[0]).all():
        return None
    strides = []
    for d, n_ in enumerate(shape):
        if n_ > 1:
            unit = np.zeros(len(shape), np.int64)
            unit[d] = 1
            strides.append(int(rel[0][int((local == unit).all(1).argmax())]))
        else:
            strides.append(int(dv.parts[0].strides[d]))
    if not ((local * np.asarray(strides, np.int64)).sum(1) == rel[0]).all():
        return None
    if tr.arena is not None:
        bpe = bytes_per_elem(dv.dtype)
        names = {getattr(tr.arena.find(int(a0) * bpe), "name", None) for a0 in np.unique(addr[:, 0])}
        if len(names) != 1:
            return None
    origin = addr[:, 0].reshape(axes) if axes else int(addr[0, 0])
    view = View(int(addr[:, 0].min()), tuple(dv.shape), tuple(strides), dv.dtype, "global")
    return Access(view, origin, shape, tuple(strides))


@rule("ktdp.construct_access_tile")
def _access_tile(tr, op, scope):
    view = tr.get(scope, op.operands[0])
    idx = [tr.get(scope, i) if isinstance(i, str) else i for i in op.attrs["indices"]]
    bm = op.attrs.get("base_map")
    coords = bm.eval(idx) if isinstance(bm, AffineMap) else idx
    if isinstance(view, DistView):
        aset_d: AffineSet = op.attrs.get("set")
        if aset_d is not None and aset_d.n_syms:
            raise NotImplementedError("construct_access_tile: symbolic access_tile_set is not yet supported")
        return _distributed_access(tr, view, coords, tuple(op.attrs["shape"]), aset_d, op.attrs.get("order"))
    if not isinstance(view, View):
        raise Unsupported("construct_access_tile on a value that is not a memory view")
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
    if box is not None:
        # a box walked in another order: its points, row-major, through the order map — whole columns at once
        lo, hi = box
        cols = np.indices(tuple(h - l for l, h in zip(lo, hi)), dtype=np.int64).reshape(len(lo), -1)
        cols = [c + l for c, l in zip(cols, lo)]
        mapped = order.eval(cols)
        coords_arr = np.stack([np.broadcast_to(np.asarray(m, np.int64), cols[0].shape) for m in mapped], 1)
        return Access(view, off, shape, tuple(view.strides), np.ascontiguousarray(coords_arr))
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
        return Node("iload", rshape, at.view.dtype, (), {"access": at, "axes": tuple(tr.axes), "stores_before": len(tr.stores)})
    if isinstance(at, TableAccess):
        return Node("tload", rshape if int(np.prod(rshape)) == int(np.prod(at.shape)) else tuple(at.shape), at.dtype, (),
                    {"access": at, "axes": tuple(tr.axes), "stores_before": len(tr.stores)})
    if not isinstance(at, Access):
        raise Unsupported("ktdp.load from a value that is not an access tile")
    shape = tuple(at.shape) if at.coords is None else rshape
    return Node("load", shape, at.view.dtype, (), {"access": at, "axes": tuple(tr.axes), "stores_before": len(tr.stores)})


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
    elif isinstance(at, TableAccess):
        if at.multi:
            raise Unsupported("store through a distributed view whose partitions overlap")
    elif not isinstance(at, Access):
        raise Unsupported("ktdp.store to a value that is not an access tile")
    tr.stores.append(Store(value, at, tuple(tr.axes),
                           None if tr.active is None else tr.active.copy(),
                           len(tr.stores), tuple(tr.loop_path)))
    return None

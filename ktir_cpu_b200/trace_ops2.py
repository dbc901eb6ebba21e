"""Trace rules for tensor / linalg / scf / ktdp ops (second half of the table)."""
from __future__ import annotations

from typing import Any, Dict, List

import numpy as np

from .affine import AffineMap, AffineSet
from .dtypes import canon
from .ir import Op
from .trace import (MAX_UNROLL, Access, IndirectAccess, LoopInfo, Node, Store, Tracer, Unsupported,
                    View, _Yield, is_iv, iv_align, iv_bin, iv_full, iv_uniform)
from .trace_ops import (TABLE, _as_operand, cast, const_node, ew, is_fscalar, is_node, param_node, rule)


# ---- tensor dialect --------------------------------------------------------------
@rule("tensor.empty")
def _empty(tr, op, scope):
    ty = op.result_types[0]
    n = const_node(0.0 if ty.dtype in ("f16", "f32") else 0, ty.shape, ty.dtype)
    n.attrs["empty"] = True
    return n


@rule("tensor.splat")
def _splat(tr, op, scope):
    s = tr.get(scope, op.operands[0])
    ty = op.result_types[0]
    shape, dtype = tuple(ty.shape), canon(ty.dtype)
    if is_node(s):
        src = s if s.shape == () else Node("extract", (), s.dtype, (s,), {"index": (0,) * len(s.shape)})
        if src.dtype in ("i32", "i64"):
            src, dtype = cast(src, "i32"), "i32"
        else:
            src = cast(src, dtype)
        return Node("bcast", shape, dtype, (src,), {"dims": list(range(len(shape)))})
    if isinstance(s, np.ndarray):
        return Node("bcast", shape, "i32", (cast(param_node(s), "i32"),), {"dims": list(range(len(shape)))})
    if isinstance(s, (int, np.integer)) and not isinstance(s, (bool, np.bool_)):
        return const_node(int(s), shape, "i32")
    return const_node(float(np.asarray(s, dtype={"f16": np.float16, "f32": np.float32}.get(dtype, np.float32))),
                      shape, dtype)


@rule("tensor.extract")
def _extract(tr, op, scope):
    src = tr.get(scope, op.operands[0])
    if not is_node(src):
        return src
    idx = []
    for i in op.attrs.get("indices", []):
        v = tr.get(scope, i) if isinstance(i, str) else i
        u = iv_uniform(v)
        if u is None:
            raise Unsupported("tensor.extract with a per-core index")
        idx.append(u)
    if not idx:
        idx = [0] * len(src.shape)
    return Node("extract", (), src.dtype, (src,), {"index": tuple(idx)})


@rule("tensor.collapse_shape", "tensor.expand_shape", "tensor.reshape")
def _reshape(tr, op, scope):
    src = tr.get(scope, op.operands[0])
    if not is_node(src):
        return src
    return Node("reshape", tuple(op.result_types[0].shape), src.dtype, (src,), {})


# ---- linalg ------------------------------------------------------------------------
def _combiner_of(op: Op):
    if "combiner" in op.attrs:
        return op.attrs["combiner"]
    if not op.regions:
        return "arith.addf"
    reg = op.regions[0]
    body = [o for o in reg.ops if o.name != "linalg.yield"]
    if len(body) == 1 and len(body[0].operands) == 2:
        names = reg.arg_names or list(body[0].operands)
        if set(body[0].operands) == set(names[:2]):
            return body[0].name
    return None


_CANON_COMB = {"arith.maxf": "arith.maximumf", "arith.minf": "arith.minimumf"}


@rule("linalg.reduce")
def _reduce(tr, op, scope):
    tile = tr.get(scope, op.operands[0])
    outs_name = op.operands[1] if len(op.operands) > 1 else None
    outs = tr.get(scope, outs_name) if outs_name else None
    if not is_node(tile):
        result = tile
    else:
        comb = _combiner_of(op)
        if comb is None:
            return _reduce_by_region(tr, op, scope, tile, outs_name, outs)
        comb = _CANON_COMB.get(comb, comb)
        dims = op.attrs.get("dimensions")
        if dims is None:
            shape = ()
        else:
            shape = tuple(s for i, s in enumerate(tile.shape) if i not in dims)
        result = Node("reduce", shape, tile.dtype, (tile,),
                      {"op": comb, "dims": None if dims is None else tuple(sorted(dims))})
        if tr.lx is not None:
            _reduce_transients(tr, op, tile, dims, shape, outs)
        if is_node(outs):
            result = ew(comb, [result, outs], dtype=tile.dtype)
    if outs_name and result is not None:
        scope[outs_name] = result
        if tr.lx is not None and is_node(result):
            tr.lx.set_value(outs_name, result, tr.cores_active())      # the result is bound under the outs name too
    return result


def _slice(node: Node, dim: int, lo: int, hi: int) -> Node:
    shape = list(node.shape)
    shape[dim] = hi - lo
    return Node("slice", tuple(shape), node.dtype, (node,), {"dim": dim, "lo": lo, "hi": hi})


def _reduce_by_region(tr, op, scope, tile: Node, outs_name, outs):
    """A combiner region of several ops (e.g. max written as cmpf + select): the pairwise fold of the
    reference spelled out in the DAG (ktir_cpu/dialects/linalg_ops.py:86-133) — per level the two
    halves of the reduced axis go through the region, an odd leftover slice is carried to the next
    level — followed by the combine with ``outs``.  The region's ops are charged by the level-wise
    latency and scratchpad replays that every reduce gets, so it is traced here without them."""
    reg = op.regions[0]
    names = list(reg.arg_names)
    if len(names) < 2:
        raise ValueError("linalg.reduce: combiner region needs two block arguments")

    def combine(lhs, rhs):
        inner = dict(scope)
        inner[names[0]], inner[names[1]] = lhs, rhs
        y = tr.trace_ops(reg.ops, inner)
        if not isinstance(y, _Yield) or not y.values:
            raise TypeError("linalg.reduce: combiner region did not yield a value")
        v = y.values[0]
        if not is_node(v):
            raise Unsupported("linalg.reduce whose combiner region yields a non-tile value")
        return v if tuple(v.shape) == tuple(lhs.shape) else Node("bcast", tuple(lhs.shape), v.dtype, (v,), {"numpy": True})

    dims = op.attrs.get("dimensions")
    saved = tr.latency, tr.lx
    tr.latency = tr.lx = None
    try:
        acc = tile
        if dims is None:
            acc = Node("reshape", (int(np.prod(tile.shape, dtype=np.int64)),), tile.dtype, (tile,), {})
            fold = [0]
        else:
            fold = sorted(dims, reverse=True)
        for d in fold:
            n = acc.shape[d]
            while n > 1:
                half = n // 2
                combined = combine(_slice(acc, d, 0, half), _slice(acc, d, half, 2 * half))
                if n % 2:
                    tail = _slice(acc, d, 2 * half, n)
                    shape = list(combined.shape)
                    shape[d] = half + 1
                    combined = Node("concat", tuple(shape), combined.dtype, (combined, tail), {"dim": d})
                acc = combined
                n = acc.shape[d]
        out_shape = () if dims is None else tuple(s_ for i, s_ in enumerate(tile.shape) if i not in dims)
        result = Node("reshape", out_shape, tile.dtype, (acc,), {})
        if is_node(outs):
            result = combine(result, outs)
    finally:
        tr.latency, tr.lx = saved
    if tr.lx is not None:
        _reduce_transients(tr, op, tile, dims, out_shape, outs)
    if outs_name:
        scope[outs_name] = result
        if tr.lx is not None:
            tr.lx.set_value(outs_name, result, tr.cores_active())
    return result


def _reduce_transients(tr, op, tile, dims, out_shape, outs):
    """Replay the scratchpad traffic of the pairwise fold (ktir_cpu/dialects/linalg_ops.py:61-133,
    160-246): every level binds its two halves and runs the combiner ops on them in a scope of its
    own, and the folded value is combined once more with ``outs``.  The shorthand form
    (``linalg.reduce { arith.addf }``) runs a synthesised one-op region whose names no use count
    knows, so nothing in it is released early."""
    lx = tr.lx
    cores = tr.cores_active()
    if op.regions and op.regions[0].ops:
        reg = op.regions[0]
        body = reg.ops
        names = list(reg.arg_names) or list(body[0].operands)
    else:
        names = ["__reduce_in__", "__reduce_acc__"]
        body = [Op(op.attrs.get("combiner") or "arith.addf", ["__reduce_combined__"], list(names)),
                Op("linalg.yield", [], ["__reduce_combined__"])]

    def run(shape, rhs_tile=None):
        lx.push()
        try:
            lx.set_value(names[0], Node("held", tuple(shape), tile.dtype), cores)
            if len(names) > 1:
                lx.set_value(names[1], rhs_tile if rhs_tile is not None else Node("held", tuple(shape), tile.dtype), cores)
            for o in body:
                for n in o.operands:
                    lx.fetch(n)
                for r in o.results:
                    lx.set_value(r, Node("held", tuple(shape), tile.dtype), cores)
        finally:
            lx.pop()
    shape = list(tile.shape)
    if dims is None:
        shape, fold = [int(np.prod(shape, dtype=np.int64))], [0]
    else:
        fold = sorted(dims, reverse=True)
    for d in fold:
        n = shape[d]
        while n > 1:
            half = n // 2
            lvl = list(shape)
            lvl[d] = half
            run(lvl)
            n = half + (n % 2)
        shape[d] = 1
    if is_node(outs) and len(out_shape):
        run(out_shape, outs)


@rule("linalg.fill")
def _fill(tr, op, scope):
    s, out = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if is_node(s) or isinstance(s, np.ndarray):
        raise Unsupported("linalg.fill with a non-constant scalar")
    return const_node(float(s), out.shape, out.dtype)


@rule("linalg.broadcast")
def _broadcast(tr, op, scope):
    inp, out = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    dims = sorted(op.attrs.get("dimensions", []))
    return Node("bcast", tuple(out.shape), inp.dtype, (inp,), {"dims": dims})


@rule("linalg.transpose")
def _transpose(tr, op, scope):
    inp = tr.get(scope, op.operands[0])
    perm = op.attrs.get("permutation")
    if perm is None:
        raise ValueError("linalg.transpose: missing permutation attribute")
    return Node("transpose", tuple(inp.shape[i] for i in perm), inp.dtype, (inp,), {"perm": tuple(perm)})


@rule("linalg.add", "linalg.max")
def _named_bin(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if not is_node(a) or not is_node(b):
        raise TypeError(f"{op.name}: ins must be Tiles")
    return ew("arith.addf" if op.name == "linalg.add" else "arith.maximumf", [a, b], dtype=a.dtype)


@rule("linalg.matmul", "linalg.batch_matmul")
def _matmul(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    acc = tr.get(scope, op.operands[2]) if len(op.operands) > 2 else None
    shape = tuple(a.shape[:-1]) + (b.shape[-1],)
    args = (a, b) + ((acc,) if is_node(acc) else ())
    n = Node("matmul", shape, acc.dtype if is_node(acc) else a.dtype, args,
             {"batched": op.name.endswith("batch_matmul"), "prod_dtype": a.dtype})
    if is_node(acc):
        scope[op.operands[2]] = n
        if tr.lx is not None and not tr.lx.is_free(acc):
            tr.lx.same_tile(n, acc)              # accumulated in place: the result is the outs tile
    return n


@rule("linalg.index")
def _index(tr, op, scope):
    shape = scope["__linalg_shape__"]
    d = op.attrs["dim"]
    rs = [1] * len(shape)
    rs[d] = shape[d]
    return Node("iota", tuple(rs), "i64", (), {"dim": d})


@rule("linalg.yield", "scf.yield", "tensor.yield")
def _yield(tr, op, scope):
    return _Yield([tr.get(scope, n) for n in op.operands])


def _map_input(node: Node, m: AffineMap, iter_shape) -> Node:
    """View an input through a projection indexing map (linalg_ops.py:398-419)."""
    if not all(e[0] == "dim" for e in m.exprs):
        raise Unsupported("linalg.generic with a non-projection indexing map")
    plain = [e[1] for e in m.exprs]
    if plain != sorted(plain):
        perm = tuple(plain.index(d) for d in sorted(plain))
        node = Node("transpose", tuple(node.shape[i] for i in perm), node.dtype, (node,), {"perm": perm})
        plain = sorted(plain)
    if len(plain) == len(iter_shape):
        return node
    missing = [d for d in range(len(iter_shape)) if d not in plain]
    return Node("bcast", tuple(iter_shape), node.dtype, (node,), {"dims": missing})


@rule("linalg.generic")
def _generic(tr, op, scope):
    n_ins = op.attrs["n_ins"]
    maps = op.attrs.get("indexing_maps", [])
    iters = op.attrs.get("iterator_types") or []
    ins = [tr.get(scope, o) for o in op.operands[:n_ins]]
    outs = tr.get(scope, op.operands[n_ins])
    if any(t == "reduction" for t in iters):
        return _generic_reduction(tr, op, scope, ins, outs, maps, [i for i, t in enumerate(iters) if t == "reduction"])
    if not is_node(outs):
        raise TypeError(f"linalg.generic: outs must be a Tile, got {type(outs)}")
    reg = op.regions[0]
    if not reg.arg_names:
        raise ValueError("linalg.generic: cannot determine bb0 argument names")
    inner = dict(scope)
    inner["__linalg_shape__"] = tuple(outs.shape)
    held = []          # every tile input is gathered into the iteration shape, outs is copied: new tiles in the body's scope
    for i, (v, m) in enumerate(zip(ins, maps[:n_ins])):
        inner[reg.arg_names[i]] = _map_input(v, m, outs.shape) if is_node(v) else v
        if is_node(v):
            held.append((reg.arg_names[i], Node("held", tuple(outs.shape), v.dtype)))
    if n_ins < len(reg.arg_names):
        inner[reg.arg_names[n_ins]] = outs
        held.append((reg.arg_names[n_ins], Node("held", tuple(outs.shape), outs.dtype)))
    r = tr.trace_region(reg.ops, inner, held)
    v = r.values[0] if isinstance(r, _Yield) else None
    if is_node(v):
        v = cast(v, outs.dtype)
        if tuple(v.shape) != tuple(outs.shape):
            v = Node("bcast", tuple(outs.shape), v.dtype, (v,), {"dims": [], "numpy": True})
        return v
    if isinstance(v, np.ndarray):
        raise Unsupported("linalg.generic yielding a per-core scalar")
    return const_node(v, outs.shape, outs.dtype)


_GENERIC_IDENTITY = {"arith.addf": 0.0, "arith.addi": 0, "arith.mulf": 1.0, "arith.muli": 1,
                     "arith.maxf": float("-inf"), "arith.maximumf": float("-inf"),
                     "arith.minf": float("inf"), "arith.minimumf": float("inf")}


def _generic_reduction(tr, op, scope, ins, outs, maps, red):
    """``linalg.generic`` with reduction iterators (ktir_cpu/dialects/linalg_ops.py:466-585): the body
    runs once over the full iteration space with the ``outs`` argument bound to the combiner's identity,
    its result is folded pairwise along the reduction dims (rightmost first) by the combiner — the op
    that produces the yielded value from the ``outs`` argument — and the fold is combined with the real
    ``outs``."""
    n_ins = op.attrs["n_ins"]
    if not is_node(outs):
        raise TypeError(f"linalg.generic: outs must be a Tile, got {type(outs)}")
    reg = op.regions[0]
    if not reg.arg_names:
        raise ValueError("linalg.generic: cannot determine bb0 argument names")
    extent = [None] * maps[0].n_dims
    shapes = [v.shape for v in ins if is_node(v)] + [outs.shape]
    for m, shp in zip(maps, shapes):
        for k, e in enumerate(m.exprs):
            if e[0] == "dim" and extent[e[1]] is None:
                extent[e[1]] = shp[k]
    if any(e is None for e in extent):
        raise ValueError(f"linalg.generic: cannot infer extent for dims {[i for i, e in enumerate(extent) if e is None]}")
    iter_shape = tuple(int(e) for e in extent)
    outs_arg = reg.arg_names[n_ins] if n_ins < len(reg.arg_names) else None
    yop = next((o for o in reg.ops if o.name == "linalg.yield"), None)
    comb = None
    if yop is not None and yop.operands:
        comb = next((o for o in reg.ops if o.results and o.results[0] == yop.operands[0] and outs_arg in o.operands), None)
    if comb is None:
        raise ValueError(f"linalg.generic: cannot identify combiner op for reduction (outs block-arg '{outs_arg}' "
                         "not found in body ops)")
    if comb.name not in _GENERIC_IDENTITY:
        raise ValueError(f"linalg.generic: unsupported combiner '{comb.name}' for reduction; "
                         f"supported: {list(_GENERIC_IDENTITY)}")
    inner = dict(scope)
    inner["__linalg_shape__"] = iter_shape
    held = []
    for i, (v, m) in enumerate(zip(ins, maps[:n_ins])):
        inner[reg.arg_names[i]] = _map_input(v, m, iter_shape) if is_node(v) else v
        if is_node(v):
            held.append((reg.arg_names[i], Node("held", iter_shape, v.dtype)))
    inner[outs_arg] = const_node(_GENERIC_IDENTITY[comb.name], iter_shape, outs.dtype)
    held.append((outs_arg, Node("held", iter_shape, outs.dtype)))
    r = tr.trace_region(reg.ops, inner, held)
    v = r.values[0] if isinstance(r, _Yield) else None
    if isinstance(v, np.ndarray):
        raise Unsupported("linalg.generic yielding a per-core scalar")
    if not is_node(v):
        v = const_node(v, iter_shape, outs.dtype)
    elif tuple(v.shape) != iter_shape:
        v = Node("bcast", iter_shape, v.dtype, (v,), {"dims": [], "numpy": True})
    name = _CANON_COMB.get(comb.name, comb.name)
    out_shape = tuple(s_ for i, s_ in enumerate(iter_shape) if i not in red)
    folded = Node("reduce", out_shape, v.dtype, (v,), {"op": name, "dims": tuple(sorted(red))})
    fake = Op("linalg.reduce", [], [], {"combiner": comb.name, "dimensions": list(red)})
    if tr.lx is not None:
        _reduce_transients(tr, fake, v, list(red), out_shape, outs)
    if tr.latency is not None:
        tr.latency._reduce(tr, fake, [v, outs])
    result = ew(name, [cast(folded, outs.dtype), outs], dtype=outs.dtype)
    if tuple(result.shape) != tuple(outs.shape):
        result = Node("reshape", tuple(outs.shape), result.dtype, (result,), {})
    return result


# ---- control flow -------------------------------------------------------------------
def _loop_operand(tr, op, scope, k, key):
    name = op.operands[k]
    if name.startswith("__const_"):
        return op.attrs["const_operands"][key]
    return tr.get(scope, name)


def _has_op(ops, names) -> bool:
    from .ir import walk
    return any(o.name in names for o in walk(ops))


@rule("scf.for")
def _for(tr: Tracer, op: Op, scope):
    lb = _loop_operand(tr, op, scope, 0, "lb")
    ub = _loop_operand(tr, op, scope, 1, "ub")
    step = _loop_operand(tr, op, scope, 2, "step")
    if not (is_iv(lb) and is_iv(ub) and is_iv(step)):
        raise Unsupported("scf.for bounds must be integer values")
    step = iv_bin(np.maximum, step, 1) if isinstance(step, np.ndarray) else max(int(step), 1)
    span = iv_bin(lambda a, b: a - b, ub, lb)
    trips = iv_bin(lambda s, st: np.maximum(-((-s) // st), 0), span, step)
    trips_full = iv_full(trips, tuple(tr.axes))
    if tr.active is not None:
        trips_full = np.where(tr.active, trips_full, 0)
    T = int(trips_full.max()) if trips_full.size else 0
    reg = op.regions[0]
    iv_name, iter_names = reg.arg_names[0], reg.arg_names[1:]
    inits = [tr.get(scope, n) for n in op.operands[3:]]

    if not iter_names and not tr.unroll_loops:
        if T == 0:
            return None
        depth = len(tr.axes)
        k = np.arange(T, dtype=np.int64)
        lb_f = iv_full(lb, tuple(tr.axes))[..., None]
        st_f = iv_full(step, tuple(tr.axes))[..., None]
        ivs = lb_f + k.reshape((1,) * depth + (T,)) * st_f
        mask = k.reshape((1,) * depth + (T,)) < trips_full[..., None]
        saved_axes, saved_active = list(tr.axes), tr.active
        tr.axes.append(T)
        tr.active = None if mask.all() else mask
        tr._loop_counter += 1
        tr.loop_path.append(tr._loop_counter)
        inner = dict(scope)
        inner[iv_name] = ivs
        tr.trace_region(reg.ops, inner)
        tr.loop_path.pop()
        tr.axes, tr.active = saved_axes, saved_active
        return None

    # loop-carried values
    tmin = int(trips_full.min()) if trips_full.size else 0
    live = trips_full if tr.active is None else trips_full[tr.active]
    if live.size and int(live.min()) != T:
        raise Unsupported("scf.for traced iteration by iteration (iter_args, or iterations that touch each other's "
                          "memory) and a trip count that differs between cores")
    tile_carried = any(is_node(v) for v in inits)
    if tile_carried and _has_op(reg.ops, ("linalg.matmul", "linalg.batch_matmul")) and T >= 1:
        return _symbolic_loop(tr, op, scope, lb, step, T, inits)
    if T > MAX_UNROLL:
        raise Unsupported(f"scf.for traced iteration by iteration with {T} iterations")
    vals = list(inits)
    _lx_bind_carried(tr, iter_names, [Node("held", v.shape, v.dtype) if is_node(v) else v for v in vals])
    for k in range(T):
        inner = dict(scope)
        inner[iv_name] = iv_bin(lambda a, b: a + b, lb, iv_bin(lambda s, kk: s * kk, step, k))
        for n, v in zip(iter_names, vals):
            inner[n] = v
        r = tr.trace_region(reg.ops, inner)
        if isinstance(r, _Yield):
            vals = list(r.values)
            _lx_bind_carried(tr, iter_names, vals)
    if not op.results:
        return None
    return vals[0] if len(vals) == 1 else tuple(vals)


def _lx_bind_carried(tr: Tracer, names, values):
    """Loop-carried tiles live in the scope AROUND the loop: bound there before the first iteration
    (private copies of the inits) and re-bound there after every iteration's body scope has been
    left (ktir_cpu/ops/control_ops.py:56-98, 160-182) — so the body can never release them early."""
    if tr.lx is None:
        return
    cores = tr.cores_active()
    for n, v in zip(names, values):
        if is_node(v):
            tr.lx.set_value(n, v, cores)


def _symbolic_loop(tr: Tracer, op: Op, scope, lb, step, T: int, inits):
    """Trace the body once with the trip count as an extra (sequential) axis."""
    reg = op.regions[0]
    iv_name, iter_names = reg.arg_names[0], reg.arg_names[1:]
    depth = len(tr.axes)
    k = np.arange(T, dtype=np.int64)
    ivs = (iv_full(lb, tuple(tr.axes))[..., None]
           + k.reshape((1,) * depth + (T,)) * iv_full(step, tuple(tr.axes))[..., None])
    saved_axes, n_stores = list(tr.axes), len(tr.stores)
    tr.axes.append(T)
    inner = dict(scope)
    inner[iv_name] = ivs
    placeholders = []
    for i, (n, v) in enumerate(zip(iter_names, inits)):
        if not is_node(v):
            raise Unsupported("scf.for carrying both tiles and scalars around a matmul")
        ph = Node("iter", v.shape, v.dtype, (), {"index": i})
        placeholders.append(ph)
        inner[n] = ph
    _lx_bind_carried(tr, iter_names, placeholders)
    r = tr.trace_region(reg.ops, inner)
    tr.axes = saved_axes
    if len(tr.stores) != n_stores:
        raise Unsupported("ktdp.store inside an scf.for that carries a matmul accumulator")
    if not isinstance(r, _Yield):
        raise ValueError("scf.for with iter_args must end in scf.yield")
    info = LoopInfo(T, depth, list(inits), list(r.values))
    for ph in placeholders:
        ph.attrs["loop"] = info
    results = [Node("loopres", v.shape, v.dtype, (), {"loop": info, "index": i})
               for i, v in enumerate(inits)]
    _lx_bind_carried(tr, iter_names, list(r.values))
    if tr.lx is not None:
        for res, y in zip(results, r.values):
            if is_node(y):
                tr.lx.same_tile(res, y)          # the loop's results are the tiles of the last yield
    if not op.results:
        return None
    return results[0] if len(results) == 1 else tuple(results)


@rule("scf.if")
def _if(tr, op, scope):
    cond = tr.get(scope, op.operands[0])
    if is_node(cond):
        raise Unsupported("scf.if on a tile condition")
    if isinstance(cond, np.ndarray):
        if op.results:
            raise Unsupported("scf.if with results on a per-core condition")
        full = iv_full(cond.astype(np.int64), tuple(tr.axes)).astype(bool)
        saved = tr.active
        for reg, m in zip(op.regions, (full, ~full)):
            tr.active = m if saved is None else (saved & m)
            if tr.active.any():
                tr.trace_region(reg.ops, dict(scope))
        tr.active = saved
        return None
    reg = op.regions[0] if cond else (op.regions[1] if len(op.regions) > 1 else None)
    if reg is None:
        return None
    r = tr.trace_region(reg.ops, dict(scope))
    if isinstance(r, _Yield) and r.values:
        return r.values[0] if len(r.values) == 1 else tuple(r.values)
    return None


@rule("return", "func.return")
def _return(tr, op, scope):
    return None

"""Per-op trace rules: how each KTIR op extends the whole-grid trace.

Scalar semantics mirror the reference handlers so that host-side index math
gives the same numbers: integer ops act on Python ints / int64 arrays
(ktir_cpu/dialects/arith_ops.py:98-135), scalar float binops are coerced through
``np.float16`` (ktir_cpu/dialects/_helpers.py:39-54), ``tensor.splat`` of an
integer makes an i32 tile (ktir_cpu/dialects/tensor_ops.py:57-85).
"""
from __future__ import annotations

import operator
from typing import Any, Dict, List

import numpy as np

from .affine import AffineMap
from .dtypes import canon
from .ir import Op
from .trace import (MAX_UNROLL, Access, IndirectAccess, LoopInfo, Node, Store, Tracer, Unsupported,
                    View, _Yield, is_iv, iv_align, iv_bin, iv_full, iv_uniform)

TABLE: Dict[str, Any] = {}


def rule(*names):
    def deco(fn):
        for n in names:
            TABLE[n] = fn
        return fn
    return deco


def is_node(v):
    return isinstance(v, Node)


def is_fscalar(v):
    return isinstance(v, (float, np.floating))


def const_node(value, shape, dtype) -> Node:
    return Node("const", tuple(shape), canon(dtype), (), {"value": value})


def param_node(values, dtype="i64") -> Node:
    """A per-iteration-point scalar (an integer value over the iteration space)."""
    return Node("param", (), dtype, (), {"values": values})


def _np_result_dtype(a: str, b: str) -> str:
    order = ["i1", "i32", "i64", "f16", "f32"]
    if a == b:
        return a
    if a in ("f16", "f32") and b in ("f16", "f32"):
        return "f32"
    return a if order.index(a) > order.index(b) else b


def _bshape(a, b):
    return tuple(np.broadcast_shapes(tuple(a), tuple(b)))


def ew(opname: str, args: List[Node], dtype=None, shape=None, **attrs) -> Node:
    if shape is None:
        shape = ()
        for a in args:
            shape = _bshape(shape, a.shape)
    if dtype is None:
        dtype = args[0].dtype
        for a in args[1:]:
            dtype = _np_result_dtype(dtype, a.dtype)
    return Node("ew", tuple(shape), dtype, tuple(args), dict(op=opname, **attrs))


def cast(node: Node, dtype: str) -> Node:
    dtype = canon(dtype)
    if node.dtype == dtype:
        return node
    return Node("cast", node.shape, dtype, (node,), {})


# ---- float arithmetic -----------------------------------------------------
_PYF = {"arith.addf": operator.add, "arith.subf": operator.sub, "arith.mulf": operator.mul,
        "arith.divf": operator.truediv, "arith.remf": operator.mod}


def _as_operand(v, like: Node, coerce16: bool) -> Node:
    if is_node(v):
        return v
    if isinstance(v, np.ndarray):
        return cast(param_node(v), like.dtype)
    val = float(np.float16(v)) if coerce16 else float(v)
    return const_node(val, (), like.dtype if like.dtype in ("f16", "f32") else "f32")


@rule(*_PYF)
def _float_bin(tr: Tracer, op: Op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if not is_node(a) and not is_node(b):
        if isinstance(a, np.ndarray) or isinstance(b, np.ndarray):
            raise Unsupported(f"{op.name} on per-core scalar values")
        with np.errstate(all="ignore"):
            return np.float16(_PYF[op.name](np.float16(a), np.float16(b)))
    like = a if is_node(a) else b
    na, nb = _as_operand(a, like, True), _as_operand(b, like, True)
    if na.shape == () and is_node(a) and not nb.shape == ():
        na = cast(na, "f16") if na.dtype == "f32" else na     # scalar operands pass through np.float16
    if nb.shape == () and is_node(b) and not na.shape == ():
        nb = cast(nb, "f16") if nb.dtype == "f32" else nb
    dtype = like.dtype if not (is_node(a) and is_node(b)) else None
    return ew(op.name, [na, nb], dtype=dtype)


@rule("arith.maxf", "arith.maximumf", "arith.maxnumf", "arith.minf", "arith.minimumf", "arith.minnumf")
def _minmax(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if not is_node(a) and not is_node(b):
        raise Unsupported(f"{op.name} on scalars")
    like = a if is_node(a) else b
    name = {"arith.maxf": "arith.maximumf", "arith.minf": "arith.minimumf"}.get(op.name, op.name)
    return ew(name, [_as_operand(a, like, False), _as_operand(b, like, False)])


@rule("arith.negf", "arith.absf", "math.absf")
def _negabs(tr, op, scope):
    a = tr.get(scope, op.operands[0])
    name = "arith.negf" if op.name == "arith.negf" else "math.absf"
    if is_node(a):
        return ew(name, [a])
    return -a if name == "arith.negf" else abs(a)


_MATH = {"math.exp": np.exp, "math.sqrt": np.sqrt, "math.rsqrt": lambda x: 1.0 / np.sqrt(x),
         "math.log": np.log, "math.log2": np.log2, "math.log1p": np.log1p, "math.tanh": np.tanh,
         "math.sin": np.sin, "math.cos": np.cos, "math.ceil": np.ceil, "math.floor": np.floor,
         "math.erf": None}


_ERF_C = (0.254829592, -0.284496736, 1.421413741, -1.453152027, 1.061405429)


def _erf_tile(x: Node) -> Node:
    """``math.erf`` of a tile as the reference evaluates it: the Abramowitz & Stegun 7.1.26 formula
    written with NumPy ufuncs on the tile's own dtype (ktir_cpu/ops/math_ops.py:99-111), so every
    step — and every constant — is rounded to that dtype.  Expanded into the same chain of
    elementwise nodes: sign(x) * (1 - poly(t) * exp(-|x| * |x|)), t = 1 / (1 + 0.3275911 |x|)."""
    c = lambda v: const_node(v, (), x.dtype)     # noqa: E731  (rounded to the tile dtype when lowered)
    a = ew("math.absf", [x])
    t = ew("arith.divf", [c(1.0), ew("arith.addf", [c(1.0), ew("arith.mulf", [c(0.3275911), a])])])
    inner = ew("arith.mulf", [t, c(_ERF_C[4])])
    for k in (3, 2, 1, 0):
        inner = ew("arith.mulf", [t, ew("arith.addf", [c(_ERF_C[k]), inner])])
    e = ew("math.exp", [ew("arith.mulf", [ew("arith.negf", [a]), a])])
    return ew("arith.mulf", [ew("math.sign", [x]), ew("arith.subf", [c(1.0), ew("arith.mulf", [inner, e])])])


@rule(*_MATH)
def _math_unary(tr, op, scope):
    a = tr.get(scope, op.operands[0])
    if is_node(a):
        if op.name == "math.erf":
            return _erf_tile(a)
        if op.name == "math.rsqrt":
            # 1.0 / np.sqrt(x) on the tile dtype (ktir_cpu/ops/math_ops.py:38-41): two ops, two roundings
            return ew("arith.divf", [const_node(1.0, (), a.dtype), ew("math.sqrt", [a])])
        return ew(op.name, [a])
    if _MATH[op.name] is None or isinstance(a, np.ndarray):
        raise Unsupported(f"{op.name} on a scalar")
    cast_t = type(a) if is_fscalar(a) else float
    with np.errstate(all="ignore"):
        return cast_t(_MATH[op.name](a))


@rule("math.fma")
def _fma(tr, op, scope):
    a, b, c = (tr.get(scope, x) for x in op.operands[:3])
    if is_node(a):
        return ew("math.fma", [a, b, c], dtype=a.dtype)
    return type(a)(float(a) * float(b) + float(c))


@rule("math.powf")
def _powf(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if is_node(a):
        return ew("math.powf", [a, _as_operand(b, a, False)], dtype=a.dtype)
    return type(a)(float(a) ** float(b))


# ---- integer arithmetic ------------------------------------------------------
def _truncdiv(a, b):
    return np.trunc(a / b).astype(np.int64) if isinstance(a, np.ndarray) or isinstance(b, np.ndarray) \
        else int(a / b)


_INT = {
    "arith.addi": operator.add, "arith.subi": operator.sub, "arith.muli": operator.mul,
    "arith.divui": operator.floordiv, "arith.floordivsi": operator.floordiv,
    "arith.divsi": _truncdiv, "arith.remui": operator.mod,
    "arith.remsi": lambda a, b: a - _truncdiv(a, b) * b,
    "arith.andi": operator.and_, "arith.ori": operator.or_, "arith.xori": operator.xor,
    "arith.shli": operator.lshift, "arith.shrsi": operator.rshift, "arith.shrui": operator.rshift,
    "arith.minsi": lambda a, b: np.minimum(a, b), "arith.maxsi": lambda a, b: np.maximum(a, b),
    "arith.minui": lambda a, b: np.minimum(a, b), "arith.maxui": lambda a, b: np.maximum(a, b),
    "arith.ceildivsi": lambda a, b: -((-a) // b), "arith.ceildivui": lambda a, b: -((-a) // b),
}


def _int_operand(v, like: Node) -> Node:
    if is_node(v):
        return v
    if isinstance(v, np.ndarray):
        return param_node(v)
    return const_node(int(v), (), like.dtype)


@rule(*_INT)
def _int_bin(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    if is_node(a) or is_node(b):
        like = a if is_node(a) else b
        return ew(op.name, [_int_operand(a, like), _int_operand(b, like)], dtype=like.dtype)
    if isinstance(a, (bool, np.bool_)) or isinstance(b, (bool, np.bool_)):
        a, b = bool(a), bool(b)
        return _INT[op.name](a, b)
    return iv_bin(_INT[op.name], a, b)


_CMPI = {"slt": operator.lt, "ult": operator.lt, "sle": operator.le, "ule": operator.le,
         "sgt": operator.gt, "ugt": operator.gt, "sge": operator.ge, "uge": operator.ge,
         "eq": operator.eq, "ne": operator.ne}


@rule("arith.cmpi")
def _cmpi(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    pred = op.attrs["predicate"]
    if pred not in _CMPI:
        raise NotImplementedError(f"arith.cmpi: unsupported predicate '{pred}'")
    if is_node(a) or is_node(b):
        like = a if is_node(a) else b
        return ew("arith.cmpi", [_int_operand(a, like), _int_operand(b, like)], dtype="i1", pred=pred)
    a, b = iv_align(a, b)
    r = _CMPI[pred](a, b)
    return r if isinstance(r, np.ndarray) else bool(r)


@rule("arith.cmpf")
def _cmpf(tr, op, scope):
    a, b = tr.get(scope, op.operands[0]), tr.get(scope, op.operands[1])
    pred = op.attrs["predicate"]
    if is_node(a) or is_node(b):
        like = a if is_node(a) else b
        return ew("arith.cmpf", [_as_operand(a, like, False), _as_operand(b, like, False)],
                  dtype="i1", pred=pred)
    raise Unsupported("arith.cmpf on scalars")


@rule("arith.select")
def _select(tr, op, scope):
    c, t, f = (tr.get(scope, x) for x in op.operands[:3])
    if is_node(c):
        like = t if is_node(t) else (f if is_node(f) else None)
        if like is None:
            like = const_node(0.0, (), "f16")
        nt, nf = _as_operand(t, like, False), _as_operand(f, like, False)
        return ew("arith.select", [c, nt, nf], dtype=like.dtype)
    if isinstance(c, np.ndarray):
        # a condition that differs between cores / loop points picks between integer values
        if is_node(t) or is_node(f):
            raise Unsupported("arith.select of tiles on a per-core condition")
        if not (is_iv(t) and is_iv(f)):
            raise Unsupported("arith.select of float scalars on a per-core condition")
        n = max(x.ndim for x in (c, t, f) if isinstance(x, np.ndarray))
        grow = lambda x: x.reshape(x.shape + (1,) * (n - x.ndim)) if isinstance(x, np.ndarray) else x   # noqa: E731
        return np.where(grow(c.astype(bool)), grow(t), grow(f)).astype(np.int64)
    return t if c else f


# ---- constants and casts -------------------------------------------------------
@rule("arith.constant")
def _constant(tr, op, scope):
    v = op.attrs.get("value", 0)
    ty = op.result_types[0]
    if op.attrs.get("is_tensor"):
        if op.attrs.get("dense_list"):
            return Node("const", tuple(ty.shape), canon(ty.dtype), (), {"value": None, "list": list(v)})
        return const_node(v, ty.shape, ty.dtype)
    return v


def _cast_rule(dtype, scalar_fn):
    def fn(tr, op, scope):
        v = tr.get(scope, op.operands[0])
        if is_node(v):
            return cast(v, dtype)
        if isinstance(v, np.ndarray):
            return v
        return scalar_fn(v)
    return fn


TABLE["arith.extf"] = _cast_rule("f32", np.float32)
TABLE["arith.truncf"] = _cast_rule("f16", np.float16)
TABLE["arith.extsi"] = _cast_rule("i64", int)
TABLE["arith.extui"] = _cast_rule("i32", int)
TABLE["arith.trunci"] = _cast_rule("i32", int)
TABLE["arith.fptosi"] = _cast_rule("i32", int)


@rule("arith.sitofp", "arith.uitofp")
def _sitofp(tr, op, scope):
    v = tr.get(scope, op.operands[0])
    dt = canon(op.result_types[0].dtype) if op.result_types else "f32"
    if op.name == "arith.uitofp":
        dt = "f32"
    if is_node(v):
        return cast(v, dt)
    if isinstance(v, np.ndarray):
        raise Unsupported(f"{op.name} on a per-core scalar")
    return {"f16": np.float16, "f32": np.float32}[dt](v)


@rule("arith.index_cast", "arith.index_castui")
def _index_cast(tr, op, scope):
    v = tr.get(scope, op.operands[0])
    if is_node(v):
        raise Unsupported("arith.index_cast of a tile")
    return v if isinstance(v, np.ndarray) else int(v)


@rule("arith.bitcast")
def _bitcast(tr, op, scope):
    v = tr.get(scope, op.operands[0])
    dst = canon(op.result_types[0].dtype)
    if is_node(v):
        return Node("bitcast", v.shape, dst, (v,), {})
    if dst == "f32":
        return float(np.frombuffer(int(v).to_bytes(4, "little", signed=(v < 0)), dtype=np.float32)[0])
    if dst in ("i32",):
        return int(np.frombuffer(np.float32(v).tobytes(), dtype=np.int32)[0])
    raise NotImplementedError(f"arith.bitcast: unsupported dst_type '{dst}' for scalar")

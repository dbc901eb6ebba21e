"""Op plug-in seam: add an operation to the backend without touching it.

Counterpart of ``@register(*op_names, latency_category=..., inplace_outs=..., no_lx_charge=...)``
and ``@register_parser`` of the reference (ktir_cpu/dialects/registry.py:33-36, 98-136).  There a
handler ``(op, context, env)`` computes NumPy tiles for one core; here the function is traced once
for the whole grid, so a handler gets the same three arguments but builds its result out of
existing operations:

    @register("mylib.leaky_relu", latency_category=LatencyCategory.COMPUTE_FLOAT)
    def leaky_relu(op, context, env):
        x = context.get_value(op.operands[0])
        slope = env.constant(op.attrs.get("slope", 0.01), like=x)
        return env.elementwise("arith.maximumf", x, env.elementwise("arith.mulf", x, slope))

``context.get_value`` returns what the tracer holds for an SSA name — a tile expression, an integer
(one value, or one per core / loop point) or a float; ``context.core_id`` is the linear core id per
core.  ``env`` builds tile expressions: ``elementwise`` (any arith / math op name the backend knows),
``constant``, ``cast`` and ``execute_region``.  The result is bound to the op's result name(s) and
runs through the same fused or step-by-step kernels as built-in ops, with the same rounding
points.  ``latency_category`` feeds the latency model, ``no_lx_charge`` marks results that occupy no
scratchpad, ``inplace_outs`` says the result is the last operand's tile.

Ops of a new dialect prefix are parsed in the generic form ``%r = name %a, %b {attrs} : types``;
``register_parser`` installs a custom syntax.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Sequence

import numpy as np

from . import parser as P
from . import trace_ops as T
from .latency import CATEGORY_OF, LatencyCategory
from .trace import Node, Tracer

NO_LX_CHARGE = {"arith.constant"}
INPLACE_OUTS = {"linalg.matmul", "linalg.batch_matmul"}
_PLUGIN_PARSERS: Dict[str, Callable] = {}


class TraceContext:
    """What a handler sees of the core contexts (ktir_cpu/grid.py:41-361): SSA values and core ids."""

    def __init__(self, tracer: Tracer, scope: Dict[str, Any]):
        self._tr, self._scope = tracer, scope

    def get_value(self, name: str, *, peek: bool = False) -> Any:
        return self._tr.get(self._scope, name)

    def has_value(self, name: str) -> bool:
        return name in self._scope

    def set_value(self, name: str, value: Any):
        self._scope[name] = value

    @property
    def core_id(self) -> np.ndarray:
        return self._tr.core_base + np.arange(self._tr.ncores, dtype=np.int64)

    @property
    def num_cores(self) -> int:
        return self._tr.total_cores


class TraceEnv:
    """Builders for tile expressions (the role of ``ExecutionEnv``, which runs regions for a handler)."""

    def __init__(self, tracer: Tracer, scope: Dict[str, Any]):
        self._tr, self._scope = tracer, scope

    def elementwise(self, op_name: str, *args, **attrs) -> Node:
        nodes = [a if isinstance(a, Node) else self.constant(a, like=next(x for x in args if isinstance(x, Node)))
                 for a in args]
        return T.ew(op_name, nodes, **attrs)

    def constant(self, value, like: Node = None, shape: Sequence[int] = (), dtype: str = None) -> Node:
        return T.const_node(value, tuple(shape), dtype or (like.dtype if like is not None else "f32"))

    def cast(self, node: Node, dtype: str) -> Node:
        return T.cast(node, dtype)

    def execute_region(self, context: TraceContext, ops, bind: Dict[str, Any] = None):
        inner = dict(self._scope)
        inner.update(bind or {})
        r = self._tr.trace_region(ops, inner)
        return getattr(r, "values", r)


def register(*op_names: str, latency_category: str = LatencyCategory.ZERO, inplace_outs: bool = False,
             no_lx_charge: bool = False):
    """Register ``fn(op, context, env)`` as the implementation of ``op_names``."""
    def deco(fn):
        def rule(tr: Tracer, op, scope):
            result = fn(op, TraceContext(tr, scope), TraceEnv(tr, scope))
            if inplace_outs and tr.lx is not None and isinstance(result, Node) and op.operands:
                outs = scope.get(op.operands[-1])
                if isinstance(outs, Node) and not tr.lx.is_free(outs):
                    tr.lx.same_tile(result, outs)
            return result
        for name in op_names:
            T.TABLE[name] = rule
            CATEGORY_OF[name] = latency_category
            (NO_LX_CHARGE.add if no_lx_charge else NO_LX_CHARGE.discard)(name)
            (INPLACE_OUTS.add if inplace_outs else INPLACE_OUTS.discard)(name)
            prefix = name.split(".", 1)[0] + "."
            if prefix not in P._DIALECTS:
                P._DIALECTS = P._DIALECTS + (prefix,)
        return fn
    return deco


def unregister(*op_names: str):
    for name in op_names:
        T.TABLE.pop(name, None)
        CATEGORY_OF.pop(name, None)
        NO_LX_CHARGE.discard(name)
        INPLACE_OUTS.discard(name)
        _PLUGIN_PARSERS.pop(name, None)


def register_parser(op_name: str):
    """Register ``fn(parser, name, results) -> Op`` for an op with a custom assembly format
    (``parser`` is the token-level ``ModuleParser``; see ``parser_ops`` for examples)."""
    def deco(fn):
        _PLUGIN_PARSERS[op_name] = fn
        return fn
    return deco


def plugin_parser(op_name: str):
    return _PLUGIN_PARSERS.get(op_name)

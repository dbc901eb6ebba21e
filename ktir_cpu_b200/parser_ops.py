"""Per-op assembly-format parsers (the ``HANDLERS`` table).

Each routine receives the :class:`parser_impl.ModuleParser` positioned just
after the op name and returns an :class:`ir.Op`.  Formats follow the examples
and parser routines of the reference: arith/math/tensor simple forms
(ktir_cpu/dialects/arith_ops.py:312-491), ktdp views and tiles
(ktir_cpu/dialects/ktdp_ops.py:262-590, 745-849), linalg named ops
(ktir_cpu/dialects/linalg_ops.py:617-836) and scf (ktir_cpu/dialects/scf_ops.py:112-188).
"""
from __future__ import annotations

import re
from typing import Any, Dict, List

from .affine import AffineMap
from .ir import Op, Region, Type
from . import parser as P


def _result_types(results: List[str], types: List[Type], after: List[Type]) -> List[Type]:
    if not results:
        return []
    if after:
        return after if len(after) == len(results) else [after[-1]] * len(results)
    if len(types) == len(results):
        return types
    return [types[-1]] * len(results) if types else []


def parse_simple(p, name: str, results: List[str]) -> Op:
    """``op [pred,] %a[, %b ...][[idx]] [{attrs}] : types [to|into|-> type]``."""
    operands: List[str] = []
    attrs: Dict[str, Any] = {}
    while True:
        t = p.peek()
        if t is None or t.kind == "arrow" or (t.kind != "str" and t.text in (":", "to", "into", "}")):
            break
        if t.kind == "ssa":
            if p._starts_statement(0):
                break
            p.i += 1
            operands.append(t.text)
            if p.at("[") and name in ("tensor.extract", "tensor.insert"):
                idx = p.int_or_ssa_list()
                attrs["indices"] = idx
                operands.extend(x for x in idx if isinstance(x, str))
        elif t.kind == "id":
            if p._starts_statement(0):
                break
            p.i += 1
            if t.text == "output_shape":
                attrs["output_shape"] = p.int_or_ssa_list()
            else:
                attrs.setdefault("predicate", t.text)
        elif t.text == "(" and p.at(")", 1):
            p.i += 2
        elif t.kind == "num" or (t.text == "-" and p.peek(1) is not None and p.peek(1).kind == "num"):
            attrs["literal"] = p.number()
        elif t.text == "[":
            attrs["reassociation" if "shape" in name else "list"] = p.attr_value()
        elif t.text == "{":
            attrs.update(p.attr_dict())
        elif t.text == ",":
            p.i += 1
        else:
            break
    types: List[Type] = []
    after: List[Type] = []
    if p.accept(":"):
        types = p.type_list()
    if p.at("to") or p.at("into"):
        p.i += 1
        after = p.type_list()
    elif p.peek() is not None and p.peek().kind == "arrow":
        p.i += 1
        after = p.type_list()
    attrs["types"] = types
    return Op(name, results, operands, attrs, _result_types(results, types, after))


def parse_opaque(p, name: str, results: List[str]) -> Op:
    """Unknown op: swallow tokens (brace-balanced) up to the next statement."""
    depth = 0
    operands: List[str] = []
    while p.peek() is not None:
        t = p.peek()
        if depth == 0 and p._starts_statement(0):
            break
        if t.text in "{([" and t.kind == "punct":
            depth += 1
        elif t.text in "})]" and t.kind == "punct":
            depth -= 1
        elif t.kind == "ssa":
            operands.append(t.text)
        p.i += 1
    return Op(name, results, operands, {"opaque": True}, [])


def parse_constant(p, name, results) -> Op:
    attrs: Dict[str, Any] = {}
    t = p.peek()
    raw_hex = None
    if t.kind == "dense":
        p.i += 1
        body = t.text[t.text.index("<") + 1:-1].strip()
        attrs["dense"] = body
    elif t.text in ("true", "false"):
        p.i += 1
        attrs["value"] = (t.text == "true")
    else:
        if t.kind == "num" and t.text.startswith(("0x", "0X")):
            raw_hex = int(t.text, 16)
        attrs["value"] = p.number()
    p.eat(":")
    ty = P.parse_type(p.eat_kind("type").text)
    fl = ty.dtype in ("f16", "f32", "bf16", "f64", "fp16", "float16", "float32")
    if "dense" in attrs:
        body = attrs.pop("dense")
        if body.startswith("["):
            vals = [float(x) if fl else int(float(x))
                    for x in re.split(r"[\s,\[\]]+", body) if x]
            attrs["value"] = vals
            attrs["dense_list"] = True
        else:
            if body.startswith(("0x", "0X")):
                v = P._hex_to_float(int(body, 16), ty.dtype) if fl else int(body, 16)
            elif body in ("true", "false"):
                v = body == "true"
            else:
                v = float(body) if fl else int(float(body))
            attrs["value"] = v
        attrs["is_tensor"] = True
    elif raw_hex is not None and fl:
        attrs["value"] = P._hex_to_float(raw_hex, ty.dtype)
    elif fl:
        attrs["value"] = float(attrs["value"])
    return Op(name, results, [], attrs, [ty])


def parse_memory_view(p, name, results) -> Op:
    ptr = p.eat_kind("ssa").text
    operands = [ptr]
    attrs: Dict[str, Any] = {}
    p.accept(",")
    while p.at("sizes") or p.at("strides"):
        key = p.eat().text
        p.eat(":")
        vals = p.int_or_ssa_list()
        attrs[key] = vals
        operands.extend(v for v in vals if isinstance(v, str))
        p.accept(",")
    if p.at("{"):
        d = p.attr_dict()
        attrs["coordinate_set"] = d.get("coordinate_set")
        ms = d.get("memory_space", "#ktdp.memory_space<global>")
        attrs["memory_space_raw"] = ms
        m = re.search(r"<\s*([A-Za-z_]+)", str(ms))
        attrs["memory_space"] = m.group(1) if m else "global"
        m = re.search(r"ct_id\s*=\s*(\d+)", str(ms))
        if m:
            attrs["ct_id"] = int(m.group(1))
    p.eat(":")
    ty = P.parse_type(p.eat_kind("type").text)
    attrs["dtype"] = ty.dtype
    attrs.setdefault("sizes", list(ty.shape))
    if "strides" not in attrs:
        st, acc = [], 1
        for s in reversed(attrs["sizes"]):
            st.append(acc)
            acc *= s
        attrs["strides"] = list(reversed(st))
    return Op(name, results, operands, attrs, [ty])


def parse_distributed_view(p, name, results) -> Op:
    """``ktdp.construct_distributed_memory_view (%p0, %p1 : memref<..>, memref<..>) : memref<..>``"""
    p.eat("(")
    parts = []
    while p.peek().kind == "ssa":
        parts.append(p.eat_kind("ssa").text)
        p.accept(",")
    p.eat(":")
    while p.peek().kind == "type":
        p.i += 1
        p.accept(",")
    p.eat(")")
    p.eat(":")
    ty = P.parse_type(p.eat_kind("type").text)
    return Op(name, results, parts, {"shape": tuple(ty.shape), "dtype": ty.dtype}, [ty])


def parse_access_tile(p, name, results) -> Op:
    view = p.eat_kind("ssa").text
    idx = p.int_or_ssa_list()
    attrs: Dict[str, Any] = {"indices": idx}
    if p.at("{"):
        d = p.attr_dict()
        attrs["set"] = d.get("access_tile_set")
        attrs["order"] = d.get("access_tile_order")
        attrs["base_map"] = d.get("base_map")
    p.eat(":")
    p.type_list()
    after = []
    if p.peek().kind == "arrow":
        p.i += 1
        after = p.type_list()
    attrs["shape"] = tuple(after[-1].shape) if after else ()
    operands = [view] + [x for x in idx if isinstance(x, str)]
    return Op(name, results, operands, attrs, after[-1:] if after else [])


def _subscript_expr(p, var_names: List[str], ssa_refs: List[str]):
    """Quasi-affine expression over intermediate variables, SSA scalars and ints."""
    def atom():
        t = p.peek()
        if t.text == "(":
            p.eat("(")
            e = expr()
            p.eat(")")
            return e
        if t.text == "-":
            p.eat("-")
            return ("neg", atom())
        if t.kind == "ssa":
            p.i += 1
            if t.text in var_names:
                return ("var", var_names.index(t.text))
            if t.text not in ssa_refs:
                ssa_refs.append(t.text)
            return ("ssa", t.text)
        if t.kind == "num":
            return ("const", p.number())
        raise ValueError(f"line {t.line}: bad subscript token {t.text!r}")

    def term():
        node = atom()
        while p.at("*") or p.at("floordiv") or p.at("mod") or p.at("/"):
            op = p.eat().text
            node = ({"*": "mul", "/": "floordiv"}.get(op, op), node, atom())
        return node

    def expr():
        node = term()
        while p.at("+") or p.at("-"):
            op = p.eat().text
            node = ("add" if op == "+" else "sub", node, term())
        return node

    return expr()


def parse_indirect_access_tile(p, name, results) -> Op:
    p.eat("intermediate_variables")
    p.eat("(")
    var_names: List[str] = []
    while not p.at(")"):
        var_names.append(p.eat_kind("ssa").text)
        p.accept(",")
    p.eat(")")
    view = p.eat_kind("ssa").text
    ssa_refs: List[str] = []
    index_views: List[str] = []
    subs: List[Dict[str, Any]] = []
    p.eat("[")
    while not p.at("]"):
        if p.at("ind"):
            p.eat("ind")
            p.eat("(")
            iv = p.eat_kind("ssa").text
            index_views.append(iv)
            exprs = []
            p.eat("[")
            while not p.at("]"):
                exprs.append(_subscript_expr(p, var_names, ssa_refs))
                p.accept(",")
            p.eat("]")
            p.eat(")")
            subs.append({"kind": "indirect", "view": iv, "exprs": exprs})
        else:
            subs.append({"kind": "direct", "expr": _subscript_expr(p, var_names, ssa_refs)})
        p.accept(",")
    p.eat("]")
    attrs: Dict[str, Any] = {"var_names": var_names, "subscripts": subs}
    if p.at("{"):
        d = p.attr_dict()
        attrs["set"] = d.get("variables_space_set")
        attrs["order"] = d.get("variables_space_order")
    p.eat(":")
    p.type_list()
    after = []
    if p.peek().kind == "arrow":
        p.i += 1
        after = p.type_list()
    attrs["shape"] = tuple(after[-1].shape) if after else ()
    attrs["ssa_refs"] = ssa_refs
    operands = [view] + index_views + ssa_refs
    return Op(name, results, operands, attrs, after[-1:] if after else [])


def _ins_outs(p, key: str):
    names: List[str] = []
    types: List[Type] = []
    if p.at(key):
        p.eat(key)
        p.eat("(")
        while p.peek().kind == "ssa":
            names.append(p.eat().text)
            p.accept(",")
        if p.accept(":"):
            while not p.at(")"):
                types.append(P.parse_type(p.eat_kind("type").text))
                p.accept(",")
        p.eat(")")
    return names, types


def _bb_region(p) -> Region:
    """``{ [^bb0(%a: t, ...):] ops }``"""
    p.eat("{")
    reg = Region()
    if p.peek().kind == "caret":
        p.i += 1
        p.eat("(")
        while not p.at(")"):
            reg.arg_names.append(p.eat_kind("ssa").text)
            p.eat(":")
            reg.arg_types.append(P.parse_type(p.eat_kind("type").text))
            p.accept(",")
        p.eat(")")
        p.eat(":")
    reg.ops = p.block()
    p.eat("}")
    return reg


def parse_linalg_named(p, name, results) -> Op:
    attrs: Dict[str, Any] = {}
    regions: List[Region] = []
    if p.at("{"):
        nxt = p.peek(1)
        if nxt.kind == "id" and "." in nxt.text and p.at("}", 2):
            p.i += 1
            attrs["combiner"] = p.eat().text
            p.eat("}")
        else:
            attrs.update(p.attr_dict())
    ins, in_types = _ins_outs(p, "ins")
    outs, out_types = _ins_outs(p, "outs")
    while p.at("dimensions") or p.at("permutation"):
        key = p.eat().text
        p.eat("=")
        attrs[key] = p.int_or_ssa_list()
    if p.at("(") and p.peek(1).kind == "ssa":      # reduce explicit region header
        reg = Region()
        p.eat("(")
        while not p.at(")"):
            reg.arg_names.append(p.eat_kind("ssa").text)
            p.eat(":")
            reg.arg_types.append(P.parse_type(p.eat_kind("type").text))
            p.accept(",")
        p.eat(")")
        p.eat("{")
        reg.ops = p.block()
        p.eat("}")
        # in this form the reference reads the block arguments off the operands of the region's first
        # op, not off the header (ktir_cpu/dialects/linalg_ops.py:30-58): lhs and rhs bind in THAT order
        if reg.ops:
            reg.arg_names = [o_ for o_ in reg.ops[0].operands if isinstance(o_, str)]
        regions.append(reg)
    elif p.at("{"):
        regions.append(_bb_region(p))
    after: List[Type] = []
    if p.peek() is not None and p.peek().kind == "arrow":
        p.i += 1
        after = p.type_list()
    attrs["n_ins"] = len(ins)
    attrs["in_types"], attrs["out_types"] = in_types, out_types
    rt = after or out_types
    if name == "linalg.reduce" and not after:
        rt = out_types
    return Op(name, results, ins + outs, attrs, _result_types(results, rt, []), regions)


def parse_linalg_index(p, name, results) -> Op:
    dim = p.number()
    p.eat(":")
    ty = P.parse_type(p.eat_kind("type").text)
    return Op(name, results, [], {"dim": dim}, [ty])


def parse_terminator(p, name, results) -> Op:
    operands: List[str] = []
    while p.peek() is not None and p.peek().kind == "ssa" and not p._starts_statement(0):
        operands.append(p.eat().text)
        if not p.accept(","):
            break
    types: List[Type] = []
    if p.accept(":"):
        types = p.type_list()
    return Op(name, results, operands, {"types": types}, [])


def _operand_or_const(p, attrs, key) -> str:
    t = p.peek()
    if t.kind == "ssa":
        p.i += 1
        return t.text
    attrs.setdefault("const_operands", {})[key] = p.number()
    return f"__const_{key}"


def parse_for(p, name, results) -> Op:
    attrs: Dict[str, Any] = {}
    iv = p.eat_kind("ssa").text
    p.eat("=")
    lb = _operand_or_const(p, attrs, "lb")
    p.eat("to")
    ub = _operand_or_const(p, attrs, "ub")
    p.eat("step")
    st = _operand_or_const(p, attrs, "step")
    iter_names: List[str] = []
    inits: List[str] = []
    rtypes: List[Type] = []
    if p.at("iter_args"):
        p.eat("iter_args")
        p.eat("(")
        while not p.at(")"):
            iter_names.append(p.eat_kind("ssa").text)
            p.eat("=")
            inits.append(p.eat_kind("ssa").text)
            p.accept(",")
        p.eat(")")
    if p.peek().kind == "arrow":
        p.i += 1
        rtypes = p.type_list()
    if p.accept(":"):
        p.eat_kind("type")
    p.eat("{")
    body = p.block()
    p.eat("}")
    attrs["iter_var"] = iv
    attrs["iter_args"] = iter_names
    reg = Region([iv] + iter_names, [Type("scalar", "index")] + rtypes, body)
    return Op(name, results, [lb, ub, st] + inits, attrs, _result_types(results, rtypes, []), [reg])


def parse_if(p, name, results) -> Op:
    cond = p.eat_kind("ssa").text
    rtypes: List[Type] = []
    if p.peek().kind == "arrow":
        p.i += 1
        rtypes = p.type_list()
    regions = []
    p.eat("{")
    regions.append(Region(ops=p.block()))
    p.eat("}")
    if p.accept("else"):
        p.eat("{")
        regions.append(Region(ops=p.block()))
        p.eat("}")
    return Op(name, results, [cond], {}, _result_types(results, rtypes, []), regions)


def _split_top(text: str) -> List[str]:
    """Split on commas outside angle / round brackets ('->', '>=' and '<=' are not brackets)."""
    out, depth, cur, i = [], 0, [], 0
    while i < len(text):
        c = text[i]
        two = text[i:i + 2]
        if two in ("->", ">=", "<="):
            cur.append(two)
            i += 2
            continue
        if c in "<(":
            depth += 1
        elif c in ">)":
            depth -= 1
        if c == "," and depth == 0:
            out.append("".join(cur))
            cur = []
        else:
            cur.append(c)
        i += 1
    if "".join(cur).strip():
        out.append("".join(cur))
    return out


def _tile_future_type(p):
    """``!ktdp.tile_future<T {, T} [, groups = <affine set>]>`` -> (partial types, groups set or None).
    The prefix may be elided (``<T, groups = ...>``), as the MLIR printer writes it."""
    t = p.peek()
    if t.kind == "type" and t.text.startswith("!ktdp.tile_future"):
        p.i += 1
        inner = t.text[t.text.index("<") + 1:-1]
    else:
        # elided prefix: collect the source text between the balanced '<' ... '>'
        p.eat("<")
        depth, parts = 1, []
        while depth:
            tok = p.eat()
            if tok.kind == "punct" and tok.text == "<":
                depth += 1
            elif tok.kind == "punct" and tok.text == ">":
                depth -= 1
                if depth == 0:
                    break
            parts.append(tok.text)
        inner = " ".join(parts)
    types, groups = [], None
    for part in _split_top(inner):
        part = part.strip()
        if part.startswith("groups"):
            g = part.split("=", 1)[1].strip()
            groups = p.aliases[g] if g.startswith("#") else p.affine(g)
        elif part:
            for t in _split_top(part.strip("() ")):
                if t.strip():
                    types.append(P.parse_type(t.strip()))
    return types, groups


def parse_inter_tile_produce(p, name, results) -> Op:
    """``ktdp.inter_tile_produce producer_tiles_per_group = <set> : T -> !ktdp.tile_future<T, groups = <set>>
    { ^bb0(%gid: index): ... ktdp.yield_partial %t : T }`` (ktir_cpu/dialects/ktdp_ops.py:1040-1097)."""
    attrs: Dict[str, Any] = {}
    while p.peek().kind == "id" and p.at("=", 1):
        key = p.eat().text
        p.eat("=")
        attrs[key] = p.attr_value()
        p.accept(",")
    if "producer_tiles_per_group" not in attrs:
        raise ValueError("ktdp.inter_tile_produce: missing producer_tiles_per_group")
    if p.accept(":"):
        attrs["partial_types"] = p.type_list()
    if p.peek().kind != "arrow":
        raise ValueError("ktdp.inter_tile_produce/reduce: missing !ktdp.tile_future<...> type")
    p.i += 1
    types, groups = _tile_future_type(p)
    if groups is None:
        raise ValueError("ktdp.inter_tile_produce: missing groups inside !ktdp.tile_future<...> type")
    attrs["groups"] = groups
    attrs["future_types"] = types
    attrs.setdefault("partial_types", types)
    regions = [_bb_region(p)] if p.at("{") else []
    return Op(name, results, [], attrs, [Type("scalar", "tile_future")], regions)


def parse_inter_tile_reduce(p, name, results) -> Op:
    """``ktdp.inter_tile_reduce(%fut) consumer_tiles_per_group = <set>, identity(%id : T)
    [, producer_dependency_per_consumer = <set>] : !ktdp.tile_future<...> -> T_r
    { ^bb0(%lhs: T, %rhs: T): ... ktdp.yield_reduced %t : T }`` (ktir_cpu/dialects/ktdp_ops.py:1242-1330)."""
    p.eat("(")
    fut = p.eat_kind("ssa").text
    p.eat(")")
    attrs: Dict[str, Any] = {}
    identity = None
    while p.peek().kind == "id":
        key = p.eat().text
        if key == "identity":
            p.eat("(")
            identity = p.eat_kind("ssa").text
            if p.accept(":"):
                p.eat_kind("type")
            p.eat(")")
        else:
            p.eat("=")
            attrs[key] = p.attr_value()
        p.accept(",")
    if "consumer_tiles_per_group" not in attrs:
        raise ValueError("ktdp.inter_tile_reduce: missing consumer_tiles_per_group")
    if identity is None:
        raise ValueError("ktdp.inter_tile_reduce: missing identity(...) operand")
    p.eat(":")
    _tile_future_type(p)
    rtypes: List[Type] = []
    if p.peek().kind == "arrow":
        p.i += 1
        rtypes = p.type_list()
    regions = [_bb_region(p)] if p.at("{") else []
    return Op(name, results, [fut, identity], attrs, _result_types(results, rtypes, []), regions)


HANDLERS = {
    "ktdp.inter_tile_produce": parse_inter_tile_produce,
    "ktdp.inter_tile_reduce": parse_inter_tile_reduce,
    "ktdp.yield_partial": parse_terminator,
    "ktdp.yield_reduced": parse_terminator,
    "arith.constant": parse_constant,
    "ktdp.construct_memory_view": parse_memory_view,
    "ktdp.construct_distributed_memory_view": parse_distributed_view,
    "ktdp.construct_access_tile": parse_access_tile,
    "ktdp.construct_indirect_access_tile": parse_indirect_access_tile,
    "linalg.reduce": parse_linalg_named,
    "linalg.matmul": parse_linalg_named,
    "linalg.batch_matmul": parse_linalg_named,
    "linalg.generic": parse_linalg_named,
    "linalg.fill": parse_linalg_named,
    "linalg.broadcast": parse_linalg_named,
    "linalg.transpose": parse_linalg_named,
    "linalg.add": parse_linalg_named,
    "linalg.max": parse_linalg_named,
    "linalg.index": parse_linalg_index,
    "linalg.yield": parse_terminator,
    "scf.yield": parse_terminator,
    "tensor.yield": parse_terminator,
    "return": parse_terminator,
    "func.return": parse_terminator,
    "scf.for": parse_for,
    "scf.if": parse_if,
}

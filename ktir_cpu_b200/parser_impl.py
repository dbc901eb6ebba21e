"""Recursive-descent statement parser used by :class:`parser.KTIRParser`."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from .affine import AffineMap, AffineSet, parse_affine_map, parse_affine_set
from .ir import IRFunction, IRModule, Op, Region, Type
from . import parser as P


class ParseError(ValueError):
    pass


class ModuleParser:
    def __init__(self, source: str):
        self.toks = P.tokenize(source)
        self.i = 0
        self.aliases: Dict[str, Any] = {}

    # ---- token helpers -------------------------------------------------
    def peek(self, k: int = 0) -> Optional[P.Tok]:
        j = self.i + k
        return self.toks[j] if j < len(self.toks) else None

    def at(self, text: str, k: int = 0) -> bool:
        t = self.peek(k)
        return t is not None and t.text == text and t.kind not in ("str",)

    def eat(self, text: Optional[str] = None) -> P.Tok:
        t = self.peek()
        if t is None:
            raise ParseError(f"unexpected end of input (expected {text!r})")
        if text is not None and t.text != text:
            raise ParseError(f"line {t.line}: expected {text!r}, got {t.text!r}")
        self.i += 1
        return t

    def accept(self, text: str) -> bool:
        if self.at(text):
            self.i += 1
            return True
        return False

    def eat_kind(self, kind: str) -> P.Tok:
        t = self.peek()
        if t is None or t.kind != kind:
            raise ParseError(f"line {t.line if t else '?'}: expected {kind}, got {t!r}")
        self.i += 1
        return t

    # ---- values ----------------------------------------------------------
    def affine(self, text: str):
        return parse_affine_map(text) if text.startswith("affine_map") else parse_affine_set(text)

    def number(self) -> Any:
        neg = self.accept("-")
        if not neg:
            self.accept("+")
        t = self.eat_kind("num")
        s = t.text
        if s.startswith(("0x", "0X")):
            v: Any = int(s, 16)
        elif any(c in s for c in ".eE"):
            v = float(s)
        else:
            v = int(s)
        return -v if neg else v

    def attr_value(self) -> Any:
        t = self.peek()
        if t.kind == "affine":
            self.i += 1
            return self.affine(t.text)
        if t.kind == "attr":
            self.i += 1
            if t.text in self.aliases:
                return self.aliases[t.text]
            return t.text
        if t.kind == "str":
            self.i += 1
            return t.text[1:-1]
        if t.kind == "num" or t.text in "-+":
            v = self.number()
            if self.accept(":"):
                self.eat_kind("type")
            return v
        if t.text == "[":
            self.eat("[")
            out = []
            while not self.at("]"):
                out.append(self.attr_value())
                self.accept(",")
            self.eat("]")
            return out
        if t.kind == "type":
            self.i += 1
            return P.parse_type(t.text)
        if t.kind == "dense":
            self.i += 1
            return t.text
        if t.kind in ("id", "ssa", "sym"):
            self.i += 1
            return {"true": True, "false": False}.get(t.text, t.text)
        raise ParseError(f"line {t.line}: bad attribute value {t.text!r}")

    def attr_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        self.eat("{")
        while not self.at("}"):
            key = self.eat().text
            if self.accept("="):
                out[key] = self.attr_value()
            else:
                out[key] = True
            self.accept(",")
        self.eat("}")
        return out

    def int_or_ssa_list(self) -> List[Any]:
        out: List[Any] = []
        self.eat("[")
        while not self.at("]"):
            t = self.peek()
            if t.kind == "ssa":
                self.i += 1
                out.append(t.text)
            else:
                out.append(self.number())
            self.accept(",")
        self.eat("]")
        return out

    def type_list(self) -> List[Type]:
        """type (',' type)* — also accepts a parenthesised list."""
        out: List[Type] = []
        if self.accept("("):
            while not self.at(")"):
                out.append(P.parse_type(self.eat_kind("type").text))
                self.accept(",")
            self.eat(")")
            return out
        out.append(P.parse_type(self.eat_kind("type").text))
        while self.at(",") and self.peek(1) is not None and self.peek(1).kind == "type":
            self.eat(",")
            out.append(P.parse_type(self.eat_kind("type").text))
        return out

    # ---- module / function ---------------------------------------------
    def parse(self) -> IRModule:
        mod = IRModule()
        while self.peek() is not None:
            t = self.peek()
            if t.kind == "attr" and self.at("=", 1):
                self.i += 2
                v = self.peek()
                if v.kind == "affine":
                    self.i += 1
                    self.aliases[t.text] = self.affine(v.text)
                else:
                    self.aliases[t.text] = self.attr_value()
            elif t.text == "module":
                self.i += 1
                if self.peek().kind == "sym":
                    self.i += 1
                if self.at("attributes"):
                    self.i += 1
                    self.attr_dict()
                self.eat("{")
            elif t.text == "}":
                self.i += 1
            elif t.text == "func.func":
                fn = self.function()
                mod.functions[fn.name] = fn
            else:
                raise ParseError(f"line {t.line}: unexpected top-level token {t.text!r}")
        return mod

    def function(self) -> IRFunction:
        self.eat("func.func")
        if self.peek().kind == "id":      # visibility keyword
            self.i += 1
        name = self.eat_kind("sym").text[1:]
        args: List[Tuple[str, Type]] = []
        self.eat("(")
        while not self.at(")"):
            an = self.eat_kind("ssa").text
            self.eat(":")
            args.append((an, P.parse_type(self.eat_kind("type").text)))
            self.accept(",")
        self.eat(")")
        if self.peek().kind == "arrow":
            self.i += 1
            self.type_list()
        grid = (1, 1, 1)
        if self.accept("attributes"):
            attrs = self.attr_dict()
            g = list(attrs.get("grid", [])) + [1, 1, 1]
            grid = (int(g[0]), int(g[1]), int(g[2]))
        self.eat("{")
        ops = self.block()
        self.eat("}")
        fn = IRFunction(name, args, grid, ops)
        arg_names = {n for n, _ in fn.args}
        from .ir import walk
        for op in walk(ops):
            if op.name == "ktdp.construct_memory_view" and op.operands:
                p = op.operands[0]
                if p in arg_names and p[1:] not in fn.tensor_sizes:
                    shape = op.attrs["sizes"]
                    if all(isinstance(s, int) for s in shape):
                        fn.tensor_sizes[p[1:]] = {"shape": tuple(shape), "dtype": op.attrs["dtype"]}
        return fn

    def block(self) -> List[Op]:
        ops: List[Op] = []
        while not self.at("}"):
            if self.peek() is None:
                raise ParseError("unexpected end of input inside a block")
            ops.append(self.statement())
        return ops

    # ---- statements ------------------------------------------------------
    def _starts_statement(self, k: int) -> bool:
        t = self.peek(k)
        if t is None or t.text == "}":
            return True
        if t.kind == "id" and (t.text.startswith(P._DIALECTS) or t.text == "return"):
            return True
        if t.kind == "ssa":
            j = k + 1
            while self.at(",", j) and self.peek(j + 1) is not None and self.peek(j + 1).kind == "ssa":
                j += 2
            return self.at("=", j)
        return False

    def statement(self) -> Op:
        line = self.peek().line
        results: List[str] = []
        if self.peek().kind == "ssa":
            results.append(self.eat().text)
            while self.accept(","):
                results.append(self.eat_kind("ssa").text)
            self.eat("=")
        t = self.peek()
        if t.kind == "ssa":               # infix shorthand: %a = %b * %c : index
            return self._infix(results, line)
        name = self.eat().text
        from .parser_ops import HANDLERS, parse_simple, parse_opaque
        from .registry import plugin_parser
        from .trace_ops import TABLE
        fn = plugin_parser(name) or HANDLERS.get(name)
        if fn is None and name in TABLE and not name.startswith(("ktdp.", "linalg.", "scf.", "func.")):
            fn = parse_simple                  # a registered plug-in op in the generic form
        if fn is None:
            if name.startswith(("arith.", "math.", "tensor.")) or name in ("ktdp.load", "ktdp.store",
                                                                            "ktdp.get_compute_tile_id",
                                                                            "ktdp.coreid"):
                fn = parse_simple
            else:
                fn = parse_opaque
        op = fn(self, name, results)
        op.line = line
        return op

    def _infix(self, results, line) -> Op:
        a = self.eat_kind("ssa").text
        sym = self.eat().text
        b = self.eat_kind("ssa").text
        self.eat(":")
        ty = P.parse_type(self.eat_kind("type").text)
        name = {"*": "arith.muli", "+": "arith.addi", "-": "arith.subi"}.get(sym)
        if name is None:
            raise ParseError(f"line {line}: unsupported infix operator {sym!r}")
        return Op(name, results, [a, b], {}, [ty], [], line)

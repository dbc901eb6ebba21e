"""Affine maps and integer sets of the ktdp dialect (host side).

``affine_map<(d0, d1)[s0] -> (d0 + s0, d1 * 2)>`` and
``affine_set<(d0, d1) : (d0 >= 0, -d0 + 127 >= 0, ...)>`` are parsed into small
expression trees that evaluate on Python ints *and* on NumPy integer arrays, so
one evaluation covers every grid core and loop iteration of a launch at once.

Behavioural model: ktir_cpu/parser_ast.py:374-544 (parse / evaluate /
enumerate) and ktir_cpu/affine.py:216-437 (axis-aligned boxes).
"""
from __future__ import annotations

import itertools
import re
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

_TOK = re.compile(r"\s*(?:(\d+)|([A-Za-z_][A-Za-z_0-9]*)|(->|>=|<=|==|[-+*(),\[\]:]))")


def _tokenize(text: str) -> List[str]:
    out, pos = [], 0
    text = text.strip()
    while pos < len(text):
        m = _TOK.match(text, pos)
        if not m:
            raise ValueError(f"affine: cannot tokenize {text[pos:pos + 20]!r} in {text!r}")
        out.append(m.group(1) or m.group(2) or m.group(3))
        pos = m.end()
    return out


class _ExprParser:
    """Recursive descent over + - * floordiv ceildiv mod with dims/symbols."""

    def __init__(self, toks: List[str], dims: List[str], syms: List[str]):
        self.t, self.i, self.dims, self.syms = toks, 0, dims, syms

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else None

    def eat(self, tok=None):
        cur = self.peek()
        if tok is not None and cur != tok:
            raise ValueError(f"affine: expected {tok!r}, got {cur!r}")
        self.i += 1
        return cur

    def expr(self):
        node = self.term()
        while self.peek() in ("+", "-"):
            op = self.eat()
            rhs = self.term()
            node = ("add" if op == "+" else "sub", node, rhs)
        return node

    def term(self):
        node = self.factor()
        while self.peek() in ("*", "floordiv", "ceildiv", "mod"):
            op = self.eat()
            rhs = self.factor()
            node = ({"*": "mul"}.get(op, op), node, rhs)
        return node

    def factor(self):
        cur = self.peek()
        if cur == "-":
            self.eat()
            return ("neg", self.factor())
        if cur == "(":
            self.eat()
            node = self.expr()
            self.eat(")")
            return node
        self.eat()
        if cur is None:
            raise ValueError("affine: unexpected end of expression")
        if cur.isdigit():
            return ("const", int(cur))
        if cur in self.dims:
            return ("dim", self.dims.index(cur))
        if cur in self.syms:
            return ("sym", self.syms.index(cur))
        raise ValueError(f"affine: unknown identifier {cur!r}")


def eval_expr(node, dims: Sequence, syms: Sequence = ()):
    """Evaluate an expression tree; operands may be ints or integer ndarrays."""
    k = node[0]
    if k == "const":
        return node[1]
    if k == "dim":
        return dims[node[1]]
    if k == "sym":
        return syms[node[1]]
    if k == "neg":
        return -eval_expr(node[1], dims, syms)
    a, b = eval_expr(node[1], dims, syms), eval_expr(node[2], dims, syms)
    if k == "add":
        return a + b
    if k == "sub":
        return a - b
    if k == "mul":
        return a * b
    if k == "floordiv":
        return a // b
    if k == "ceildiv":
        return -((-a) // b)
    if k == "mod":
        return a % b
    raise ValueError(f"affine: bad node {k}")


def _linear(node, n_dims: int):
    """Return (coeffs, const) if node is linear in dims with no symbols, else None."""
    k = node[0]
    if k == "const":
        return [0] * n_dims, node[1]
    if k == "dim":
        c = [0] * n_dims
        c[node[1]] = 1
        return c, 0
    if k == "neg":
        r = _linear(node[1], n_dims)
        return None if r is None else ([-x for x in r[0]], -r[1])
    if k in ("add", "sub"):
        a, b = _linear(node[1], n_dims), _linear(node[2], n_dims)
        if a is None or b is None:
            return None
        s = 1 if k == "add" else -1
        return [x + s * y for x, y in zip(a[0], b[0])], a[1] + s * b[1]
    if k == "mul":
        a, b = _linear(node[1], n_dims), _linear(node[2], n_dims)
        if a is None or b is None:
            return None
        if not any(a[0]):
            return [a[1] * y for y in b[0]], a[1] * b[1]
        if not any(b[0]):
            return [b[1] * x for x in a[0]], a[1] * b[1]
    return None


def _split_header(text: str, kind: str):
    text = text.strip()
    m = re.match(rf"{kind}\s*<(.*)>\s*$", text, re.S)
    if m:
        text = m.group(1)
    return text


def _parse_names(p: _ExprParser, open_tok: str, close_tok: str) -> List[str]:
    names = []
    p.eat(open_tok)
    while p.peek() != close_tok:
        names.append(p.eat())
        if p.peek() == ",":
            p.eat()
    p.eat(close_tok)
    return names


@dataclass
class AffineMap:
    n_dims: int
    n_syms: int
    exprs: Tuple
    source: str = ""

    def eval(self, dims: Sequence, syms: Sequence = ()):
        if len(dims) != self.n_dims:
            raise ValueError(
                f"AffineMap expects {self.n_dims} dim(s), got {len(dims)}: {self.source!r}")
        return tuple(eval_expr(e, dims, syms) for e in self.exprs)

    def is_identity(self) -> bool:
        return (len(self.exprs) == self.n_dims
                and all(e == ("dim", i) for i, e in enumerate(self.exprs)))

    def permutation(self) -> Optional[List[int]]:
        """Output position -> input dim, when the map only permutes its dims."""
        if len(self.exprs) != self.n_dims or any(e[0] != "dim" for e in self.exprs):
            return None
        perm = [e[1] for e in self.exprs]
        return perm if sorted(perm) == list(range(self.n_dims)) else None

    def is_permutation(self) -> bool:
        return self.permutation() is not None

    @staticmethod
    def identity(n: int) -> "AffineMap":
        return AffineMap(n, 0, tuple(("dim", i) for i in range(n)), "identity")


@dataclass
class AffineSet:
    n_dims: int
    n_syms: int
    constraints: Tuple          # (expr, 'ge'|'eq') meaning expr >= 0 / expr == 0
    source: str = ""

    def contains(self, point: Sequence[int], syms: Sequence[int] = ()) -> bool:
        for e, kind in self.constraints:
            v = eval_expr(e, point, syms)
            if (kind == "ge" and v < 0) or (kind == "eq" and v != 0):
                return False
        return True

    def box(self) -> Optional[Tuple[Tuple[int, ...], Tuple[int, ...]]]:
        """(lo, hi) with hi exclusive when every constraint bounds one dim."""
        if self.n_syms:
            return None
        lo = [None] * self.n_dims
        hi = [None] * self.n_dims
        for e, kind in self.constraints:
            lin = _linear(e, self.n_dims)
            if lin is None:
                return None
            coeffs, c = lin
            nz = [i for i, x in enumerate(coeffs) if x]
            if len(nz) != 1 or abs(coeffs[nz[0]]) != 1:
                return None
            d, s = nz[0], coeffs[nz[0]]
            if kind == "eq":          # s*d + c == 0
                v = -c * s
                lo[d] = v if lo[d] is None else max(lo[d], v)
                hi[d] = v + 1 if hi[d] is None else min(hi[d], v + 1)
            elif s == 1:              # d + c >= 0
                lo[d] = -c if lo[d] is None else max(lo[d], -c)
            else:                     # -d + c >= 0
                hi[d] = c + 1 if hi[d] is None else min(hi[d], c + 1)
        if any(x is None for x in lo) or any(x is None for x in hi):
            return None
        return tuple(lo), tuple(hi)

    def box_with(self, syms: Sequence[int]) -> Optional[Tuple[Tuple[int, ...], Tuple[int, ...]]]:
        """``box()`` with the set's symbols bound to ``syms`` (left to right); None when the set is
        not a box.  Coefficients are read off numerically, which is exact for affine constraints."""
        if not self.n_syms:
            return self.box()
        if len(syms) < self.n_syms:
            raise ValueError(f"AffineSet needs {self.n_syms} symbol value(s), got {len(syms)}: {self.source!r}")
        syms = [int(x) for x in syms[:self.n_syms]]
        lo = [None] * self.n_dims
        hi = [None] * self.n_dims
        zero = [0] * self.n_dims
        for e, kind in self.constraints:
            c = eval_expr(e, zero, syms)
            coeffs = []
            for d in range(self.n_dims):
                unit = list(zero)
                unit[d] = 1
                k = eval_expr(e, unit, syms) - c
                unit[d] = 2
                if eval_expr(e, unit, syms) - c != 2 * k:
                    return None
                coeffs.append(k)
            nz = [i for i, x in enumerate(coeffs) if x]
            if len(nz) != 1 or abs(coeffs[nz[0]]) != 1:
                return None
            d, sgn = nz[0], coeffs[nz[0]]
            if kind == "eq":
                v = -c * sgn
                lo[d] = v if lo[d] is None else max(lo[d], v)
                hi[d] = v + 1 if hi[d] is None else min(hi[d], v + 1)
            elif sgn == 1:
                lo[d] = -c if lo[d] is None else max(lo[d], -c)
            else:
                hi[d] = c + 1 if hi[d] is None else min(hi[d], c + 1)
        if any(x is None for x in lo) or any(x is None for x in hi):
            return None
        return tuple(lo), tuple(hi)

    def enumerate(self, shape: Sequence[int], syms: Sequence[int] = ()) -> List[Tuple[int, ...]]:
        """Points of ``[0, shape)`` in the set, row-major (parser_ast.py:525-544)."""
        if len(shape) != self.n_dims:
            raise ValueError(
                f"AffineSet has {self.n_dims} dim(s), got shape with {len(shape)}: {self.source!r}")
        b = self.box()
        if b is not None:
            return list(itertools.product(*(range(l, h) for l, h in zip(*b))))
        return [pt for pt in itertools.product(*(range(s) for s in shape))
                if self.contains(pt, syms)]


def parse_affine_map(text: str) -> AffineMap:
    src = text
    toks = _tokenize(_split_header(text, "affine_map"))
    p = _ExprParser(toks, [], [])
    dims = _parse_names(p, "(", ")")
    syms = _parse_names(p, "[", "]") if p.peek() == "[" else []
    p.dims, p.syms = dims, syms
    p.eat("->")
    p.eat("(")
    exprs = []
    while p.peek() != ")":
        exprs.append(p.expr())
        if p.peek() == ",":
            p.eat()
    p.eat(")")
    return AffineMap(len(dims), len(syms), tuple(exprs), src)


def parse_affine_set(text: str) -> AffineSet:
    src = text
    toks = _tokenize(_split_header(text, "affine_set"))
    p = _ExprParser(toks, [], [])
    dims = _parse_names(p, "(", ")")
    syms = _parse_names(p, "[", "]") if p.peek() == "[" else []
    p.dims, p.syms = dims, syms
    p.eat(":")
    p.eat("(")
    cons = []
    while p.peek() != ")":
        lhs = p.expr()
        op = p.eat()
        rhs = p.expr()
        if op == ">=":
            cons.append((("sub", lhs, rhs), "ge"))
        elif op == "<=":
            cons.append((("sub", rhs, lhs), "ge"))
        elif op == "==":
            cons.append((("sub", lhs, rhs), "eq"))
        else:
            raise ValueError(f"affine_set: unsupported relation {op!r} in {src!r}")
        if p.peek() == ",":
            p.eat()
    p.eat(")")
    return AffineSet(len(dims), len(syms), tuple(cons), src)

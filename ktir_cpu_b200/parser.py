"""Text front end: KTIR (MLIR ``ktdp`` dialect) source -> :class:`IRModule`.

A tokenizer plus one small recursive-descent routine per custom assembly
format.  Covers the surface syntax accepted by the reference's regex parser
(ktir_cpu/parser.py:85-147 and the per-dialect ``register_parser`` routines,
e.g. ktir_cpu/dialects/ktdp_ops.py:262-590) for the ops this backend executes;
unknown ops are kept as opaque :class:`Op` nodes so that execution, not parsing,
reports ``Unknown operation``.
"""
from __future__ import annotations

import re
import struct
from typing import Any, Dict, List, Optional, Tuple

from .affine import AffineMap, AffineSet, parse_affine_map, parse_affine_set
from .ir import IRFunction, IRModule, Op, Region, Type

_SCALAR_TYPES = {"index", "f16", "f32", "f64", "bf16", "i1", "i8", "i16", "i32", "i64",
                 "si32", "si64", "fp8", "mxfp8", "fp16", "float16", "float32"}
_ANGLE_IDENTS = {"tensor", "memref", "affine_map", "affine_set", "dense", "vector"}
_DIALECTS = ("ktdp.", "arith.", "math.", "linalg.", "tensor.", "scf.", "func.", "tt.")

_SIMPLE = re.compile(r"""
    (?P<ws>\s+|//[^\n]*)
  | (?P<str>"(?:[^"\\]|\\.)*")
  | (?P<ssa>%[A-Za-z0-9_.$\-]+(?:\#\d+)?)
  | (?P<sym>@[A-Za-z0-9_.$\-]+)
  | (?P<caret>\^[A-Za-z0-9_]+)
  | (?P<num>0x[0-9a-fA-F]+|\d+\.\d*(?:[eE][-+]?\d+)?|\d+[eE][-+]?\d+|\d+)
  | (?P<id>[A-Za-z_][A-Za-z0-9_.$]*)
  | (?P<arrow>->)
  | (?P<punct>[-+*/=,:(){}\[\]<>?])
""", re.X)


_ELIDED = re.compile(r"<(?:(?:\d+|\?)x)*index>")


class Tok:
    __slots__ = ("kind", "text", "line")

    def __init__(self, kind, text, line):
        self.kind, self.text, self.line = kind, text, line

    def __repr__(self):
        return f"{self.kind}:{self.text!r}"


def _angle_end(src: str, start: int) -> int:
    """Index just past the '>' matching the '<' at ``start`` ('->', '>=' and '<=' are skipped)."""
    depth, i, n = 0, start, len(src)
    while i < n:
        c = src[i]
        if c == "<" and not (i + 1 < n and src[i + 1] == "="):
            depth += 1
        elif c == ">":
            if i > 0 and src[i - 1] == "-":
                pass
            elif i + 1 < n and src[i + 1] == "=":
                pass
            else:
                depth -= 1
                if depth == 0:
                    return i + 1
        i += 1
    raise ValueError(f"unbalanced '<' near {src[start:start + 40]!r}")


def tokenize(src: str) -> List[Tok]:
    toks: List[Tok] = []
    pos, line, n = 0, 1, len(src)
    while pos < n:
        c = src[pos]
        if c in "#!":
            m = re.compile(r"[#!][A-Za-z_][A-Za-z0-9_.$]*").match(src, pos)
            if not m:
                raise ValueError(f"line {line}: stray {c!r}")
            end = m.end()
            if end < n and src[end] == "<":
                end = _angle_end(src, end)
            text = src[pos:end]
            toks.append(Tok("attr" if c == "#" else "type", text, line))
            line += text.count("\n")
            pos = end
            continue
        if c == "<":          # elided dialect type: `<128xindex>` == !ktdp.access_tile<128xindex>
            em = _ELIDED.match(src, pos)
            if em:
                toks.append(Tok("type", "!ktdp.access_tile" + em.group(0), line))
                pos = em.end()
                continue
        m = _SIMPLE.match(src, pos)
        if not m:
            raise ValueError(f"line {line}: cannot tokenize {src[pos:pos + 30]!r}")
        kind = m.lastgroup
        text = m.group(kind)
        end = m.end()
        if kind == "ws":
            line += text.count("\n")
            pos = end
            continue
        if kind == "id" and text in _ANGLE_IDENTS and end < n and src[end] == "<":
            end = _angle_end(src, end)
            text = src[pos:end]
            kind = {"affine_map": "affine", "affine_set": "affine", "dense": "dense"}.get(
                text.split("<", 1)[0], "type")
        elif kind == "id" and text in _SCALAR_TYPES:
            kind = "type"
        toks.append(Tok(kind, text, line))
        line += text.count("\n")
        pos = end
    return toks


def parse_type(text: str) -> Type:
    text = text.strip()
    if text in _SCALAR_TYPES:
        return Type("scalar", text)
    m = re.match(r"(!ktdp\.access_tile|tensor|memref|vector)\s*<(.*)>$", text, re.S)
    if not m:
        return Type("scalar", text)
    kind = {"!ktdp.access_tile": "access_tile"}.get(m.group(1), m.group(1))
    body = m.group(2).split(",")[0].strip()
    dims = []
    while True:
        dm = re.match(r"\s*(\d+|\?)\s*x", body)
        if not dm:
            break
        dims.append(None if dm.group(1) == "?" else int(dm.group(1)))
        body = body[dm.end():]
    dtype = body.strip()
    shape = tuple(dims)
    return Type(kind, dtype, shape)


def _hex_to_float(bits: int, dtype: str) -> float:
    if dtype in ("f16", "fp16", "float16"):
        return struct.unpack("<e", struct.pack("<H", bits & 0xFFFF))[0]
    if dtype in ("f32", "float32"):
        return struct.unpack("<f", struct.pack("<I", bits & 0xFFFFFFFF))[0]
    if dtype == "bf16":
        return struct.unpack("<f", struct.pack("<I", (bits & 0xFFFF) << 16))[0]
    raise ValueError(f"hex float literal for unsupported type {dtype}")


class KTIRParserBase:
    """Parser seam (ktir_cpu/parser.py:32-48): ``parse_module(text) -> IRModule``."""

    def parse_module(self, source: str) -> IRModule:
        raise NotImplementedError


class KTIRParser(KTIRParserBase):
    def parse_module(self, source: str) -> IRModule:
        from .parser_impl import ModuleParser
        return ModuleParser(source).parse()

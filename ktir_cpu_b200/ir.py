"""In-memory form of a parsed KTIR module (host side).

Plays the role of ktir_cpu/ir_types.py:524-600 (``Operation`` / ``IRFunction``
/ ``IRModule``) for this backend: a plain tree of operations with named SSA
results, operand names, an attribute dict and nested regions.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class Type:
    """``kind`` is one of tensor / memref / access_tile / scalar."""
    kind: str
    dtype: str
    shape: Optional[Tuple[Optional[int], ...]] = None

    def __str__(self):
        if self.kind == "scalar":
            return self.dtype
        dims = "x".join("?" if d is None else str(d) for d in (self.shape or ()))
        body = f"{dims}x{self.dtype}" if dims else self.dtype
        return f"{self.kind}<{body}>"


@dataclass
class Region:
    arg_names: List[str] = field(default_factory=list)
    arg_types: List[Type] = field(default_factory=list)
    ops: List["Op"] = field(default_factory=list)


@dataclass
class Op:
    name: str
    results: List[str] = field(default_factory=list)
    operands: List[str] = field(default_factory=list)
    attrs: Dict[str, Any] = field(default_factory=dict)
    result_types: List[Type] = field(default_factory=list)
    regions: List[Region] = field(default_factory=list)
    line: int = 0

    def __repr__(self):
        res = ", ".join(self.results)
        return f"<{res + ' = ' if res else ''}{self.name} {', '.join(self.operands)} @L{self.line}>"


@dataclass
class IRFunction:
    name: str
    args: List[Tuple[str, Type]]
    grid: Tuple[int, int, int]
    ops: List[Op]
    tensor_sizes: Dict[str, Dict[str, Any]] = field(default_factory=dict)

    @property
    def arg_names(self) -> List[str]:
        """Argument names in declaration order, without the leading ``%``."""
        return [n[1:] for n, _ in self.args]


@dataclass
class IRModule:
    functions: Dict[str, IRFunction] = field(default_factory=dict)

    def get_function(self, name: str) -> IRFunction:
        try:
            return self.functions[name]
        except KeyError:
            raise ValueError(f"Function '{name}' not found in module")


def walk(ops: List[Op]):
    """Pre-order traversal over an op list and all nested regions."""
    for op in ops:
        yield op
        for r in op.regions:
            yield from walk(r.ops)

"""Per-core LX scratchpad accounting, replayed on the whole-grid trace.

The reference charges every tile a core binds to an SSA name against that core's 2 MB scratchpad
and raises ``MemoryError("LX scratchpad overflow on core ...")`` when a new tile does not fit
(ktir_cpu/grid.py:253-361, ktir_cpu/memory.py:400-412).  Its rules, which this model follows:

* a tile is charged once, when first bound; further names for the same tile only add references;
* constants (``arith.constant``) occupy no LX; a consumer that needs a working copy pays for it;
* re-binding a name releases the tile it held; leaving a region (loop body, ``scf.if`` branch,
  combiner / ``linalg.generic`` body) releases every tile bound inside it;
* an operand whose only textual use this is, and which lives in the innermost scope, is released
  the moment it is fetched — before the op's own result is charged;
* ``linalg.matmul`` accumulates into its ``outs`` tile in place (no new tile), ``linalg.reduce``
  binds its result under the ``outs`` name as well, and its pairwise fold holds both halves of a
  level while combining them.

Tiles here are trace nodes, whose sizes are static; what differs between cores is which ops they
execute, so usage is tracked as one vector over the cores.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np

from .dtypes import bytes_per_elem
from .ir import Op, walk


def use_counts(ops: List[Op]) -> Dict[str, int]:
    """Textual operand uses over the function body and all nested regions
    (ktir_cpu/parser_utils.py:62-84)."""
    counts: Dict[str, int] = {}
    for op in walk(ops):
        # the reference keeps a reduce's outs as an attribute, not as an operand: it is not a "use"
        names = op.operands[:1] if op.name == "linalg.reduce" else op.operands
        for name in names:
            if isinstance(name, str):
                counts[name] = counts.get(name, 0) + 1
    return counts


_ITEM = {"i1": 1, "index": 4}


def tile_bytes(shape, dtype: str) -> int:
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    return n * (_ITEM.get(dtype) or bytes_per_elem(dtype))


class LXModel:
    def __init__(self, ncores: int, core_base: int, capacity_bytes: int, uses: Dict[str, int]):
        self.ncores, self.core_base, self.capacity = ncores, core_base, int(capacity_bytes)
        self.uses = uses
        self.used = np.zeros(ncores, np.int64)
        self.peak = np.zeros(ncores, np.int64)
        self.scopes: List[Dict[str, int]] = [{}]
        self.refs: Dict[int, int] = {}
        self.size: Dict[int, int] = {}
        self.mask: Dict[int, np.ndarray] = {}
        self.free_tiles = set()                 # handles that occupy no LX (compile-time literals)
        self.alias: Dict[int, int] = {}          # id(node) -> handle, for results that are their operand's tile
        self.keep: Dict[int, Any] = {}           # keeps handle objects alive so ids stay unique

    # -- handles -----------------------------------------------------------------------------
    def handle(self, node) -> int:
        h = self.alias.get(id(node), id(node))
        self.keep[id(node)] = node
        return h

    def same_tile(self, result, operand):
        """``result`` is the tile ``operand`` (an op that works in place and returns its operand)."""
        self.alias[id(result)] = self.handle(operand)
        self.keep[id(result)] = result

    # -- charging ----------------------------------------------------------------------------
    def _charge(self, h: int, nbytes: int, cores: np.ndarray):
        over = cores & (self.used + nbytes > self.capacity)
        if over.any():
            c = int(np.flatnonzero(over)[0])
            raise MemoryError(f"LX scratchpad overflow on core {self.core_base + c}: requested {nbytes} bytes, "
                              f"available {self.capacity - int(self.used[c])} bytes (capacity {self.capacity} bytes)")
        self.used += np.where(cores, nbytes, 0)
        np.maximum(self.peak, self.used, out=self.peak)
        self.size[h], self.mask[h] = nbytes, cores

    def _release(self, h: int):
        n = self.refs.get(h, 0) - 1
        if n > 0:
            self.refs[h] = n
            return
        self.refs.pop(h, None)
        if h in self.free_tiles:
            self.free_tiles.discard(h)
            return
        if h in self.size:
            self.used -= np.where(self.mask.pop(h), self.size.pop(h), 0)

    def transient(self, nbytes: int, cores: np.ndarray):
        """Tiles that exist only while an op runs (the halves of a reduction level)."""
        over = cores & (self.used + nbytes > self.capacity)
        if over.any():
            c = int(np.flatnonzero(over)[0])
            raise MemoryError(f"LX scratchpad overflow on core {self.core_base + c}: requested {nbytes} bytes, "
                              f"available {self.capacity - int(self.used[c])} bytes (capacity {self.capacity} bytes)")
        np.maximum(self.peak, self.used + np.where(cores, nbytes, 0), out=self.peak)

    # -- the reference's CoreContext interface -----------------------------------------------------
    def push(self):
        self.scopes.append({})

    def pop(self):
        for h in self.scopes.pop().values():
            self._release(h)

    def set_value(self, name: str, node, cores: np.ndarray, charge: bool = True):
        top = self.scopes[-1]
        old = top.pop(name, None)
        if old is not None:
            self._release(old)
        h = self.handle(node)
        top[name] = h
        first = self.refs.get(h, 0) == 0
        self.refs[h] = self.refs.get(h, 0) + 1
        if not charge or h in self.free_tiles:
            self.free_tiles.add(h)
            return
        if first:
            self._charge(h, tile_bytes(node.shape, node.dtype), cores)

    def fetch(self, name: str):
        """An operand is read: its last textual use, in the innermost scope, frees it."""
        top = self.scopes[-1]
        h = top.get(name)
        if h is not None and self.uses.get(name, 0) == 1:
            del top[name]
            self._release(h)

    def is_free(self, node) -> bool:
        return self.handle(node) in self.free_tiles

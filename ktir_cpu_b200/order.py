"""Program order of loads and stores on one core.

The reference runs a core's operations one after another (ktir_cpu/interpreter.py:196-281,
ktir_cpu/grid.py:595-613): a ``ktdp.load`` sees memory as it is at the load's position, whatever the
tile is used for later.  The device plan runs one statement per ``ktdp.store`` — all points of the
first store, then all points of the second, each statement reading its inputs when it runs.  The two
orders give the same memory unless, on one core,

* a tile is loaded BEFORE an earlier statement's store to the same bytes and used by a later
  statement (the plan would read the new bytes, the reference the old ones), or
* two statements inside the same ``scf.for`` touch the same bytes in different iterations and the
  earlier statement's access belongs to the LATER iteration (the reference interleaves the
  iterations, the plan does not).

``program_order`` finds both on the traced stores.  The first is cured by launching the later statement
first when nothing else ties the two (``x = load X; store f(x) -> X; store x -> Y`` runs as
``store x -> Y; store f(x) -> X``); what no order of whole statements cures raises ``Unsupported``.
Overlaps between different cores are the business of ``lower.check_hazards``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np

from .dtypes import bytes_per_elem
from .trace import Access, CoreOrderHazard, IndirectAccess, Node, Store, TableAccess, Unsupported, iv_full


class _Runs:
    """Byte intervals of one access at the active points of an iteration space, with the core and
    the flat point index of each."""

    def __init__(self, lo, hi, point, axes):
        self.lo, self.hi, self.point, self.axes = lo, hi, point, tuple(axes)
        inner = int(np.prod(self.axes[1:], dtype=np.int64)) if len(self.axes) > 1 else 1
        self.core = point // max(inner, 1)
        self.lo_min = int(lo.min()) if len(lo) else 0
        self.hi_max = int(hi.max()) if len(hi) else 0
        self._keys, self._shifted, self._tables = {}, None, {}

    def key(self, common: int) -> np.ndarray:
        """Trip indices of the first ``common`` loop axes, flattened (0 when there are none)."""
        k = self._keys.get(common)
        if k is None:
            if not common or len(self.axes) < 1 + common:
                k = np.zeros(len(self.point), np.int64)
            else:
                coords = np.unravel_index(self.point, self.axes)
                k = np.ravel_multi_index(coords[1:1 + common], self.axes[1:1 + common]).astype(np.int64)
            self._keys[common] = k
        return k

    def shifted(self, span: int):
        """(lo, hi) with every core moved into an address range of its own: runs of different cores never meet."""
        if self._shifted is None:
            off = self.core * span
            self._shifted = (self.lo + off, self.hi + off)
        return self._shifted

    def table(self, common: int, span: int):
        """Runs sorted by start, ends made monotone (a superset of the true overlaps), and a sparse table
        for the maximum key over a range of them."""
        t = self._tables.get(common)
        if t is None:
            lo, hi = self.shifted(span)
            order = np.argsort(lo, kind="stable")
            ka = self.key(common)[order]
            levels = [ka]
            w = 1
            while 2 * w <= len(ka):
                prev = levels[-1]
                levels.append(np.maximum(prev[:len(prev) - w], prev[w:]))
                w *= 2
            t = (lo[order], np.maximum.accumulate(hi[order]), levels)
            self._tables[common] = t
        return t


def _alloc_span(arena, view) -> Tuple[int, int]:
    base = int(np.asarray(view.base).reshape(-1)[0]) * bytes_per_elem(view.dtype)
    a = arena.find(base)
    if a is None:
        return 0, max((x.byte_hi for x in arena.allocs), default=1)
    return a.byte_lo, a.byte_hi


def _runs(acc, axes, active, arena) -> List[_Runs]:
    n = int(np.prod(axes, dtype=np.int64))
    point = np.arange(n, dtype=np.int64)
    if active is not None and tuple(active.shape) == tuple(axes):
        point = point[active.reshape(-1)]
    if isinstance(acc, Access):
        bpe = bytes_per_elem(acc.view.dtype)
        off = iv_full(acc.off, tuple(axes)).reshape(-1)[point].astype(np.int64)
        if acc.coords is not None:
            rel = acc.coords.astype(np.int64) @ np.asarray(acc.view.strides, np.int64)
            lo_rel, hi_rel = (int(rel.min()), int(rel.max())) if rel.size else (0, 0)
        else:
            steps = [(s - 1) * st for s, st in zip(acc.shape, acc.strides)]
            lo_rel, hi_rel = sum(min(x, 0) for x in steps), sum(max(x, 0) for x in steps)
        return [_Runs((off + lo_rel) * bpe, (off + hi_rel + 1) * bpe, point, axes)]
    if isinstance(acc, TableAccess):
        bpe = bytes_per_elem(acc.dtype)
        tab = np.asarray(acc.addr).reshape(-1, acc.addr.shape[-1]) if acc.addr.ndim > 1 else np.asarray(acc.addr).reshape(1, -1)
        if tab.shape[0] == n:
            tab = tab[point]
        else:                                          # one table for every point
            tab = np.broadcast_to(tab[:1], (len(point), tab.shape[1]))
        big = np.iinfo(np.int64).max
        lo = np.where(tab >= 0, tab, big).min(axis=1) if tab.shape[1] else np.zeros(len(point), np.int64)
        hi = tab.max(axis=1) if tab.shape[1] else np.full(len(point), -1)
        keep = hi >= 0
        return [_Runs(lo[keep] * bpe, (hi[keep] + 1) * bpe, point[keep], axes)]
    if isinstance(acc, IndirectAccess):
        out = []
        for view in [acc.view] + list(acc.index_views.values()):
            lo, hi = _alloc_span(arena, view)
            out.append(_Runs(np.full(len(point), lo, np.int64), np.full(len(point), hi, np.int64), point, axes))
        return out
    return []


def _loads(value: Node) -> List[Node]:
    seen, out, stack = set(), [], [value]
    while stack:
        n = stack.pop()
        if id(n) in seen:
            continue
        seen.add(id(n))
        if n.kind in ("load", "iload", "tload"):
            out.append(n)
        stack.extend(a for a in n.args if isinstance(a, Node))
        for v in n.attrs.values():                      # loop bodies keep their yields in attrs
            if isinstance(v, Node):
                stack.append(v)
            elif isinstance(v, (list, tuple)):
                stack.extend(x for x in v if isinstance(x, Node))
    return out


def _later_than(a: _Runs, b: _Runs, common: int, span: int, strict: bool) -> bool:
    """True if some run of ``a`` overlaps a run of ``b`` on the same core with a trip key (over the
    first ``common`` loops) greater than b's (``strict``) or at least b's (not ``strict``)."""
    if not len(a.lo) or not len(b.lo) or a.lo_min >= b.hi_max or b.lo_min >= a.hi_max:
        return False
    alo, ahi, levels = a.table(common, span)
    blo, bhi = b.shifted(span)
    first = np.searchsorted(ahi, blo, side="right")      # runs before `first` end at or before b starts
    last = np.searchsorted(alo, bhi, side="left")        # runs from `last` on start at or after b ends
    has = last > first
    if not has.any():
        return False
    f, l = first[has], last[has]
    lg = np.floor(np.log2(np.maximum(l - f, 1))).astype(np.int64)
    best = np.empty(len(f), np.int64)
    for g in np.unique(lg):
        m = lg == g
        t = levels[int(g)]
        best[m] = np.maximum(t[f[m]], t[l[m] - (1 << int(g))])
    kb = b.key(common)[has]
    return bool((best > kb).any() if strict else (best >= kb).any())


def program_order(stores: List[Store], arena) -> List[int]:
    """The order to launch the stores' statements in (indices into ``stores``): program order unless a
    statement has to move in front of an earlier one whose store would otherwise clobber a tile it
    loaded first.  Raises ``Unsupported`` when no order of whole statements reproduces what a core of
    the reference sees (see the module docstring)."""
    if len(stores) < 2:
        return list(range(len(stores)))
    span = max((a.byte_hi for a in arena.allocs), default=0) + 1
    writes = [_runs(st.target, st.axes, st.active, arena) for st in stores]
    index_reads: List[List[_Runs]] = []
    for st, w in zip(stores, writes):
        # an indirect store reads its index tensors when it runs; only the parent view is written
        index_reads.append(w[1:] if isinstance(st.target, IndirectAccess) else [])
        if isinstance(st.target, IndirectAccess):
            del w[1:]
    reads: List[List[Tuple[_Runs, int, int]]] = []       # per store: (runs, stores traced before the load, loop depth of the load)
    seen = {}                                            # a tile loaded once and stored several times: one set of runs
    for j, st in enumerate(stores):
        rs = []
        for node in _loads(st.value):
            own = tuple(node.attrs.get("axes", st.axes))
            axes, active = (tuple(st.axes), st.active) if len(own) <= len(st.axes) else (own, None)
            before = int(node.attrs.get("stores_before", j))
            k = (id(node), axes, None if active is None else active.tobytes())
            if k not in seen:
                seen[k] = _runs(node.attrs["access"], axes, active, arena)
            rs.extend((r, before, len(own) - 1) for r in seen[k])
        rs.extend((r, j, len(st.axes) - 1) for r in index_reads[j])
        reads.append(rs)
    # (cured by tracing the loop iteration by iteration: ``lower.lower_core_groups``)
    inverted = CoreOrderHazard("two statements inside one scf.for touch the same memory in different iterations, the "
                               "earlier statement in the later iteration: the statements cannot run one after the other")
    count = len(stores)
    commons = {}
    for j in range(1, count):
        for i in range(j):
            c = 0
            for x, y in zip(stores[i].loop_path, stores[j].loop_path):
                if x != y:
                    break
                c += 1
            commons[i, j] = c
    # What can force a statement in front of an earlier one, or rule every order out: a tile loaded before an
    # earlier store to its bytes, and accesses of two statements of one loop that meet in the wrong iterations.
    bwd = set()
    for j in range(1, count):
        for i in range(j):
            common = commons[i, j]
            stale = False
            for wa in writes[i]:
                for rb, before, depth in reads[j]:
                    # B's load against A's store.  Run after A, B sees every byte A wrote; the reference shows it
                    # those written before the load: in an earlier iteration of the loops both sit in, or in
                    # the same one if the load comes after A's store.
                    c = min(common, depth)
                    if c and _later_than(wa, rb, c, span, strict=True):
                        raise inverted
                    if before <= i and not stale:
                        stale = _later_than(wa, rb, c, span, strict=False)     # same iteration: B must read first
                if common:
                    for wb in writes[j]:
                        if _later_than(wa, wb, common, span, strict=True):
                            raise inverted
            for ra, _, depth in reads[i]:
                c = min(common, depth)
                if c:
                    for wb in writes[j]:
                        if _later_than(ra, wb, c, span, strict=True):
                            raise inverted
            if stale:
                bwd.add((i, j))
    if not bwd:
        return list(range(count))                         # program order works as it is

    # Some statement has to move: find what else ties the pairs together (any other overlap keeps program order)
    after = {j: set() for j in range(count)}              # after[j]: statements that must run before j
    for j in range(1, count):
        for i in range(j):
            common = commons[i, j]
            fwd = False
            for wa in writes[i]:
                for rb, before, depth in reads[j]:
                    c = min(common, depth)
                    if before <= i:
                        fwd = fwd or (c > 0 and _later_than(rb, wa, c, span, strict=True))   # bytes of earlier iterations
                    else:
                        fwd = fwd or _later_than(rb, wa, c, span, strict=False)
                for wb in writes[j]:
                    fwd = fwd or _later_than(wb, wa, common, span, strict=False)          # B's bytes land last
            for ra, _, depth in reads[i]:
                c = min(common, depth)
                for wb in writes[j]:
                    fwd = fwd or _later_than(wb, ra, c, span, strict=False)               # A reads before B writes
            if fwd and (i, j) in bwd:
                raise Unsupported("a tile is loaded before an earlier store to the same memory and used after it, "
                                  "by a statement that also depends on that store: the statements cannot run one "
                                  "after the other")
            if (i, j) in bwd:
                after[i].add(j)
            elif fwd:
                after[j].add(i)
    order, done = [], set()
    while len(order) < len(stores):
        ready = [k for k in range(len(stores)) if k not in done and after[k] <= done]
        if not ready:
            raise Unsupported("tiles loaded before earlier stores to the same memory and used after them tie the "
                              "statements into a cycle: they cannot run one after the other")
        order.append(ready[0])
        done.add(ready[0])
    return order

"""Lowering of statements that mix elementwise ops with reductions along the rows of a tile.

Layer norm, RMS norm and the softmax forms the dedicated kernel does not take have the same shape of
tile program: ``linalg.reduce`` over the last dimension (ktir_cpu/dialects/linalg_ops.py:136-246), a few
ops on the reduced ``[rows]`` tile (scale by 1/n, add eps, rsqrt ...), a broadcast back to the full tile
(linalg_ops.py:349-465) and elementwise ops around all of it.  ``RowProgramStatement`` turns such a DAG
into the phases of ``ktb_launch_row_program``:

* every ``reduce`` node becomes a reduction phase — a register program for the reduced expression,
  evaluated per 8-element vector of a row, and the fold;
* every broadcast of a per-row value becomes a *row scalar* — a register program over the reduction
  results, evaluated once per row — and enters the later programs as one more input register;
* the stored expression becomes the output phase.

Rounding follows the tile dtypes as in the elementwise lowering (an op on an f16 tile rounds to f16).
Anything that does not fit — other reductions, tiles whose rows are not a power of two long, more
operands, scalars or registers than the kernel has — raises ``Unsupported`` and the statement runs
step by step.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Tuple

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem
from .lower import (F_DT, ArenaMap, Footprint, Statement, _VM_BIN, _VM_UN, _access_offsets, _copy_args,
                    _order_item_table, _points, strip_views, tile_geom)
from .trace import Access, Node, Store, Unsupported

_RED_OPS = {"arith.addf": "add", "arith.maximumf": "max", "arith.maxnumf": "maxnum", "arith.maxf": "max"}


def _prod(shape) -> int:
    return int(np.prod(shape)) if len(shape) else 1


def has_row_reduce(n: Node, seen=None) -> bool:
    seen = seen if seen is not None else set()
    if id(n) in seen:
        return False
    seen.add(id(n))
    return n.kind == "reduce" or any(isinstance(a, Node) and has_row_reduce(a, seen) for a in n.args)


def _canon(n: Node) -> Node:
    """The node whose register a node shares: reshapes, casts to f32 (f16 values are exact in the f32
    registers) and full-shape broadcasts of constants add no op."""
    while True:
        n = strip_views(n)
        if n.kind == "cast" and n.dtype == "f32" and n.args[0].dtype in F_DT:
            n = n.args[0]
        elif n.kind == "bcast" and strip_views(n.args[0]).kind == "const":
            n = n.args[0]
        elif n.kind == "extract" and _prod(n.args[0].shape) == 1:
            n = n.args[0]
        else:
            return n


class _Compiler:
    """Register program of one expression.  ``leaves`` maps node ids to input registers; temporaries are
    handed back as soon as their last user has been emitted, so long chains fit the eight registers."""

    def __init__(self, leaves: Dict[int, int], n_in: int, elems: int, immediates: bool = False):
        """``immediates``: a constant operand of a two-operand op rides in the op itself (row-value programs, whose
        evaluator takes them; saves the CONST op in front)."""
        self.leaves, self.n_in, self.elems, self.immediates = leaves, n_in, elems, immediates
        self.ops: List[Tuple[int, int, int, int, int, float]] = []
        self.reg_of: Dict[int, int] = {}
        self.uses: Dict[int, int] = {}
        self.free = list(range(R.VM_REGS - 1, n_in - 1, -1))
        self.used_inputs = set()

    def _count(self, n: Node):
        n = _canon(n)
        self.uses[id(n)] = self.uses.get(id(n), 0) + 1
        if self.uses[id(n)] > 1 or id(n) in self.leaves:
            return
        for a in n.args:
            self._count(a)

    def _alloc(self) -> int:
        if not self.free:
            raise Unsupported("row program needs more than 8 live registers")
        return self.free.pop()

    def _release(self, n: Node):
        n = _canon(n)
        self.uses[id(n)] -= 1
        r = self.reg_of.get(id(n))
        if self.uses[id(n)] == 0 and r is not None and r >= self.n_in:
            self.free.append(r)

    def _emit(self, code: str, dst: int, a=0, b=0, c=0, imm=0.0, r16=False):
        if len(self.ops) >= R.VM_MAX_OPS:
            raise Unsupported("row program phase longer than 12 ops")
        self.ops.append((R.VM[code] | (R.VM_ROUND16 if r16 else 0), dst, a, b, c, float(imm)))

    def _visit(self, n: Node) -> int:
        n = _canon(n)
        if id(n) in self.leaves:
            self.used_inputs.add(self.leaves[id(n)])
            return self.leaves[id(n)]
        if id(n) in self.reg_of:
            return self.reg_of[id(n)]
        r16 = n.dtype == "f16"
        if n.kind == "const":
            if n.attrs.get("list") is not None:
                raise Unsupported("dense list constant in a row program")
            v = n.attrs["value"]
            v = float(np.float16(v)) if n.dtype == "f16" else float(np.float32(v))
            r = self._alloc()
            self._emit("CONST", r, imm=v)
        elif n.kind == "cast":
            if n.args[0].dtype not in F_DT or n.dtype not in F_DT:
                raise Unsupported(f"cast {n.args[0].dtype}->{n.dtype} in a row program")
            src = self._visit(n.args[0])
            self._release(n.args[0])
            r = self._alloc()
            self._emit("MOV", r, src, r16=True)
        elif n.kind == "ew":
            op = n.attrs["op"]
            if n.dtype not in F_DT:
                raise Unsupported(f"{op} producing {n.dtype} in a row program")
            for a in n.args:
                ca = _canon(a)
                if ca.kind != "const" and id(ca) not in self.leaves and _prod(ca.shape) != self.elems:
                    raise Unsupported("operand of another shape in a row program")
            imm_at = None
            if self.immediates and op in _VM_BIN and len(n.args) == 2:
                consts = [k for k, a in enumerate(n.args) if _canon(a).kind == "const" and _canon(a).attrs.get("list") is None]
                if len(consts) == 1:
                    imm_at = consts[0]
            if imm_at is not None:
                other = n.args[1 - imm_at]
                ro = self._visit(other)
                self._release(other)
                self.uses[id(_canon(n.args[imm_at]))] -= 1
                cn = _canon(n.args[imm_at])
                v = float(np.float16(cn.attrs["value"])) if cn.dtype == "f16" else float(np.float32(cn.attrs["value"]))
                r = self._alloc()
                self.ops.append((R.VM[_VM_BIN[op]] | (R.VM_ROUND16 if r16 else 0) | (R.VM_IMM_A if imm_at == 0 else R.VM_IMM_B),
                                 r, ro, ro, 0, v))
                if len(self.ops) > R.VM_MAX_OPS:
                    raise Unsupported("row program phase longer than 12 ops")
                self.reg_of[id(n)] = r
                return r
            regs = [self._visit(a) for a in n.args]
            for a in n.args:
                self._release(a)
            r = self._alloc()
            if op in _VM_BIN:
                self._emit(_VM_BIN[op], r, regs[0], regs[1], r16=r16)
            elif op in _VM_UN:
                self._emit(_VM_UN[op], r, regs[0], r16=r16)
            elif op == "math.fma":
                self._emit("FMA", r, regs[0], regs[1], regs[2], r16=r16)
            else:
                raise Unsupported(f"{op} in a row program")
        else:
            raise Unsupported(f"{n.kind} node in a row program")
        self.reg_of[id(n)] = r
        return r

    def compile(self, root: Node) -> R.VmProgram:
        self._count(root)
        res = self._visit(root)
        p = R.VmProgram()
        p.n_in, p.n_ops, p.result_reg = self.n_in, len(self.ops), res
        for i, op in enumerate(self.ops):
            p.ops[i] = R.VmOp(*op)
        return p


def _first_reduce(n: Node, seen=None):
    seen = seen if seen is not None else set()
    if id(n) in seen:
        return None
    seen.add(id(n))
    if n.kind == "reduce":
        return n
    for a in n.args:
        if isinstance(a, Node):
            r = _first_reduce(a, seen)
            if r is not None:
                return r
    return None


def _signature(n: Node, loads: List[Node], fixed: Dict[int, int]):
    """Structure of an expression with its loads numbered in the order they are met (``loads`` collects
    them); nodes listed in ``fixed`` (row values) count as themselves."""
    n = _canon(n)
    if id(n) in fixed:
        return ("S", id(n))
    if n.kind == "load":
        loads.append(n)
        return ("L", len(loads) - 1, n.dtype)
    if n.kind == "const":
        return ("C", repr(n.attrs.get("value")), n.dtype, n.attrs.get("list") is not None)
    if n.kind == "bcast":                                # of a row value: same node or no match
        return ("B", id(n))
    if n.kind in ("ew", "cast"):
        return (n.kind, n.attrs.get("op"), n.dtype, tuple(_signature(a, loads, fixed) for a in n.args))
    return ("?", id(n))


def _block_chain(src: Node):
    """``src = (((init + t_0) + t_1) + ... + t_{B-1})``, the accumulator a column-blocked kernel carries
    through its loop over the blocks of a row: (init value, [t_0 ...], adds round to f16) or None."""
    terms = []
    n = _canon(src)
    dtype = n.dtype
    while n.kind == "ew" and n.attrs.get("op") == "arith.addf" and len(n.args) == 2 and n.dtype == dtype:
        terms.append(n.args[1])
        n = _canon(n.args[0])
    if n.kind != "const" or n.attrs.get("list") is not None or len(terms) < 2:
        return None
    terms.reverse()
    return float(n.attrs["value"]), terms, dtype == "f16"


class _Operand:
    """One operand tile of the statement: where it lives per item, how its rows and column blocks advance."""

    def __init__(self, acc: Access, offs: np.ndarray, shared_row: bool, blk_stride: int):
        self.acc, self.offs, self.shared_row, self.blk_stride = acc, offs, shared_row, blk_stride

    def key(self):
        return (self.acc.view.dtype, tuple(self.acc.shape), tuple(self.acc.strides), self.shared_row, self.blk_stride,
                self.offs.tobytes())


class RowProgramStatement(Statement):
    kind = "row_program"

    def __init__(self, dev: R.Device, store: Store, arena: ArenaMap, stmt_id: int):
        tgt = store.target
        if not isinstance(tgt, Access) or tgt.coords is not None:
            raise Unsupported("row program needs a plain rectangular destination tile")
        # the tile that is reduced gives the row length; the stored tile is either of that shape or holds
        # one value per row
        first = _first_reduce(store.value)
        src_shape = tuple(strip_views(first.args[0]).shape)
        if not src_shape:
            raise Unsupported("reduction of a scalar")
        cols, full = int(src_shape[-1]), _prod(src_shape)
        if cols < 8 or cols > 16384 or cols & (cols - 1):
            raise Unsupported(f"row program over rows of {cols} elements (power of two in [8, 16384] only)")
        rows_total = full // cols
        per_row = _prod(tgt.shape) == rows_total and rows_total != full
        if not per_row and _prod(tgt.shape) != full:
            raise Unsupported("stored tile is neither the reduced tile's shape nor one value per row")

        # --- iteration points.  A statement inside a loop over the column blocks of a row (its last axis) whose
        # reductions walk the same blocks is taken row by row: the block axis moves into the operands.
        axes = tuple(store.axes)
        sel_all, cores_all = _points(store)
        chains = {}

        def find_chains(n: Node, seen):
            n = strip_views(n)
            if id(n) in seen:
                return
            seen.add(id(n))
            if n.kind == "reduce":
                c = _block_chain(n.args[0])
                if c is not None:
                    chains[id(n)] = c
            for a_ in n.args:
                if isinstance(a_, Node):
                    find_chains(a_, seen)

        find_chains(store.value, set())
        n_blocks = 1
        if chains:
            counts = {len(c[1]) for c in chains.values()}
            if len(counts) != 1:
                raise Unsupported("blocked reductions over different numbers of column blocks")
            n_blocks = counts.pop()
        absorb = bool(chains) and not per_row and len(axes) >= 2 and axes[-1] == n_blocks and \
            (store.active is None or bool((store.active == store.active[..., :1]).all()))
        if chains and not per_row and not absorb:
            raise Unsupported("blocked reductions next to a stored tile that does not walk the same column blocks")
        if absorb:
            keep = (sel_all % n_blocks) == 0                # points with block index 0 stand for their row
            sel, cores = sel_all[keep], cores_all[keep]
        else:
            sel, cores = sel_all, cores_all

        def offsets_of(acc: Access, own_axes) -> Tuple[np.ndarray, int]:
            """Element offset of the tile at every item, and the step between column blocks (0: none)."""
            from .trace import iv_full
            offs_full = np.asarray(iv_full(acc.off, axes)).reshape(-1).astype(np.int64)
            offs = offs_full[sel]
            if not absorb:
                return offs, 0
            cube = offs_full.reshape(-1, n_blocks)
            step = cube[:, 1:] - cube[:, :-1]
            if step.size and (step != step.flat[0]).any():
                raise Unsupported("tile that does not advance evenly over the column blocks")
            return offs, int(step.flat[0]) if step.size else 0

        operands: List[_Operand] = []
        op_index: Dict[tuple, int] = {}

        def operand(acc: Access, shared: bool, blk_stride=None) -> int:
            if acc.coords is not None:
                raise Unsupported("coordinate-set tile in a row program")
            offs, step = offsets_of(acc, None)
            o = _Operand(acc, offs, shared, step if blk_stride is None else blk_stride)
            k = op_index.get(o.key())
            if k is None:
                k = op_index[o.key()] = len(operands)
                operands.append(o)
            return k

        # --- the DAG: operand tiles, reductions (in dependency order), broadcast row values -------------
        leaves: Dict[int, int] = {}         # node id -> operand index (row values are added below)
        reduces: List[Node] = []
        scalars: List[Node] = []            # bcast nodes whose argument is a per-row value
        blocked_terms: Dict[int, Node] = {} # reduce node id -> the term evaluated per block
        seen = set()

        def is_row_value(n: Node) -> bool:
            return _prod(strip_views(n).shape) == rows_total and rows_total != full

        def walk(n: Node):
            n = strip_views(n)
            if id(n) in seen:
                return
            seen.add(id(n))
            if n.kind == "load":
                if n.dtype not in F_DT:
                    raise Unsupported(f"{n.dtype} tile in a row program")
                if _prod(n.shape) != full:
                    raise Unsupported("operand tile of another shape in a row program")
                leaves[id(n)] = operand(n.attrs["access"], False)
                return
            if n.kind == "reduce":
                dims = n.attrs.get("dims")
                src = strip_views(n.args[0])
                if _prod(src.shape) != full or dims is None or tuple(dims) != (len(src.shape) - 1,) or \
                        src.shape[-1] != cols:
                    raise Unsupported("reduction that is not along the rows of the reduced tile")
                if n.attrs["op"] not in _RED_OPS:
                    raise Unsupported(f"row reduction with {n.attrs['op']}")
                chain = chains.get(id(n))
                if chain is None:
                    walk(n.args[0])
                else:
                    # every term must be the first one with its loads moved on by a whole number of blocks
                    _, terms, _ = chain
                    fixed = {}
                    first_loads: List[Node] = []
                    for t_ in terms:                     # row values inside the terms come first
                        collect_row_values(t_)
                    sig0 = _signature(terms[0], first_loads, fixed)
                    steps = [None] * len(first_loads)
                    for j_, t_ in enumerate(terms[1:], 1):
                        lj: List[Node] = []
                        if _signature(t_, lj, fixed) != sig0 or len(lj) != len(first_loads):
                            raise Unsupported("blocked reduction whose blocks are not computed alike")
                        for q, (l0, l1) in enumerate(zip(first_loads, lj)):
                            a0, a1 = l0.attrs["access"], l1.attrs["access"]
                            if (a0.view.dtype, tuple(a0.shape), tuple(a0.strides)) != (a1.view.dtype, tuple(a1.shape), tuple(a1.strides)):
                                raise Unsupported("blocked reduction over tiles of different layouts")
                            o0, _ = offsets_of(a0, None)
                            o1, _ = offsets_of(a1, None)
                            d = o1 - o0
                            if d.size and (d != d.flat[0]).any():
                                raise Unsupported("blocked reduction whose blocks are not evenly spaced")
                            step = int(d.flat[0]) if d.size else 0
                            if step % j_ or (steps[q] is not None and steps[q] != step // j_):
                                raise Unsupported("blocked reduction whose blocks are not evenly spaced")
                            steps[q] = step // j_
                    for l0, st_ in zip(first_loads, steps):
                        if l0.dtype not in F_DT or _prod(l0.shape) != full:
                            raise Unsupported("operand tile of another shape in a row program")
                        leaves[id(l0)] = operand(l0.attrs["access"], False, blk_stride=st_ or 0)
                    blocked_terms[id(n)] = terms[0]
                reduces.append(n)            # post-order: what it depends on is already listed
                return
            if n.kind == "bcast" and strip_views(n.args[0]).kind != "const":
                if is_row_value(n.args[0]) and _prod(n.shape) == full and \
                        (rows_total == 1 or list(n.attrs.get("dims", [])) == [len(n.shape) - 1]):
                    walk(n.args[0])
                    scalars.append(n)
                    return
                src = _canon(n.args[0])
                if src.kind == "load" and _prod(n.shape) == full and _prod(src.shape) == cols and rows_total > 1 and \
                        sorted(n.attrs.get("dims", [])) == list(range(len(n.shape) - 1)):
                    # one row of weights for all rows of the tile: an operand whose rows do not advance
                    if src.dtype not in F_DT:
                        raise Unsupported(f"{src.dtype} tile in a row program")
                    leaves[id(n)] = operand(src.attrs["access"], True)
                    return
                raise Unsupported("broadcast that is neither a per-row value along the columns nor a shared row")
            if n.kind in ("const", "cast", "ew", "bcast", "extract"):
                for a_ in n.args:
                    walk(a_)
                return
            raise Unsupported(f"{n.kind} node in a row program")

        def collect_row_values(n: Node):
            """Row values used inside a blocked term are walked (their reductions come first) without
            registering the term's own loads block by block."""
            n = strip_views(n)
            if n.kind == "bcast" and strip_views(n.args[0]).kind != "const" and is_row_value(n.args[0]):
                walk(n)
                return
            for a_ in n.args:
                if isinstance(a_, Node):
                    collect_row_values(a_)

        walk(store.value)
        if len(reduces) > R.RP_MAX_RED or len(scalars) > R.RP_MAX_SCAL or len(operands) > R.VM_MAX_IN or not operands:
            raise Unsupported("row program with more reductions, row values or operand tiles than the kernel takes")
        n_in, n_red = len(operands), len(reduces)
        if n_in + len(scalars) >= R.VM_REGS:
            raise Unsupported("row program with too many inputs")
        red_index = {id(r): k for k, r in enumerate(reduces)}

        # --- row scalars: programs over the reduction results ------------------------------------------
        def last_reduce(n: Node, memo) -> int:
            n = strip_views(n)
            if id(n) not in memo:
                memo[id(n)] = red_index[id(n)] if id(n) in red_index else \
                    max([last_reduce(a_, memo) for a_ in n.args if isinstance(a_, Node)] + [-1])
            return memo[id(n)]

        def scalar_program(root: Node) -> R.VmProgram:
            return _Compiler(dict(red_index), n_red, rows_total, immediates=True).compile(root)

        scal_progs = sorted(((last_reduce(s_.args[0], {}), k, scalar_program(s_.args[0]), s_) for k, s_ in enumerate(scalars)),
                            key=lambda x: x[:2])
        for k, (_, _, _, s_) in enumerate(scal_progs):
            leaves[id(s_)] = n_in + k

        # --- vector programs ----------------------------------------------------------------------------
        def vector_program(root: Node):
            comp = _Compiler(leaves, n_in + len(scalars), full)
            prog = comp.compile(root)
            return prog, sum(1 << r for r in comp.used_inputs if r < n_in)

        self.args = a = R.RowProgArgs()
        a.n_in, a.n_red, a.n_scal, a.out_per_row, a.n_blocks = n_in, n_red, len(scal_progs), int(per_row), n_blocks
        for k, r in enumerate(reduces):
            ph = a.red[k]
            term = blocked_terms.get(id(r))
            ph.prog, ph.load_mask = vector_program(term if term is not None else r.args[0])
            ph.op = R.RP_OPS[_RED_OPS[r.attrs["op"]]]
            ph.round16 = 1 if r.dtype == "f16" else 0
            if term is not None:
                init, _, r16 = chains[id(r)]
                ph.blocked, ph.acc_round16, ph.acc_init = 1, int(r16), init
        for k, (ready, _, prog, _) in enumerate(scal_progs):
            a.scal[k].prog, a.scal[k].ready_after = prog, ready
        if per_row:
            a.out.prog, a.out.load_mask = scalar_program(store.value), 0
        else:
            a.out.prog, a.out.load_mask = vector_program(store.value)
            a.out.blocked = int(absorb)

        # --- geometry: one table row per item, operand tiles then the destination -------------------------
        full_ops = [o for o in operands if not o.shared_row]
        if not full_ops:
            raise Unsupported("row program without an operand tile of the reduced shape")
        expand = len(tile_geom(full_ops[0].acc, False).lead) != 1
        geoms = [tile_geom(o.acc, False if o.shared_row else expand) for o in operands]
        g0 = geoms[[o.shared_row for o in operands].index(False)]
        for g, o in zip(geoms, operands):
            if o.shared_row and (g.rows, g.cols, len(g.lead)) != (1, cols, 1):
                raise Unsupported("shared operand row of another length")
            if not o.shared_row and (g.rows, g.cols, len(g.lead)) != (g0.rows, g0.cols, len(g0.lead)):
                raise Unsupported("operand tiles with another row structure in a row program")
        n_lead = len(g0.lead)
        if g0.cols != cols or ((any(o.shared_row for o in operands) or n_blocks > 1) and n_lead != 1):
            raise Unsupported("operand tiles with another row structure in a row program")
        out_step = 0
        if per_row:
            # the stored tile has one element per row of an operand tile; its elements sit `stride` apart
            big = [d for d, n_ in enumerate(tgt.shape) if n_ > 1]
            if len(big) > 1 or n_lead != 1 or (big and tgt.shape[big[0]] != g0.rows):
                raise Unsupported("per-row result tile of more than one dimension")
            out_stride = int(tgt.strides[big[0]]) if big else 1
            out_offs, _ = offsets_of(tgt, None)
        else:
            go = tile_geom(tgt, expand)
            if (go.rows, go.cols, len(go.lead)) != (g0.rows, g0.cols, n_lead):
                raise Unsupported("stored tile with another row structure than the operands")
            out_offs, out_step = offsets_of(tgt, None)
        table = np.empty((len(sel) * n_lead, n_in + 1), np.int64)
        self.fps: List[Footprint] = []
        blocks = np.arange(n_blocks, dtype=np.int64)

        def footprint(offs, g, step, bpe, write):
            rs = (offs[:, None, None] + np.arange(g.rows, dtype=np.int64)[None, :, None] * g.row_stride +
                  blocks[None, None, :] * step).reshape(-1) * bpe
            rep = n_lead * g.rows * n_blocks
            self.fps.append(Footprint(rs, rs + g.cols * bpe, np.repeat(sel, rep), np.repeat(cores, rep), write, stmt_id))

        for k, (o, g) in enumerate(zip(operands, geoms)):
            bpe = bytes_per_elem(o.acc.view.dtype)
            offs = (o.offs[:, None] + g.lead[None, :]).reshape(-1)
            table[:, k] = offs
            a.dtype[k] = R.DTYPE_CODE[o.acc.view.dtype]
            a.blk_stride[k] = o.blk_stride
            if len(offs):
                arena.check_range(int(offs.min()), int(offs.max()) + (g.rows - 1) * g.row_stride +
                                  (n_blocks - 1) * max(o.blk_stride, 0) + g.cols, o.acc.view.dtype, "Read from")
            footprint(offs, g, o.blk_stride, bpe, False)
            a.row_stride[k] = 0 if o.shared_row else (max(g.row_stride, 8) if g.rows == 1 else g.row_stride)
            if (offs % 8).any() or (g.rows > 1 and g.row_stride % 8) or o.blk_stride % 8 or o.blk_stride < 0:
                raise Unsupported("row program needs 16-byte aligned rows")
        bpe = bytes_per_elem(tgt.view.dtype)
        a.dtype[n_in] = R.DTYPE_CODE[tgt.view.dtype]
        if per_row:
            table[:, n_in] = out_offs
            if len(out_offs):
                arena.check_range(int(out_offs.min()), int(out_offs.max()) + (g0.rows - 1) * out_stride + 1,
                                  tgt.view.dtype, "Scatter to")
            rs = (out_offs[:, None] + np.arange(g0.rows, dtype=np.int64)[None, :] * out_stride).reshape(-1) * bpe
            self.fps.append(Footprint(rs, rs + bpe, np.repeat(sel, g0.rows), np.repeat(cores, g0.rows), True, stmt_id))
            a.row_stride[n_in] = out_stride
        else:
            offs = (out_offs[:, None] + go.lead[None, :]).reshape(-1)
            table[:, n_in] = offs
            a.blk_stride[n_in] = out_step
            if len(offs):
                arena.check_range(int(offs.min()), int(offs.max()) + (go.rows - 1) * go.row_stride +
                                  (n_blocks - 1) * max(out_step, 0) + go.cols, tgt.view.dtype, "Scatter to")
            footprint(offs, go, out_step if absorb else 0, bpe, True)
            a.row_stride[n_in] = max(go.row_stride, 8) if go.rows == 1 else go.row_stride
            if (offs % 8).any() or (go.rows > 1 and go.row_stride % 8) or out_step % 8 or out_step < 0 or \
                    (absorb and out_step == 0):
                raise Unsupported("row program needs 16-byte aligned rows")
        a.n_items, a.rows_per_item, a.cols = table.shape[0], g0.rows, cols
        self.table = table
        self._sel, self._n_lead, self._dev, self.rounds = sel, n_lead, dev, None
        self.stores = [store]
        self._side_ctx = None if per_row or n_lead != 1 else dict(
            red_index=red_index, n_red=n_red, rows_total=rows_total, axes=axes, cores=cores, rows=g0.rows,
            div=n_blocks if absorb else 1, arena=arena, stmt_id=stmt_id)
        self.dev_table = dev.upload(table)
        a.dev_item_offsets = self.dev_table
        self.device_arrays = [self.dev_table]
        self._n_op = n_in + 1
        self._bytes = int(table.shape[0]) * g0.rows * n_blocks * (
            cols * sum(bytes_per_elem(o.acc.view.dtype) for o in operands) + (0 if per_row else cols) * bpe)

    def try_absorb(self, side: Store) -> bool:
        """Take over a neighbouring statement that stores one value per row made of this statement's own reduction
        results (the Mean and Rstd vectors next to a layer norm's output,
        examples/triton-ktir/layernorm_fwd_ktir.mlir:127-128): the kernel writes it from the sums it has anyway
        instead of a second launch re-reading the rows.  False (and nothing changed) if it does not fit."""
        c, a = self._side_ctx, self.args
        tgt = side.target
        if c is None or a.n_side >= R.RP_MAX_SIDE or not isinstance(tgt, Access) or tgt.coords is not None or \
                tgt.view.dtype not in F_DT:
            return False
        rows_total, axes = c["rows_total"], c["axes"]
        if _prod(tgt.shape) != rows_total:
            return False
        # the same iteration points: the side store sits at this statement's loop depth, or one level above the
        # loop over column blocks this statement has absorbed
        s_axes = tuple(side.axes)
        if s_axes != (axes if c["div"] == 1 else axes[:-1]):
            return False
        s_sel, s_cores = _points(side)
        if len(s_sel) != len(self._sel) or (s_sel != self._sel // c["div"]).any() or (s_cores != c["cores"]).any():
            return False
        # its value: a program over this statement's reduction results, nothing else
        red_index = c["red_index"]

        def only_known(n: Node, seen) -> bool:
            n = strip_views(n)
            if id(n) in seen or id(n) in red_index:
                return True
            seen.add(id(n))
            if n.kind == "reduce" or n.kind == "load" or n.kind not in ("const", "cast", "ew", "bcast", "extract"):
                return False
            return all(only_known(x, seen) for x in n.args if isinstance(x, Node))

        if not only_known(side.value, set()):
            return False
        try:
            prog = _Compiler(dict(red_index), c["n_red"], rows_total, immediates=True).compile(side.value)
        except Unsupported:
            return False
        big = [d for d, n_ in enumerate(tgt.shape) if n_ > 1]
        if len(big) > 1 or (big and tgt.shape[big[0]] != c["rows"]):
            return False
        stride = int(tgt.strides[big[0]]) if big else 1
        from .trace import iv_full
        offs = np.asarray(iv_full(tgt.off, s_axes)).reshape(-1).astype(np.int64)[s_sel]
        bpe = bytes_per_elem(tgt.view.dtype)
        rs = (offs[:, None] + np.arange(c["rows"], dtype=np.int64)[None, :] * stride).reshape(-1) * bpe
        # moving the store into this launch must not change what anything reads: its bytes are apart from
        # everything the statement touches
        for f in self.fps:
            if len(f.starts) and len(rs) and _runs_overlap(rs, rs + bpe, f.starts, f.ends):
                return False
        if len(offs):
            c["arena"].check_range(int(offs.min()), int(offs.max()) + (c["rows"] - 1) * stride + 1, tgt.view.dtype,
                                   "Scatter to")
        k = a.n_side
        a.side[k].prog, a.side[k].row_stride, a.side[k].dtype = prog, stride, R.DTYPE_CODE[tgt.view.dtype]
        a.n_side = k + 1
        self.fps.append(Footprint(rs, rs + bpe, np.repeat(self._sel, c["rows"]), np.repeat(c["cores"], c["rows"]),
                                  True, c["stmt_id"]))
        self.table = np.ascontiguousarray(np.concatenate([self.table, offs[:, None]], axis=1))
        self._dev.free(self.dev_table)
        self.dev_table = self._dev.upload(self.table)
        a.dev_item_offsets = self.dev_table
        self.device_arrays = [self.dev_table]
        self._n_op += 1
        self._bytes += len(rs) * bpe
        self.stores.append(side)
        return True

    def renumber(self, stmt_id: int):
        for f in self.fps:
            f.stmt = stmt_id
        if self._side_ctx is not None:
            self._side_ctx["stmt_id"] = stmt_id

    def launch(self, dev, arena_ptr):
        self.args.arena = arena_ptr
        if self.rounds:
            for lo, hi in self.rounds:
                sub = _copy_args(self.args)
                sub.dev_item_offsets = self.dev_table + lo * self._n_op * 8
                sub.n_items = hi - lo
                dev.check(dev.lib.ktb_launch_row_program(dev.h, C.byref(sub)))
            return
        dev.check(dev.lib.ktb_launch_row_program(dev.h, C.byref(self.args)))

    def order_points(self, rounds: Dict[int, int]):
        _order_item_table(self, self._sel, self._n_lead, rounds, self._dev)

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


def _runs_overlap(s0, e0, s1, e1) -> bool:
    """True if some run [s0, e0) meets some run [s1, e1)."""
    if s0.min() >= e1.max() or s1.min() >= e0.max():
        return False
    order = np.argsort(s1, kind="stable")
    s1, e1 = s1[order], np.maximum.accumulate(e1[order])
    k = np.searchsorted(s1, e0, side="left") - 1          # last run of the second set that starts before each e0
    ok = k >= 0
    return bool((e1[k[ok]] > s0[ok]).any())


def try_lower_row_program(dev, store: Store, arena: ArenaMap, stmt_id: int):
    """The fused row kernel for a statement with row reductions, or None if it has none."""
    if not isinstance(store.target, Access) or not has_row_reduce(store.value):
        return None
    return RowProgramStatement(dev, store, arena, stmt_id)

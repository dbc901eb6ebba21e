"""Lowering of statements that move whole rows through an index tensor.

``ktdp.load`` / ``ktdp.store`` through an indirect access tile resolve, per
point of the variable space, one coordinate per dimension of the parent view —
either an affine expression of the point or a value read from an index view
(ktir_cpu/ops/memory_ops.py:488-576).  The device kernels handle the common
blocked form: a tile of R rows x C contiguous columns whose row address is
``base + IDX[i0 + r * istride] * mult + r * rstride`` (MoE / paged-attention /
embedding-style gathers and scatters).  Anything else raises ``Unsupported``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem
from .lower import ArenaMap, Footprint, ProgramBuilder, Statement, _points
from .trace import Access, IndirectAccess, Node, Store, Unsupported, iv_bin, iv_full


def _lin(expr, n_vars: int, ssa) -> Tuple[List[int], Any]:
    """expr -> (integer coefficient per variable, constant part as an integer value)."""
    k = expr[0]
    if k == "const":
        return [0] * n_vars, int(expr[1])
    if k == "var":
        c = [0] * n_vars
        c[expr[1]] = 1
        return c, 0
    if k == "ssa":
        return [0] * n_vars, ssa[expr[1]]
    if k == "neg":
        c, b = _lin(expr[1], n_vars, ssa)
        return [-x for x in c], iv_bin(lambda a, _: -a, b, 0)
    ca, ba = _lin(expr[1], n_vars, ssa)
    cb, bb = _lin(expr[2], n_vars, ssa)
    if k in ("add", "sub"):
        s = 1 if k == "add" else -1
        return [x + s * y for x, y in zip(ca, cb)], iv_bin(lambda a, b: a + s * b, ba, bb)
    if k == "mul":
        if not any(ca) and isinstance(ba, (int, np.integer)):
            return [int(ba) * y for y in cb], iv_bin(lambda a, b: a * b, ba, bb)
        if not any(cb) and isinstance(bb, (int, np.integer)):
            return [int(bb) * x for x in ca], iv_bin(lambda a, b: a * b, ba, bb)
        if not any(ca) and not any(cb):
            return [0] * n_vars, iv_bin(lambda a, b: a * b, ba, bb)
    raise Unsupported(f"non-affine subscript ({k}) in an indirect access tile")


def sub_values(expr, vars_e: np.ndarray, at):
    """Value of a subscript expression at every point (rows) and every element of the variable space
    (columns), for expressions ``_lin`` cannot split into a per-point and a per-element part
    (``floordiv`` / ``mod`` of the variables, products of variables and SSA values).  ``vars_e`` is
    ``[n_vars, elems]``; ``at(ssa name)`` gives that value per point."""
    k = expr[0]
    if k == "const":
        return np.int64(expr[1])
    if k == "var":
        return vars_e[expr[1]][None, :]
    if k == "ssa":
        return at(expr[1])[:, None]
    if k == "neg":
        return -sub_values(expr[1], vars_e, at)
    a, b = sub_values(expr[1], vars_e, at), sub_values(expr[2], vars_e, at)
    if k == "add":
        return a + b
    if k == "sub":
        return a - b
    if k == "mul":
        return a * b
    if k == "floordiv":
        return np.floor_divide(a, b)
    if k == "mod":
        return np.mod(a, b)
    raise ValueError(f"bad subscript node {k}")


@dataclass
class RowForm:
    """Row-addressing of one operand over the tiles of a statement."""
    indirect: bool
    dtype: str
    base: np.ndarray                 # [n_tiles] element offsets
    pos_stride: int
    idx_dtype: str = "i32"
    idx_off: Optional[np.ndarray] = None
    idx_stride: int = 0
    idx_mult: int = 0
    rows: int = 1
    cols: int = 1
    idx2_dtype: str = "i32"          # second index lookup of a two-subscript gather (joint_forms only)
    idx2_off: Optional[np.ndarray] = None
    idx2_stride: int = 0
    idx2_mult: int = 0

    def same_rows(self, o: "RowForm") -> bool:
        if self.idx2_off is not None or o.idx2_off is not None:
            return False
        return (self.indirect and o.indirect and self.dtype == o.dtype and self.pos_stride == o.pos_stride
                and self.idx_dtype == o.idx_dtype and self.idx_stride == o.idx_stride
                and self.idx_mult == o.idx_mult and np.array_equal(self.base, o.base)
                and np.array_equal(self.idx_off, o.idx_off))


def _rc_dims(shape, unit_stride=None) -> Tuple[Optional[int], List[int]]:
    """(row dim, column dims) of a tile seen as rows of contiguous columns.  ``unit_stride[d]`` is the
    element stride dim ``d`` walks with (None: unknown, e.g. it feeds an index lookup): trailing dims
    whose strides chain up (1, n_last, n_last * n_prev, ...) are one run of columns, so a block
    gather ``X[IDX[e], m, n]`` is rows of ``m * n`` contiguous elements."""
    big = [i for i, s in enumerate(shape) if s > 1]
    if not big:
        return None, []
    cols = [big[-1]]
    if unit_stride is not None:
        expect = shape[big[-1]] * (unit_stride[big[-1]] or 0)
        for d in reversed(big[:-1]):
            if len(big) - len(cols) <= 1 or unit_stride[big[-1]] != 1 or unit_stride[d] != expect:
                break
            cols.insert(0, d)
            expect *= shape[d]
    rest = [d for d in big if d not in cols]
    if len(rest) > 1:
        raise Unsupported(f"indirect tile of shape {tuple(shape)} (more than two non-unit dims)")
    if len(big) == 1:
        return None, cols
    return (rest[0] if rest else None), cols


def row_form(acc, axes, sel: np.ndarray) -> RowForm:
    """Row addressing of ``acc`` at the iteration points ``sel`` (flat indices into ``axes``)."""

    def per_tile(v) -> np.ndarray:
        return np.ascontiguousarray(iv_full(v, axes).reshape(-1)[sel]).astype(np.int64)

    if isinstance(acc, Access):
        if acc.coords is not None:
            raise Unsupported("coordinate-set access tile next to an indirect one")
        rd, cds = _rc_dims(acc.shape, list(acc.strides))
        if cds and acc.strides[cds[-1]] != 1:
            raise Unsupported("row operand whose columns are not unit-stride")
        return RowForm(False, acc.view.dtype, per_tile(acc.off), acc.strides[rd] if rd is not None else 0,
                       rows=acc.shape[rd] if rd is not None else 1,
                       cols=int(np.prod([acc.shape[d] for d in cds], dtype=np.int64)) if cds else 1)

    ia: IndirectAccess = acc
    if ia.order is not None and not ia.order.is_identity():
        raise Unsupported("indirect access tile with a permuted variables_space_order")
    box = ia.aset.box()
    if box is None:
        raise Unsupported("indirect access tile over a non-rectangular variable space")
    lo, hi = box
    ext = [h - l for l, h in zip(lo, hi)]
    nv = len(ext)
    # element stride each variable walks the parent view with through the direct subscripts; a variable
    # that feeds an index lookup has none
    walk: List[Optional[int]] = [0] * nv
    for sub, stride in zip(ia.subs, ia.view.strides):
        if sub["kind"] == "direct":
            c, _ = _lin(sub["expr"], nv, ia.ssa)
            for i, ci in enumerate(c):
                if walk[i] is not None:
                    walk[i] += ci * stride
        else:
            for e in sub["exprs"]:
                c, _ = _lin(e, nv, ia.ssa)
                for i, ci in enumerate(c):
                    if ci:
                        walk[i] = None
    rd, cds = _rc_dims(ext, walk)
    cd = cds[-1] if cds else None
    base = ia.view.base
    pos_stride, col_stride = 0, 0
    form = RowForm(True, ia.view.dtype, None, 0, rows=ext[rd] if rd is not None else 1,
                   cols=int(np.prod([ext[d] for d in cds], dtype=np.int64)) if cds else 1)
    n_ind = 0
    for sub, stride in zip(ia.subs, ia.view.strides):
        if sub["kind"] == "direct":
            c, b = _lin(sub["expr"], nv, ia.ssa)
            b = iv_bin(lambda x, y: x + y, b, sum(ci * l for ci, l in zip(c, lo)))
            base = iv_bin(lambda x, y: x + y, base, iv_bin(lambda x, y: x * y, b, stride))
            if rd is not None:
                pos_stride += c[rd] * stride
            if cd is not None:
                col_stride += c[cd] * stride
            if any(ci for i, ci in enumerate(c) if i != rd and i not in cds and ext[i] > 1):
                raise Unsupported("indirect tile subscript over an unexpected variable")
        else:
            n_ind += 1
            if n_ind > 1:
                raise Unsupported("indirect access tile with more than one indirect dimension")
            iv = ia.index_views[sub["view"]]
            ioff, istride = iv.base, 0
            for e, s in zip(sub["exprs"], iv.strides):
                c, b = _lin(e, nv, ia.ssa)
                b = iv_bin(lambda x, y: x + y, b, sum(ci * l for ci, l in zip(c, lo)))
                ioff = iv_bin(lambda x, y: x + y, ioff, iv_bin(lambda x, y: x * y, b, s))
                if any(c[d] for d in cds):
                    raise Unsupported("index lookup that varies along the tile's columns")
                if rd is not None:
                    istride += c[rd] * s
            form.idx_dtype, form.idx_off, form.idx_stride, form.idx_mult = iv.dtype, per_tile(ioff), istride, stride
    if n_ind == 0:
        raise Unsupported("indirect access tile without an indirect subscript")
    if cd is not None and col_stride != 1:
        raise Unsupported("indirect tile whose columns are not unit-stride")
    form.base, form.pos_stride = per_tile(base), pos_stride
    return form


def _walks(acc):
    """An operand as (dims, base, direct walk, lookups): ``dims`` the extent of each tile dimension,
    ``base`` the element offset of the tile's first element (an integer value over the iteration
    axes), ``direct walk[d]`` the elements one step along dim ``d`` moves through the direct
    subscripts, and per index lookup ``(index dtype, index offset of the first element, index
    elements one step along each dim moves, data elements per unit of index value)``."""
    if isinstance(acc, Access):
        if acc.coords is not None:
            raise Unsupported("coordinate-set access tile next to an indirect one")
        return list(acc.shape), acc.off, [int(s) for s in acc.strides], []
    ia: IndirectAccess = acc
    if ia.order is not None and not ia.order.is_identity():
        raise Unsupported("indirect access tile with a permuted variables_space_order")
    box = ia.aset.box()
    if box is None:
        raise Unsupported("indirect access tile over a non-rectangular variable space")
    lo, hi = box
    nv = len(lo)
    add = lambda x, y: iv_bin(lambda a, b: a + b, x, y)
    mul = lambda x, y: iv_bin(lambda a, b: a * b, x, y)
    base, walk, lookups = ia.view.base, [0] * nv, []
    for sub, stride in zip(ia.subs, ia.view.strides):
        if sub["kind"] == "direct":
            c, b = _lin(sub["expr"], nv, ia.ssa)
            base = add(base, mul(add(b, sum(ci * l for ci, l in zip(c, lo))), stride))
            walk = [w + ci * stride for w, ci in zip(walk, c)]
        else:
            iv = ia.index_views[sub["view"]]
            ioff, iwalk = iv.base, [0] * nv
            for e, s_ in zip(sub["exprs"], iv.strides):
                c, b = _lin(e, nv, ia.ssa)
                ioff = add(ioff, mul(add(b, sum(ci * l for ci, l in zip(c, lo))), s_))
                iwalk = [w + ci * s_ for w, ci in zip(iwalk, c)]
            lookups.append((iv.dtype, ioff, iwalk, int(stride)))
    return [h - l for l, h in zip(lo, hi)], base, walk, lookups


def joint_forms(accs, axes, sel: np.ndarray) -> Tuple[List[RowForm], int]:
    """Row addressing of all operands of a statement under ONE split of the tile's dimensions:
    trailing dims every operand walks contiguously are the columns, the dim before them the rows,
    and the dims before that unroll into tiles of their own (``n_outer`` per iteration point) — so
    ``out[p, t, :] = X[P[p], T[t], :]`` is ``len(P)`` tiles of ``len(T)`` rows with one lookup fixed per
    tile and one walking the rows.  An operand takes up to two index lookups."""
    ops = [_walks(a) for a in accs]
    bigs = [[i for i, n in enumerate(d) if n > 1] for d, _, _, _ in ops]
    dims = [ops[0][0][i] for i in bigs[0]]
    if not dims or any([d[i] for i in b] != dims for (d, _, _, _), b in zip(ops, bigs)):
        raise Unsupported("row statement operands with different tile shapes")
    n = len(dims)

    def contiguous(j, run):        # dim j (position among the non-unit dims) continues a run of `run` elements
        return all(w[b[j]] == run and not any(lw[b[j]] for _, _, lw, _ in lk)
                   for (_, _, w, lk), b in zip(ops, bigs))

    if not contiguous(n - 1, 1):
        raise Unsupported("indirect tile whose columns are not unit-stride")
    k, run = 1, dims[-1]
    while n - k > 1 and contiguous(n - k - 1, run):
        k, run = k + 1, run * dims[n - k - 1]
    rd = n - k - 1 if n - k >= 1 else None
    outer = list(range(rd)) if rd is not None else []
    n_outer = int(np.prod([dims[j] for j in outer], dtype=np.int64)) if outer else 1
    coords = (np.indices([dims[j] for j in outer]).reshape(len(outer), -1).astype(np.int64)
              if outer else np.zeros((0, 1), np.int64))

    def per_tile(v, steps) -> np.ndarray:
        t = np.ascontiguousarray(iv_full(v, axes).reshape(-1)[sel]).astype(np.int64)
        return (t[:, None] + (np.asarray(steps, np.int64) @ coords)[None, :]).reshape(-1)

    forms = []
    for (d, base, walk, lookups), b, acc in zip(ops, bigs, accs):
        if len(lookups) > 2:
            raise Unsupported("indirect access tile with more than two indirect dimensions")
        f = RowForm(bool(lookups), acc.view.dtype, per_tile(base, [walk[b[j]] for j in outer]),
                    walk[b[rd]] if rd is not None else 0, rows=dims[rd] if rd is not None else 1, cols=run)
        for i, (dt, ioff, iwalk, mult) in enumerate(lookups):
            off, st = per_tile(ioff, [iwalk[b[j]] for j in outer]), iwalk[b[rd]] if rd is not None else 0
            if i == 0:
                f.idx_dtype, f.idx_off, f.idx_stride, f.idx_mult = dt, off, st, mult
            else:
                f.idx2_dtype, f.idx2_off, f.idx2_stride, f.idx2_mult = dt, off, st, mult
        forms.append(f)
    return forms, n_outer


class RowsStatement(Statement):
    """rows_program (direct destination) or ordered scatter_rows (indirect destination)."""

    def __init__(self, dev: R.Device, store: Store, arena: ArenaMap, stmt_id: int, row_shard=None):
        self.owned_range = None
        self.ordered = isinstance(store.target, IndirectAccess)
        self.kind = "scatter_rows" if self.ordered else "rows_program"
        pb = ProgramBuilder(leaf_kinds=("load", "iload"))
        self.program = pb.build(store.value, store.target.shape)
        if len(pb.inputs) > R.ROWS_MAX_IN:
            raise Unsupported(f"row statement with more than {R.ROWS_MAX_IN} input tiles")
        sel, cores = _points(store)
        n_tiles = len(sel)
        accs = [n.attrs["access"] for n in pb.inputs] + [store.target]
        try:
            forms = [row_form(a, store.axes, sel) for a in accs]
            if any((f.rows, f.cols) != (forms[-1].rows, forms[-1].cols) for f in forms[:-1]):
                raise Unsupported("row statement operands with different tile shapes")
        except Unsupported:
            # tiles of more than [rows, columns], or two index subscripts: one split for all operands
            forms, n_outer = joint_forms(accs, store.axes, sel)
            sel, cores = np.repeat(sel, n_outer), np.repeat(cores, n_outer)
            n_tiles *= n_outer
        out = forms[-1]
        if out.idx2_off is not None:
            raise Unsupported("indirect store through two index subscripts")
        if not self.ordered and out.cols >= 512 and n_tiles * out.rows < 65536:
            # few, very long rows (a block gather of whole expert matrices or KV pages): the kernel gives a
            # warp 32 rows to move one after the other, so each row is cut into short column segments that
            # become tiles of their own — same index look-ups, bases moved along by the segment
            seg = next((c for c in range(256, 7, -8) if out.cols % c == 0), None)
            if seg is not None:
                nseg = out.cols // seg
                shift = np.arange(nseg, dtype=np.int64) * seg
                for f in forms:
                    f.base = (f.base[:, None] + shift[None, :]).reshape(-1)
                    if f.idx_off is not None:
                        f.idx_off = np.repeat(f.idx_off, nseg)
                    if f.idx2_off is not None:
                        f.idx2_off = np.repeat(f.idx2_off, nseg)
                    f.cols = seg
                sel, cores = np.repeat(sel, nseg), np.repeat(cores, nseg)
                n_tiles *= nseg
        self.args = a = R.RowsArgs()
        a.n_tiles, a.tile_rows, a.cols, a.n_in = n_tiles, out.rows, out.cols, len(forms) - 1
        a.program = self.program
        self.device_arrays = []
        self.fps: List[Footprint] = []
        vec = out.cols % 4 == 0
        dst_alloc = None
        for k, (acc, f) in enumerate(zip(accs, forms)):
            is_out = k == len(forms) - 1
            op = a.out if is_out else a.inp[k]
            view = acc.view
            bpe = bytes_per_elem(view.dtype)
            first = int(f.base.min()) if n_tiles else int(np.asarray(view.base).reshape(-1)[0])
            alloc = arena.find(int(iv_full(view.base, store.axes).reshape(-1)[0]) * bpe)
            if alloc is None:
                raise ValueError(f"{'Scatter to' if is_out else 'Read from'} unmapped address "
                                 f"0x{first * bpe:x}")
            op.indirect, op.dtype = int(f.indirect), R.DTYPE_CODE[f.dtype]
            op.pos_stride = f.pos_stride
            op.lo, op.hi = alloc.byte_lo // bpe, alloc.byte_hi // bpe
            p = dev.upload(f.base)
            self.device_arrays.append(p)
            op.dev_base = p
            vec = vec and f.pos_stride % 4 == 0 and bool((f.base % 4 == 0).all())
            if f.indirect:
                ibpe = bytes_per_elem(f.idx_dtype)
                if n_tiles:
                    ia = arena.check_range(int(f.idx_off.min()),
                                           int(f.idx_off.max()) + (f.rows - 1) * f.idx_stride + 1,
                                           f.idx_dtype, "Read from")
                    self.fps.append(Footprint(np.array([ia.byte_lo]), np.array([ia.byte_hi]),
                                              np.array([-1]), np.array([-1]), False, stmt_id))
                op.idx_dtype, op.idx_stride, op.idx_mult = R.DTYPE_CODE[f.idx_dtype], f.idx_stride, f.idx_mult
                p = dev.upload(f.idx_off)
                self.device_arrays.append(p)
                op.dev_idx_off = p
                vec = vec and f.idx_mult % 4 == 0
                if f.idx2_off is not None:
                    if n_tiles:
                        ia = arena.check_range(int(f.idx2_off.min()),
                                               int(f.idx2_off.max()) + (f.rows - 1) * f.idx2_stride + 1,
                                               f.idx2_dtype, "Read from")
                        self.fps.append(Footprint(np.array([ia.byte_lo]), np.array([ia.byte_hi]),
                                                  np.array([-1]), np.array([-1]), False, stmt_id))
                    op.indirect = 2
                    op.idx2_dtype, op.idx2_stride, op.idx2_mult = R.DTYPE_CODE[f.idx2_dtype], f.idx2_stride, f.idx2_mult
                    p = dev.upload(f.idx2_off)
                    self.device_arrays.append(p)
                    op.dev_idx2_off = p
                    vec = vec and f.idx2_mult % 4 == 0
            else:
                if n_tiles:
                    arena.check_range(int(f.base.min()), int(f.base.max()) + (f.rows - 1) * f.pos_stride + f.cols,
                                      f.dtype, "Scatter to" if is_out else "Read from")
            if is_out:
                dst_alloc = alloc
            elif self.ordered and f.same_rows(out):
                op.alias_dst = 1
            if not (not is_out and self.ordered and f.same_rows(out)):
                whole = f.indirect or not n_tiles
                if whole:
                    self.fps.append(Footprint(np.array([alloc.byte_lo]), np.array([alloc.byte_hi]),
                                              np.array([-1]), np.array([-1]), is_out, stmt_id))
                else:
                    rs = (f.base[:, None] + np.arange(f.rows, dtype=np.int64)[None, :] * f.pos_stride).reshape(-1) * bpe
                    self.fps.append(Footprint(rs, rs + f.cols * bpe, np.repeat(sel, f.rows),
                                              np.repeat(cores, f.rows), is_out, stmt_id))
        a.vector_ok = int(vec)
        if self.ordered:
            if out.pos_stride != 0 or out.idx_mult < out.cols or (n_tiles and (out.base != out.base[0]).any()):
                raise Unsupported("indirect store whose destination rows are not whole rows of one table")
            for k, f in enumerate(forms[:-1]):
                acc = accs[k]
                al = arena.find(int(iv_full(acc.view.base, store.axes).reshape(-1)[0]) * bytes_per_elem(acc.view.dtype))
                if al is dst_alloc and not a.inp[k].alias_dst:
                    raise Unsupported("indirect store whose value reads other rows of its destination")
            a.dst_row0 = int(out.base[0]) if n_tiles else 0
            bpe = bytes_per_elem(out.dtype)
            a.dst_rows = max(0, (dst_alloc.byte_hi // bpe - a.dst_row0 - out.cols) // out.idx_mult + 1)
            if row_shard is not None:
                # destination rows are split over the ranks; a rank applies, in the global
                # (tile, position) order, only the updates that land in its rows
                rank, world = row_shard
                total = int(a.dst_rows)
                lo, hi = rank * total // world, (rank + 1) * total // world
                a.dst_row0 += lo * out.idx_mult
                a.dst_rows = hi - lo
                self.owned_range = (int(a.dst_row0) * bpe, int(a.dst_row0 + (hi - lo) * out.idx_mult) * bpe)
            nbytes = 1 << 20
            if getattr(dev, "lib", None) is not None:
                nbytes = int(dev.lib.ktb_scatter_scratch_bytes(n_tiles * out.rows, int(a.dst_rows)))
            self.scratch = dev.alloc(nbytes)
            self.device_arrays.append(self.scratch)
            a.dev_rowid_scratch = self.scratch
            self.launches = 2
        self.extra_written = [dst_alloc.name] if (self.ordered and dst_alloc is not None) else []
        self.entries = n_tiles * out.rows
        self._bytes = sum(self.entries * f.cols * bytes_per_elem(f.dtype) + (self.entries * bytes_per_elem(f.idx_dtype) if f.indirect and f.idx_stride else 0)
                          for f in forms)

    def launch(self, dev, arena_ptr):
        if self.ordered and self.args.dst_rows <= 0:
            return                     # this rank owns no destination rows
        self.args.arena = arena_ptr
        fn = dev.lib.ktb_launch_scatter_rows if self.ordered else dev.lib.ktb_launch_rows_program
        dev.check(fn(dev.h, C.byref(self.args)))

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


def lower_indirect_store(dev, store, arena, stmt_id, row_shard=None):
    return RowsStatement(dev, store, arena, stmt_id, row_shard)


def has_indirect_load(n: Node, seen=None) -> bool:
    seen = seen if seen is not None else set()
    if id(n) in seen:
        return False
    seen.add(id(n))
    return n.kind == "iload" or any(has_indirect_load(a, seen) for a in n.args)

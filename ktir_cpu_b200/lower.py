"""Lowering: traced stores -> device launches (a :class:`Plan`).

Each ``ktdp.store`` of the trace is matched against the kernel idioms this
backend has hand-written CUDA for; one launch then covers every grid core and
every iteration of the enclosing parallel loops.  The reference executes the
same work op by op and core by core (ktir_cpu/grid.py:595-613); running the
cores concurrently is only equivalent when no core (or loop iteration) touches
memory another one writes, which :func:`check_hazards` verifies on the exact
byte runs before a plan is accepted.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem
from .trace import Access, CoreOrderHazard, IndirectAccess, Node, Store, Unsupported, iv_full

F_DT = ("f16", "f32")


@dataclass
class Allocation:
    name: str
    byte_lo: int
    byte_hi: int
    dtype: str


class ArenaMap:
    """Host mirror of the allocation list (ktir_cpu/memory.py:167-214, 311-352)."""

    def __init__(self, allocs: List[Allocation]):
        self.allocs = sorted(allocs, key=lambda a: a.byte_lo)

    def find(self, byte_addr: int) -> Optional[Allocation]:
        for a in self.allocs:
            if a.byte_lo <= byte_addr < a.byte_hi:
                return a
        return None

    def check_range(self, lo_elem: int, hi_elem: int, dtype: str, what: str) -> Allocation:
        bpe = bytes_per_elem(dtype)
        a = self.find(lo_elem * bpe)
        if a is None:
            raise ValueError(f"{what} unmapped address 0x{lo_elem * bpe:x}")
        if hi_elem * bpe > a.byte_hi:
            raise Unsupported(f"{what.strip()} runs past the end of allocation '{a.name}' "
                              "(zero-padded / dropped accesses have no device path yet)")
        return a


@dataclass
class Footprint:
    """Byte runs touched by one statement: starts/ends per run plus the point each run belongs to."""
    starts: np.ndarray
    ends: np.ndarray
    points: np.ndarray
    cores: np.ndarray
    write: bool
    stmt: int


class Statement:
    kind = "?"
    device_arrays: List[int]
    launches = 1

    def launch(self, dev: R.Device, arena_ptr: int):
        raise NotImplementedError

    def footprints(self) -> List[Footprint]:
        return []

    def bytes_moved(self) -> int:
        return 0

    def split(self, piece_bytes: int):
        """Independent parts of this statement for pipelined execution (``pipeline.Chunk`` list:
        a launch over part of the work plus the arena regions it reads and writes), or None."""
        return None


def _copy_args(args):
    return type(args).from_buffer_copy(args)


def _split_item_table(stmt, table: np.ndarray, geoms, bpes, launch_fn, piece_bytes: int):
    """Split a statement whose work is rows of an item table ``[n_items][operands]`` (the last
    operand is the output) into contiguous item ranges."""
    from .pipeline import Chunk, chunk_count, tile_regions
    n_items, n_op = table.shape
    total = sum(n_items * g[0] * g[2] * b for g, b in zip(geoms, bpes))
    n = chunk_count(total, n_items, piece_bytes)
    bounds = np.linspace(0, n_items, n + 1).astype(np.int64)
    chunks = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if a == b:
            continue
        regs = []
        for k in range(n_op):
            rows, stride, cols = geoms[k]
            r = tile_regions(table[a:b, k], rows, stride, cols, bpes[k])
            if r is None:
                return None
            regs.append(r)
        chunks.append(Chunk(launch_fn(int(a), int(b)), [x for r in regs[:-1] for x in r], list(regs[-1])))
    return chunks


def _order_item_table(stmt, sel: np.ndarray, n_lead: int, rounds: Dict[int, int], dev):
    """Reorder a statement's item table so that items of later rounds come later and remember the
    round boundaries; the launches then go out round by round."""
    per_item = np.array([rounds.get(int(p), 0) for p in np.repeat(sel, n_lead)], np.int64)
    order = np.argsort(per_item, kind="stable")
    stmt.table = np.ascontiguousarray(stmt.table[order])
    dev.free(stmt.dev_table)
    stmt.dev_table = dev.upload(stmt.table)
    stmt.args.dev_item_offsets = stmt.dev_table
    stmt.device_arrays = [stmt.dev_table]
    srt = per_item[order]
    cuts = np.flatnonzero(np.diff(srt)) + 1
    stmt.rounds = list(zip(np.concatenate([[0], cuts]).tolist(), np.concatenate([cuts, [len(srt)]]).tolist()))
    stmt.launches = len(stmt.rounds)


def _points(store: Store):
    """Flat indices (and core ids) of the active iteration points of a store."""
    n = int(np.prod(store.axes))
    idx = np.arange(n, dtype=np.int64)
    if store.active is not None:
        idx = idx[store.active.reshape(-1)]
    inner = n // store.axes[0] if store.axes[0] else 1
    return idx, idx // max(inner, 1)


def _access_offsets(acc: Access, store: Store, sel: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(iv_full(acc.off, store.axes).reshape(-1)[sel])


@dataclass
class TileGeom:
    """A strided-box tile as ``lead`` row origins (element offsets) of rows x cols each."""
    lead: np.ndarray          # [n_lead] element offsets relative to the tile origin
    rows: int
    cols: int
    row_stride: int


def tile_geom(acc: Access, expand_rows: bool) -> TileGeom:
    if acc.coords is not None:
        raise Unsupported("coordinate-set (non-rectangular) access tile in a fused statement")
    shape, strides = list(acc.shape), list(acc.strides)
    if not shape:
        shape, strides = [1], [1]
    if strides[-1] != 1 and shape[-1] != 1:
        raise Unsupported("access tile whose innermost dimension is not unit-stride")
    cols = shape[-1]
    if len(shape) == 1:
        return TileGeom(np.zeros(1, np.int64), 1, cols, cols)
    if expand_rows or len(shape) > 2:
        grids = np.indices(shape[:-1], dtype=np.int64).reshape(len(shape) - 1, -1)
        lead = (np.asarray(strides[:-1], np.int64)[:, None] * grids).sum(0)
        return TileGeom(lead, 1, cols, cols)
    return TileGeom(np.zeros(1, np.int64), shape[0], cols, strides[0])


# ---------------------------------------------------------------------------
# Elementwise programs
# ---------------------------------------------------------------------------
_VM_BIN = {"arith.addf": "ADD", "arith.subf": "SUB", "arith.mulf": "MUL", "arith.divf": "DIV",
           "arith.maximumf": "MAX", "arith.maxnumf": "MAXNUM", "arith.minimumf": "MIN",
           "arith.minnumf": "MINNUM"}
_VM_UN = {"arith.negf": "NEG", "math.absf": "ABS", "math.exp": "EXP", "math.log": "LOG",
          "math.log2": "LOG2", "math.sqrt": "SQRT", "math.rsqrt": "RSQRT", "math.tanh": "TANH",
          "math.sin": "SIN", "math.cos": "COS"}


def strip_views(n: Node) -> Node:
    """Skip reshapes (row-major element order is unchanged) and full-shape broadcasts of constants."""
    while n.kind == "reshape":
        n = n.args[0]
    return n


class ProgramBuilder:
    """Compiles an elementwise DAG over same-shaped tiles into a register program."""

    def __init__(self, leaf_kinds=("load",)):
        self.inputs: List[Node] = []
        self.ops: List[Tuple[int, int, int, int, int, float]] = []
        self.reg_of: Dict[int, int] = {}
        self.free: List[int] = []
        self.next_reg = 0
        self.leaf_kinds = leaf_kinds

    def collect_inputs(self, n: Node, seen=None):
        seen = seen if seen is not None else set()
        n = strip_views(n)
        if id(n) in seen:
            return
        seen.add(id(n))
        if n.kind in self.leaf_kinds:
            if n.dtype not in F_DT:
                raise Unsupported(f"{n.dtype} tile in an elementwise statement")
            if not any(n is x for x in self.inputs):
                self.inputs.append(n)
            return
        for a in n.args:
            self.collect_inputs(a, seen)

    def alloc(self) -> int:
        if self.free:
            return self.free.pop()
        r = self.next_reg
        self.next_reg += 1
        if r >= R.VM_REGS:
            raise Unsupported("elementwise expression needs more than 8 live registers")
        return r

    def emit(self, code: str, dst: int, a=0, b=0, c=0, imm=0.0, r16=False):
        if len(self.ops) >= R.VM_MAX_OPS:
            raise Unsupported("elementwise expression longer than 12 ops")
        self.ops.append((R.VM[code] | (R.VM_ROUND16 if r16 else 0), dst, a, b, c, float(imm)))

    def build(self, root: Node, full_shape: Tuple[int, ...]) -> R.VmProgram:
        self.collect_inputs(root)
        if not self.inputs:
            raise Unsupported("store of a tile that reads no memory")
        if len(self.inputs) > R.VM_MAX_IN:
            raise Unsupported(f"elementwise statement with more than {R.VM_MAX_IN} input tiles")
        self.full_elems = int(np.prod(full_shape)) if full_shape else 1
        for i, n in enumerate(self.inputs):
            self.reg_of[id(n)] = i
        self.next_reg = len(self.inputs)
        res = self.visit(root)
        p = R.VmProgram()
        p.n_in, p.n_ops, p.result_reg = len(self.inputs), len(self.ops), res
        for i, (code, dst, a, b, c, imm) in enumerate(self.ops):
            p.ops[i] = R.VmOp(code, dst, a, b, c, imm)
        return p

    def visit(self, n: Node) -> int:
        n = strip_views(n)
        if id(n) in self.reg_of:
            return self.reg_of[id(n)]
        r16 = n.dtype == "f16"
        if n.kind == "const":
            if n.attrs.get("list") is not None:
                raise Unsupported("dense list constant in an elementwise statement")
            v = n.attrs["value"]
            v = float(np.float16(v)) if n.dtype == "f16" else float(np.float32(v))
            r = self.alloc()
            self.emit("CONST", r, imm=v)
        elif n.kind == "bcast" and strip_views(n.args[0]).kind == "const":
            return self.visit(n.args[0])
        elif n.kind == "cast":
            src = self.visit(n.args[0])
            if n.args[0].dtype not in F_DT or n.dtype not in F_DT:
                raise Unsupported(f"cast {n.args[0].dtype}->{n.dtype} in an elementwise statement")
            if n.dtype == "f32":
                return src                      # f16 values are exact in f32 registers
            r = self.alloc()
            self.emit("MOV", r, src, r16=True)
        elif n.kind == "ew":
            op = n.attrs["op"]
            for a in n.args:
                sa = strip_views(a)
                if sa.kind not in ("const",) and not (sa.kind == "bcast" and strip_views(sa.args[0]).kind == "const"):
                    if int(np.prod(sa.shape)) != self.full_elems:
                        raise Unsupported("broadcasting between tiles of different shape in an "
                                          "elementwise statement")
            if n.dtype not in F_DT:
                raise Unsupported(f"{op} producing {n.dtype} in an elementwise statement")
            regs = [self.visit(a) for a in n.args]
            r = self.alloc()
            if op in _VM_BIN:
                self.emit(_VM_BIN[op], r, regs[0], regs[1], r16=r16)
            elif op in _VM_UN:
                self.emit(_VM_UN[op], r, regs[0], r16=r16)
            elif op == "math.fma":
                self.emit("FMA", r, regs[0], regs[1], regs[2], r16=r16)
            else:
                raise Unsupported(f"{op} in an elementwise statement")
        else:
            raise Unsupported(f"{n.kind} node in an elementwise statement")
        self.reg_of[id(n)] = r
        return r


class EwStatement(Statement):
    kind = "ew_stream"

    def __init__(self, dev: R.Device, store: Store, arena: ArenaMap, stmt_id: int):
        tgt: Access = store.target
        pb = ProgramBuilder()
        self.program = pb.build(store.value, tgt.shape)
        operands: List[Access] = [n.attrs["access"] for n in pb.inputs] + [tgt]
        n_elems = int(np.prod(tgt.shape)) if tgt.shape else 1
        for acc in operands[:-1]:
            if (int(np.prod(acc.shape)) if acc.shape else 1) != n_elems:
                raise Unsupported("operand tile shape differs from the stored tile")
        simple = all(len(a.shape) <= 2 for a in operands) and len({tuple(a.shape) for a in operands}) == 1
        geoms = [tile_geom(a, not simple) for a in operands]
        g_out = geoms[-1]
        if any((g.cols, g.rows, len(g.lead)) != (g_out.cols, g_out.rows, len(g_out.lead)) for g in geoms):
            raise Unsupported("operand tiles with different row structure in an elementwise statement")
        sel, cores = _points(store)
        self.n_points = len(sel)
        n_lead = len(g_out.lead)
        table = np.empty((len(sel) * n_lead, len(operands)), np.int64)
        self.fps: List[Footprint] = []
        for k, (acc, g) in enumerate(zip(operands, geoms)):
            offs = _access_offsets(acc, store, sel)
            full = (offs[:, None] + g.lead[None, :]).reshape(-1)
            table[:, k] = full
            if len(full):
                span = (g.rows - 1) * g.row_stride + g.cols
                arena.check_range(int(full.min()), int(full.max()) + span, acc.view.dtype,
                                  "Read from" if k < len(operands) - 1 else "Scatter to")
            bpe = bytes_per_elem(acc.view.dtype)
            rstart = (full[:, None] + np.arange(g.rows, dtype=np.int64)[None, :] * g.row_stride).reshape(-1) * bpe
            pts = np.repeat(sel, n_lead * g.rows)
            self.fps.append(Footprint(rstart, rstart + g.cols * bpe, pts, np.repeat(cores, n_lead * g.rows),
                                      k == len(operands) - 1, stmt_id))
        self.table = table
        self._sel, self._n_lead, self._dev, self.rounds = sel, n_lead, dev, None
        self.args = R.EwArgs()
        a = self.args
        a.n_items = table.shape[0]
        a.rows, a.cols = g_out.rows, g_out.cols
        vec = (g_out.cols % 8 == 0) and bool((table % 8 == 0).all())
        for k, (acc, g) in enumerate(zip(operands, geoms)):
            a.row_stride[k] = g.row_stride
            a.dtype[k] = R.DTYPE_CODE[acc.view.dtype]
            vec = vec and (g.row_stride % 8 == 0 or g.rows == 1)
        a.vector_ok = 1 if vec else 0
        a.program = self.program
        self.dev_table = dev.upload(table)
        a.dev_item_offsets = self.dev_table
        self.device_arrays = [self.dev_table]
        self.elems = int(table.shape[0]) * g_out.rows * g_out.cols
        self._bytes = sum(self.elems * bytes_per_elem(acc.view.dtype) for acc in operands)

    def launch(self, dev, arena_ptr):
        self.args.arena = arena_ptr
        if self.rounds:                       # several points store to the same bytes: in sequential order
            n_op = self.table.shape[1]
            for lo, hi in self.rounds:
                sub = _copy_args(self.args)
                sub.dev_item_offsets = self.dev_table + lo * n_op * 8
                sub.n_items = hi - lo
                dev.check(dev.lib.ktb_launch_ew_stream(dev.h, C.byref(sub)))
            return
        dev.check(dev.lib.ktb_launch_ew_stream(dev.h, C.byref(self.args)))

    def order_points(self, rounds: Dict[int, int]):
        _order_item_table(self, self._sel, self._n_lead, rounds, self._dev)

    def split(self, piece_bytes: int):
        if self.rounds:
            return None
        a, n_op = self.args, self.table.shape[1]
        geoms = [(a.rows, int(a.row_stride[k]), a.cols) for k in range(n_op)]
        bpes = [2 if a.dtype[k] == R.KTB_F16 else 4 for k in range(n_op)]

        def part(lo, hi):
            sub = _copy_args(a)
            sub.dev_item_offsets = self.dev_table + lo * n_op * 8
            sub.n_items = hi - lo
            return ("ktb_launch_ew_stream", sub)
        return _split_item_table(self, self.table, geoms, bpes, part, piece_bytes)

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


# ---------------------------------------------------------------------------
# Row softmax idiom
# ---------------------------------------------------------------------------
def _skip(n: Node) -> Node:
    """Strip reshapes and single-element extracts."""
    while True:
        if n.kind == "reshape":
            n = n.args[0]
        elif n.kind == "extract" and int(np.prod(n.args[0].shape) if n.args[0].shape else 1) == 1:
            n = n.args[0]
        else:
            return n


def _row_broadcast(n: Node, tile_shape) -> Optional[Node]:
    """If ``n`` spreads one value per row along the last dim of ``tile_shape``, return that value."""
    n = strip_views(n)
    if n.kind != "bcast" or tuple(n.shape) != tuple(tile_shape):
        return None
    src = _skip(n.args[0])
    rows = int(np.prod(tile_shape[:-1])) if len(tile_shape) > 1 else 1
    if (int(np.prod(src.shape)) if src.shape else 1) != rows:
        return None
    dims = list(n.attrs.get("dims", []))
    nd = len(tile_shape)
    if dims == [nd - 1] or (rows == 1 and sorted(dims) == list(range(nd))):
        return src
    return None


def _row_reduce(n: Node, opnames) -> Optional[Tuple[Node, str, Optional[float]]]:
    """Match ``combine(reduce(op, src, last dim), const init)`` -> (src, op, init)."""
    n = _skip(n)
    init = None
    if n.kind == "ew" and n.attrs["op"] in opnames and len(n.args) == 2:
        red, c = _skip(n.args[0]), strip_views(n.args[1])
        while c.kind == "bcast":
            c = strip_views(c.args[0])
        if c.kind != "const" or c.attrs.get("list") is not None:
            return None
        init = float(c.attrs["value"])
        n = red
    if n.kind != "reduce" or n.attrs["op"] not in opnames:
        return None
    src = n.args[0]
    dims = n.attrs["dims"]
    if dims is None:
        if len([s for s in src.shape if s != 1]) > 1:
            return None
    elif tuple(dims) != (len(src.shape) - 1,):
        return None
    return src, n.attrs["op"], init


def match_softmax(value: Node):
    """Recognise store(truncf?(exp(x - rowmax(x)) / rowsum(exp(x - rowmax(x)))))."""
    root = strip_views(value)
    out_cast = False
    if root.kind == "cast" and root.dtype == "f16" and root.args[0].dtype == "f32":
        out_cast = True
        root = strip_views(root.args[0])
    if root.kind != "ew" or root.attrs["op"] != "arith.divf":
        return None
    num, den = strip_views(root.args[0]), root.args[1]
    shape = tuple(num.shape)
    if not shape:
        return None
    dsrc = _row_broadcast(den, shape)
    if dsrc is None:
        return None
    dr = _row_reduce(dsrc, ("arith.addf",))
    if dr is None or strip_views(dr[0]) is not num:
        return None
    if num.kind != "ew" or num.attrs["op"] != "math.exp":
        return None
    sub = strip_views(num.args[0])
    if sub.kind != "ew" or sub.attrs["op"] != "arith.subf":
        return None
    x = strip_views(sub.args[0])
    msrc = _row_broadcast(sub.args[1], shape)
    if msrc is None:
        return None
    mr = _row_reduce(msrc, ("arith.maximumf", "arith.maxnumf"))
    if mr is None or strip_views(mr[0]) is not x:
        return None
    xl = x
    if xl.kind == "cast" and xl.dtype == "f32":
        xl = strip_views(xl.args[0])
    if xl.kind != "load" or xl.dtype not in F_DT:
        return None
    arith = num.dtype
    if arith == "f16" and (x.dtype != "f16" or out_cast):
        return None
    return dict(load=xl, arith=arith, maxop=mr[1],
                max_init=mr[2] if mr[2] is not None else float("-inf"),
                sum_init=dr[2] if dr[2] is not None else 0.0)


class SoftmaxStatement(Statement):
    kind = "row_softmax"

    def __init__(self, dev: R.Device, store: Store, m: dict, arena: ArenaMap, stmt_id: int):
        tgt: Access = store.target
        src: Access = m["load"].attrs["access"]
        gi, go = tile_geom(src, False), tile_geom(tgt, False)
        if len(gi.lead) != 1 or len(go.lead) != 1:
            gi, go = tile_geom(src, True), tile_geom(tgt, True)
        if (gi.rows, gi.cols, len(gi.lead)) != (go.rows, go.cols, len(go.lead)):
            raise Unsupported("softmax input and output tiles differ in shape")
        cols = gi.cols
        if cols < 8 or cols > 16384 or cols & (cols - 1):
            raise Unsupported(f"fused softmax over rows of {cols} elements (power of two in [8, 16384] only)")
        sel, cores = _points(store)
        n_lead = len(gi.lead)
        table = np.empty((len(sel) * n_lead, 2), np.int64)
        self.fps = []
        for k, (acc, g) in enumerate(((src, gi), (tgt, go))):
            full = (_access_offsets(acc, store, sel)[:, None] + g.lead[None, :]).reshape(-1)
            table[:, k] = full
            if len(full):
                arena.check_range(int(full.min()), int(full.max()) + (g.rows - 1) * g.row_stride + g.cols,
                                  acc.view.dtype, "Read from" if k == 0 else "Scatter to")
            bpe = bytes_per_elem(acc.view.dtype)
            rstart = (full[:, None] + np.arange(g.rows, dtype=np.int64)[None, :] * g.row_stride).reshape(-1) * bpe
            self.fps.append(Footprint(rstart, rstart + g.cols * bpe, np.repeat(sel, n_lead * g.rows),
                                      np.repeat(cores, n_lead * g.rows), k == 1, stmt_id))
        if (table % 8).any() or (gi.rows > 1 and (gi.row_stride % 8 or go.row_stride % 8)):
            raise Unsupported("fused softmax needs 16-byte aligned rows")
        self.args = a = R.SoftmaxArgs()
        a.n_items = table.shape[0]
        a.rows_per_item, a.cols = gi.rows, cols
        a.in_row_stride, a.out_row_stride = max(gi.row_stride, 8), max(go.row_stride, 8)
        a.in_dtype, a.out_dtype = R.DTYPE_CODE[src.view.dtype], R.DTYPE_CODE[tgt.view.dtype]
        a.f16_arith = 1 if m["arith"] == "f16" else 0
        a.max_is_maxnum = 1 if m["maxop"] == "arith.maxnumf" else 0
        a.max_init, a.sum_init = m["max_init"], m["sum_init"]
        self.table = table
        self._sel, self._n_lead, self._dev, self.rounds = sel, n_lead, dev, None
        self.dev_table = dev.upload(table)
        a.dev_item_offsets = self.dev_table
        self.device_arrays = [self.dev_table]
        self.elems = int(table.shape[0]) * gi.rows * cols
        self._bytes = self.elems * (bytes_per_elem(src.view.dtype) + bytes_per_elem(tgt.view.dtype))

    def launch(self, dev, arena_ptr):
        self.args.arena = arena_ptr
        if self.rounds:
            for lo, hi in self.rounds:
                sub = _copy_args(self.args)
                sub.dev_item_offsets = self.dev_table + lo * 2 * 8
                sub.n_items = hi - lo
                dev.check(dev.lib.ktb_launch_row_softmax(dev.h, C.byref(sub)))
            return
        dev.check(dev.lib.ktb_launch_row_softmax(dev.h, C.byref(self.args)))

    def order_points(self, rounds: Dict[int, int]):
        _order_item_table(self, self._sel, self._n_lead, rounds, self._dev)

    def split(self, piece_bytes: int):
        if self.rounds:
            return None
        a = self.args
        geoms = [(a.rows_per_item, int(a.in_row_stride), a.cols), (a.rows_per_item, int(a.out_row_stride), a.cols)]
        bpes = [2 if d == R.KTB_F16 else 4 for d in (a.in_dtype, a.out_dtype)]

        def part(lo, hi):
            sub = _copy_args(a)
            sub.dev_item_offsets = self.dev_table + lo * 2 * 8
            sub.n_items = hi - lo
            return ("ktb_launch_row_softmax", sub)
        return _split_item_table(self, self.table, geoms, bpes, part, piece_bytes)

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


# ---------------------------------------------------------------------------
# Hazards and plans
# ---------------------------------------------------------------------------
def check_hazards(fps: List[Footprint]):
    """Reject plans where concurrent cores / iterations would observe each other's writes.

    All byte runs of all statements are sorted; a run that is written may only
    coincide exactly with runs of the same (statement, point) — an in-place
    update — or with runs of the same core in another statement (program order
    on one core is kept by launch order).  Any other overlap involving a write
    means the sequential core order of the reference matters.

    One such case has a device path and is returned instead of raised: byte runs that several
    points of ONE statement store to and nobody else touches (every core writing the same
    result tile, say).  The reference leaves the value of the last point in core-major order
    (ktir_cpu/grid.py:595-613); the caller orders the statement's launches accordingly.
    Returns {statement: [arrays of point ids sharing a run]}."""
    if not fps or not any(f.write for f in fps):
        return {}
    starts = np.concatenate([f.starts for f in fps])
    ends = np.concatenate([f.ends for f in fps])
    if not len(starts):
        return {}
    write = np.concatenate([np.full(len(f.starts), f.write) for f in fps])
    stmt = np.concatenate([np.full(len(f.starts), f.stmt, np.int64) for f in fps])
    point = np.concatenate([f.points for f in fps])
    core = np.concatenate([f.cores for f in fps])
    order = np.lexsort((ends, starts))
    starts, ends, write, stmt, point, core = (x[order] for x in (starts, ends, write, stmt, point, core))
    new = np.ones(len(starts), bool)
    new[1:] = (starts[1:] != starts[:-1]) | (ends[1:] != ends[:-1])
    gid = np.cumsum(new) - 1
    ng = int(gid[-1]) + 1
    g_write = np.zeros(ng, bool)
    np.logical_or.at(g_write, gid, write)
    # identical runs: with a writer in the group every member must be the same core, and members
    # of one statement the same point
    first = np.flatnonzero(new)
    same_core = core == core[first][gid]
    bad = g_write[gid] & ~same_core
    key = stmt * (int(point.max()) + 1) + point
    srt = np.lexsort((key, stmt, gid))
    g2, s2, k2 = gid[srt], stmt[srt], key[srt]
    clash = (g2[1:] == g2[:-1]) & (s2[1:] == s2[:-1]) & (k2[1:] != k2[:-1]) & g_write[g2[1:]]
    ordered: Dict[int, List[np.ndarray]] = {}
    if bad.any() or clash.any():
        # groups whose members are all writes of one statement by known points can be ordered
        g_all_write = np.ones(ng, bool)
        np.logical_and.at(g_all_write, gid, write)
        g_stmt_lo = np.full(ng, np.iinfo(np.int64).max)
        g_stmt_hi = np.full(ng, -1)
        np.minimum.at(g_stmt_lo, gid, stmt)
        np.maximum.at(g_stmt_hi, gid, stmt)
        g_known = np.ones(ng, bool)
        np.logical_and.at(g_known, gid, point >= 0)
        fixable = g_all_write & (g_stmt_lo == g_stmt_hi) & g_known
        trouble = np.zeros(ng, bool)
        trouble[gid[bad]] = True
        trouble[g2[1:][clash]] = True
        if (trouble & ~fixable).any():
            raise CoreOrderHazard("memory written by one core/iteration is accessed by another: "
                              "sequential core order matters and has no device path yet")
        for g in np.flatnonzero(trouble):
            members = np.unique(point[gid == g])
            ordered.setdefault(int(g_stmt_lo[g]), []).append(members)
    # partial overlaps between distinct runs
    us, ue = starts[first], ends[first]
    k = np.searchsorted(us, ue, side="left")        # runs i+1 .. k-1 start inside run i
    idx = np.arange(ng)
    cw = np.concatenate([[0], np.cumsum(g_write)])
    writes_after = cw[k] - cw[np.minimum(idx + 1, ng)]
    if ((k > idx + 1) & (g_write | (writes_after > 0))).any():
        raise CoreOrderHazard("overlapping tile stores/loads across cores or iterations: "
                          "sequential core order matters and has no device path yet")
    return ordered


def _reads_overlap_writes(fps: List[Footprint]) -> bool:
    """True if some byte run a statement reads overlaps a run it writes without being that very run
    (an in-place update of the same run is what the fused kernels are built for)."""
    reads = [f for f in fps if not f.write and len(f.starts)]
    writes = [f for f in fps if f.write and len(f.starts)]
    if not reads or not writes:
        return False
    rs, re_ = np.concatenate([f.starts for f in reads]), np.concatenate([f.ends for f in reads])
    ws, we = np.concatenate([f.starts for f in writes]), np.concatenate([f.ends for f in writes])
    if len(rs) * len(ws) > (1 << 22):
        return bool(rs.min() < we.max() and ws.min() < re_.max())       # too many runs to compare: go by the hulls
    over = (rs[:, None] < we[None, :]) & (ws[None, :] < re_[:, None])
    same = (rs[:, None] == ws[None, :]) & (re_[:, None] == we[None, :])
    return bool((over & ~same).any())


def launch_rounds(groups: List[np.ndarray]) -> Dict[int, int]:
    """Round of every point that shares a stored run with another point: points are taken in
    sequential (core-major) order and each goes one round after the latest earlier point it
    collides with, so launching the rounds in order reproduces last-writer-wins."""
    rounds: Dict[int, int] = {}
    by_point: Dict[int, List[np.ndarray]] = {}
    for g in groups:
        for p in g:
            by_point.setdefault(int(p), []).append(g)
    for p in sorted(by_point):
        r = 0
        for g in by_point[p]:
            for q in g:
                q = int(q)
                if q < p and q in rounds:
                    r = max(r, rounds[q] + 1)
        rounds[p] = r
    return rounds


class Plan:
    """Everything needed to run one (function, scalars, tensor layout) on the device."""

    def __init__(self):
        self.statements: List[Statement] = []
        self.written: set = set()
        self.fully_overwritten: set = set()
        self.core_groups: Optional[List[Tuple[int, int]]] = None     # set when the cores run group after group
        self.unrolled_groups: List[Tuple[int, int]] = []             # ... and the groups whose loops run iteration by iteration

    def launch(self, dev: R.Device, arena_ptr: int):
        for s in self.statements:
            s.launch(dev, arena_ptr)

    def written_ranges(self) -> List[Tuple[int, int]]:
        """Arena byte ranges the launches write, merged and sorted."""
        runs = []
        for s in self.statements:
            own = getattr(s, "owned_range", None)
            if own is not None:
                runs.append(np.array([own], np.int64))
                continue
            for f in s.footprints():
                if f.write and len(f.starts):
                    runs.append(np.stack([f.starts, f.ends], 1).astype(np.int64))
        if not runs:
            return []
        r = np.concatenate(runs)
        r = r[np.argsort(r[:, 0], kind="stable")]
        hi = np.maximum.accumulate(r[:, 1])
        new = np.ones(len(r), bool)
        new[1:] = r[1:, 0] > hi[:-1]
        first = np.flatnonzero(new)
        last = np.concatenate([first[1:] - 1, [len(r) - 1]])
        return [(int(r[a, 0]), int(hi[b])) for a, b in zip(first, last)]

    def release(self, dev: R.Device):
        for s in self.statements:
            for p in getattr(s, "device_arrays", []):
                dev.free(p)
        self.statements = []


def lower_core_groups(dev: R.Device, trace_cores, n_cores: int, arena: ArenaMap, fused: bool = True) -> Plan:
    """Plan for a grid whose cores cannot all run at once (``CoreOrderHazard``): the cores are cut into
    consecutive groups that pass the hazard check on their own, and the groups' plans run one after the
    other — inside a group nothing clashes, between groups the launch order is the reference's core
    order (ktir_cpu/grid.py:595-613), so the memory a later core sees and the bytes that survive are
    the reference's.  ``trace_cores(lo, hi, unroll)`` returns the traced stores of cores [lo, hi).  A
    group that clashes because iterations of an ``scf.for`` read or overwrite each other's bytes is
    traced with its loops unrolled instead: every iteration's store becomes a statement of its own and
    they run in program order."""
    groups: List[Tuple[int, int, bool]] = []
    probe = R.PlanOnlyDevice()
    lo, last = 0, n_cores
    while lo < n_cores:
        # the whole grid is known to clash; after that, try twice the size that last worked
        size = min(n_cores - lo, 2 * last) if lo else n_cores
        while True:
            # as they are; else with the loops unrolled (iterations that clash, cores that do not); else fewer cores
            unroll = False
            try:
                lower(probe, trace_cores(lo, lo + size, False), arena, fused=fused)
                break
            except CoreOrderHazard as plain:
                try:
                    lower(probe, trace_cores(lo, lo + size, True), arena, fused=fused)
                    unroll = True
                    break
                except Unsupported as unrolled:
                    if size == 1:
                        raise (unrolled if isinstance(unrolled, CoreOrderHazard) else plain)
            size = max(1, size // 2)
        groups.append((lo, lo + size, unroll))
        lo, last = lo + size, size
    plan = Plan()
    try:
        for lo, hi, unroll in groups:
            part = lower(dev, trace_cores(lo, hi, unroll), arena, fused=fused)
            plan.statements.extend(part.statements)
            plan.written |= part.written
    except Exception:
        plan.release(dev)
        raise
    plan.core_groups = [(lo, hi) for lo, hi, _ in groups]
    plan.unrolled_groups = [(lo, hi) for lo, hi, unroll in groups if unroll]
    return plan


def _fused_statement(dev, st: Store, arena: ArenaMap, sid: int, row_shard):
    """The fused kernel that fits this store, trying the idioms in a fixed order."""
    if isinstance(st.target, IndirectAccess):
        from .lower_scatter import lower_indirect_store
        return lower_indirect_store(dev, st, arena, sid, row_shard)
    m = match_softmax(st.value)
    if m is not None:
        return SoftmaxStatement(dev, st, m, arena, sid)
    from .lower_mm import try_lower_matmul
    stmt = try_lower_matmul(dev, st, arena, sid)
    if stmt is None:
        from .lower_attn import try_lower_attention
        stmt = try_lower_attention(dev, st, arena, sid)
    if stmt is None:
        from .lower_rowprog import try_lower_row_program
        stmt = try_lower_row_program(dev, st, arena, sid)
    if stmt is None:
        from .lower_scatter import RowsStatement, has_indirect_load
        if has_indirect_load(st.value):
            stmt = RowsStatement(dev, st, arena, sid)
    if stmt is None:
        stmt = EwStatement(dev, st, arena, sid)
    return stmt


# A statement that stores one value per row made of its neighbour's row reductions joins that neighbour's launch.
# (Switch for tests that want the stand-alone per-row statements.)
FUSE_ROW_RESULTS = True


def lower(dev: R.Device, stores: List[Store], arena: ArenaMap, row_shard=None, fused: bool = True) -> Plan:
    """``row_shard = (rank, world)``: ordered scatters apply only the destination rows this rank owns.
    ``fused=False`` skips the fused kernels and runs every direct store step by step (the op-by-op
    form of the reference, ktir_cpu/interpreter.py:196-281) — a cross-check for the fused paths."""
    from .order import program_order
    stores = [stores[k] for k in program_order(stores, arena)]
    plan = Plan()
    groups: List[List[Store]] = []          # the stores behind each statement (a row program may take in its neighbours)

    def per_row_program(s) -> bool:
        return s.kind == "row_program" and bool(s.args.out_per_row) and len(s.stores) == 1

    for st in stores:
        sid = len(plan.statements)
        last = plan.statements[-1] if plan.statements else None
        if FUSE_ROW_RESULTS and last is not None and last.kind == "row_program" and not last.args.out_per_row and \
                last.try_absorb(st):
            groups[-1].append(st)           # a per-row result of the statement before it: same launch
            continue
        try:
            if not fused and not isinstance(st.target, IndirectAccess):
                raise Unsupported("fused kernels disabled")
            stmt = _fused_statement(dev, st, arena, sid, row_shard)
        except Unsupported:
            # no fused kernel fits: run the tile program step by step
            if row_shard is not None and isinstance(st.target, IndirectAccess):
                raise
            from .lower_generic import generic_statement
            stmt = generic_statement(dev, st, arena, sid)
        group = [st]
        if FUSE_ROW_RESULTS and stmt.kind == "row_program" and not stmt.args.out_per_row:
            # ... and per-row results stored just before it
            while plan.statements and per_row_program(plan.statements[-1]) and stmt.try_absorb(groups[-1][0]):
                for ptr in plan.statements.pop().device_arrays:
                    dev.free(ptr)
                group = groups.pop() + group
            stmt.renumber(len(plan.statements))
        plan.statements.append(stmt)
        groups.append(group)
    pts = [_points(st) for st in stores]
    if stores and row_shard is None and all(len(p[0]) <= 1 for p in pts) and \
            len({int(p[1][0]) for p in pts if len(p[0])}) <= 1:
        # One core, every store executed once: the statements run in program order as they are, nothing is
        # concurrent.  What is left is a statement whose own inputs overlap its output (an index tensor that
        # shares bytes with the destination, say): the step-by-step form reads everything before it writes,
        # as the reference's load and store ops do; a fused kernel does not promise that.
        redo = []
        for stmt, group in zip(plan.statements, groups):
            if stmt.kind != "generic" and _reads_overlap_writes(stmt.footprints()):
                from .lower_generic import generic_statement
                for ptr in getattr(stmt, "device_arrays", []):
                    dev.free(ptr)
                base = len(redo)
                redo.extend([generic_statement(dev, st, arena, base + k) for k, st in enumerate(group)])
            else:
                redo.append(stmt)
        plan.statements = redo
    else:
        fps = [f for s in plan.statements for f in s.footprints()]
        for sid, groups in check_hazards(fps).items():
            stmt = plan.statements[sid]
            if not hasattr(stmt, "order_points"):
                raise CoreOrderHazard(f"several cores store to the same bytes in a {stmt.kind} statement: "
                                      "sequential core order matters and has no device path yet")
            stmt.order_points(launch_rounds(groups))
    read_names, write_runs = set(), {}
    for s in plan.statements:
        for f in s.footprints():
            if not len(f.starts):
                continue
            a = arena.find(int(f.starts[0]))
            if a is None:
                continue
            if f.write:
                plan.written.add(a.name)
                write_runs.setdefault(a.name, []).append((f.starts, f.ends))
            else:
                read_names.add(a.name)
        for name in getattr(s, "extra_written", []):
            plan.written.add(name)
            read_names.add(name)
    # tensors whose every byte is stored and none is loaded: their old contents cannot matter
    for a in arena.allocs:
        if a.name in write_runs and a.name not in read_names:
            st = np.concatenate([x for x, _ in write_runs[a.name]])
            en = np.concatenate([y for _, y in write_runs[a.name]])
            runs = np.unique(np.stack([st, en], 1), axis=0)
            if int((runs[:, 1] - runs[:, 0]).sum()) == a.byte_hi - a.byte_lo and runs[:, 0].min() == a.byte_lo:
                plan.fully_overwritten.add(a.name)
    return plan

"""Fallback lowering: any traced tile DAG as a list of simple whole-grid device steps.

The idiom matchers (softmax rows, GEMM, attention, row gather/scatter, elementwise
streams) cover the kernels that matter for speed.  Everything else — reductions in the
reference's halving order, broadcasts, transposes, small matmuls, integer tiles, general
indirect access tiles — is run op by op, like the reference does
(ktir_cpu/interpreter.py:196-281), except that one step handles every active iteration
point (core x loop iterations) at once.  A step works on buffers of ``[points, elements]``
in a scratch area; the step kinds are few and generic (``GenOp``): loads / stores through a
per-point base plus per-element offsets, gathers / scatters through an address buffer,
elementwise ops with scalar broadcast, an index map (broadcast / transpose / extract), one
level of the pairwise reduction tree, a plain matmul.

Numerics follow the reference: f16 tiles compute in f32 and round after every op
(ktir_cpu/dialects/_helpers.py:39-54), integer tiles wrap in their width, reductions fold
``x[0:h] (+) x[h:2h]`` with the odd tail carried (ktir_cpu/dialects/linalg_ops.py:86-133),
f16 matmul accumulates in f32 over k in order and rounds once (ktir_cpu/ops/arith_ops.py:323-340).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from .dtypes import bytes_per_elem, to_np_dtype
from .trace import Access, IndirectAccess, LoopInfo, Node, Store, TableAccess, Unsupported, iv_full

NP_DT = {"f16": np.float16, "f32": np.float32, "i32": np.int32, "i64": np.int64, "i1": np.uint8, "index": np.int64}
ITEM = {"f16": 2, "f32": 4, "i32": 4, "i64": 8, "i1": 1, "index": 8}

# elementwise opcodes (shared with the device switch)
EW_OPS = ["mov", "add", "sub", "mul", "div", "rem", "max", "maxnum", "min", "minnum", "neg", "abs", "exp", "log",
          "log2", "log1p", "sqrt", "rsqrt", "tanh", "sin", "cos", "ceil", "floor", "fma", "pow", "select",
          "cmp_eq", "cmp_ne", "cmp_lt", "cmp_le", "cmp_gt", "cmp_ge", "cmp_ord", "cmp_uno", "cmp_true", "cmp_false",
          "and", "or", "xor", "shl", "shr", "divt", "remt", "divf", "cdiv", "bitcast", "cmp_une_", "cmp_ueq_",
          "cmp_ult_", "cmp_ule_", "cmp_ugt_", "cmp_uge_", "sign"]
EW_CODE = {n: i for i, n in enumerate(EW_OPS)}

_FLOAT_EW = {"arith.addf": "add", "arith.subf": "sub", "arith.mulf": "mul", "arith.divf": "div", "arith.remf": "rem",
             "arith.maximumf": "max", "arith.maxnumf": "maxnum", "arith.minimumf": "min", "arith.minnumf": "minnum",
             "arith.negf": "neg", "math.absf": "abs", "math.exp": "exp", "math.log": "log", "math.log2": "log2",
             "math.log1p": "log1p", "math.sqrt": "sqrt", "math.rsqrt": "rsqrt", "math.tanh": "tanh",
             "math.sin": "sin", "math.cos": "cos", "math.ceil": "ceil", "math.floor": "floor", "math.fma": "fma",
             "math.powf": "pow", "arith.select": "select", "math.sign": "sign"}
_INT_EW = {"arith.addi": "add", "arith.subi": "sub", "arith.muli": "mul", "arith.divui": "divf",
           "arith.floordivsi": "divf", "arith.divsi": "divt", "arith.remui": "rem", "arith.remsi": "remt",
           "arith.andi": "and", "arith.ori": "or", "arith.xori": "xor", "arith.shli": "shl", "arith.shrsi": "shr",
           "arith.shrui": "shr", "arith.minsi": "min", "arith.maxsi": "max", "arith.minui": "min", "arith.maxui": "max",
           "arith.ceildivsi": "cdiv", "arith.ceildivui": "cdiv"}
_CMPI = {"slt": "cmp_lt", "ult": "cmp_lt", "sle": "cmp_le", "ule": "cmp_le", "sgt": "cmp_gt", "ugt": "cmp_gt",
         "sge": "cmp_ge", "uge": "cmp_ge", "eq": "cmp_eq", "ne": "cmp_ne"}
_CMPF = {"oeq": "cmp_eq", "ogt": "cmp_gt", "oge": "cmp_ge", "olt": "cmp_lt", "ole": "cmp_le", "one": "cmp_ne",
         "ord": "cmp_ord", "uno": "cmp_uno", "true": "cmp_true", "false": "cmp_false", "une": "cmp_une_",
         "ueq": "cmp_ueq_", "ult": "cmp_ult_", "ule": "cmp_ule_", "ugt": "cmp_ugt_", "uge": "cmp_uge_"}


@dataclass
class Buf:
    """A ``[points, elems]`` array of ``dtype`` in the scratch area."""
    id: int
    dtype: str
    elems: int
    shape: Tuple[int, ...]
    offset: int = -1          # byte offset in the scratch area (assigned by ``GenProgram.place``)


@dataclass
class GenOp:
    kind: str
    dst: Optional[Buf] = None
    srcs: Tuple[Buf, ...] = ()
    attrs: Dict[str, Any] = field(default_factory=dict)


def _prod(shape) -> int:
    return int(np.prod(shape, dtype=np.int64)) if len(shape) else 1


class GenProgram:
    """Steps of one store statement plus the host tables they reference."""

    def __init__(self, n_points: int):
        self.P = n_points
        self.ops: List[GenOp] = []
        self.bufs: List[Buf] = []
        self.scratch_bytes = 0

    def new(self, dtype: str, shape) -> Buf:
        dtype = "i64" if dtype == "index" else dtype
        b = Buf(len(self.bufs), dtype, _prod(shape), tuple(shape))
        self.bufs.append(b)
        return b

    def emit(self, kind: str, dst: Optional[Buf], srcs=(), **attrs) -> Optional[Buf]:
        self.ops.append(GenOp(kind, dst, tuple(srcs), attrs))
        return dst

    def place(self):
        """Assign scratch offsets; a buffer's space is reused after its last reader."""
        last = {}
        for i, op in enumerate(self.ops):
            for b in op.srcs:
                last[b.id] = i
            if op.dst is not None:
                last.setdefault(op.dst.id, i)
        free: List[Tuple[int, int]] = []          # (size, offset)
        top = 0
        expiring: Dict[int, List[Buf]] = {}
        for b in self.bufs:
            expiring.setdefault(last.get(b.id, -1), []).append(b)
        sized = {}
        for i, op in enumerate(self.ops):
            b = op.dst
            if b is not None and b.offset < 0:
                need = ((b.elems * self.P * ITEM[b.dtype]) + 255) & ~255
                pick = None
                for k, (sz, off) in enumerate(free):
                    if sz >= need and (pick is None or sz < free[pick][0]):
                        pick = k
                if pick is not None:
                    sz, off = free.pop(pick)
                    b.offset = off
                    sized[b.id] = sz
                else:
                    b.offset = top
                    top += need
                    sized[b.id] = need
            for dead in expiring.get(i, []):
                if dead.offset >= 0 and dead.id in sized:
                    free.append((sized.pop(dead.id), dead.offset))
        self.scratch_bytes = max(top, 256)


def _row_major_strides(shape) -> List[int]:
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= n
    return list(reversed(st))


def access_rel_offsets(acc: Access) -> np.ndarray:
    """Element offsets of every element of a direct tile relative to its origin, row-major."""
    if acc.coords is not None:
        return (acc.coords * np.asarray(acc.strides, np.int64)[None, :]).sum(1)
    shape = tuple(acc.shape) or (1,)
    strides = tuple(acc.strides) or (1,)
    rel = np.zeros(shape, np.int64)
    for d, (n, s) in enumerate(zip(shape, strides)):
        rs = [1] * len(shape)
        rs[d] = n
        rel = rel + (np.arange(n, dtype=np.int64) * s).reshape(rs)
    return rel.reshape(-1)


class GenBuilder:
    """Turns the DAG of one store into a ``GenProgram``."""

    def __init__(self, store: Store, arena, sel: np.ndarray):
        self.store = store
        self.arena = arena
        self.sel = sel
        self.A = len(store.axes)
        self.prog = GenProgram(len(sel))
        self.memo: Dict[Any, Buf] = {}
        self.loop_runs: Dict[Any, List[Buf]] = {}
        self.depth_memo: Dict[int, int] = {}
        self.loads: List[Tuple[Access, Tuple[int, ...]]] = []       # direct loads, for the hazard check
        self.tables: List[Tuple[np.ndarray, str, bool]] = []        # (addresses [points, elems], dtype, written)
        self.indirect_reads: List[Any] = []                          # allocations read through address buffers
        self.loop_state: Dict[Any, List[Buf]] = {}

    # -- iteration-space values at the store's points (and loop indices) -------------------------
    def at_points(self, v, ks: Tuple[int, ...], trips: Tuple[int, ...]) -> np.ndarray:
        axes = tuple(self.store.axes) + trips
        full = iv_full(v, axes).reshape((-1,) + trips)
        out = full[self.sel]
        for k in ks:
            out = out[:, k]
        return np.ascontiguousarray(out).astype(np.int64)

    def table_at_points(self, addr: np.ndarray, ks: Tuple[int, ...], trips: Tuple[int, ...]) -> np.ndarray:
        """Rows of an address table (iteration space + element axis) for the selected points."""
        axes = tuple(self.store.axes) + trips
        lead, E = addr.shape[:-1], addr.shape[-1]
        v = addr.reshape(lead + (1,) * (len(axes) - len(lead)) + (E,))
        full = np.broadcast_to(v, axes + (E,)).reshape((-1,) + trips + (E,))
        out = full[self.sel]
        for k in ks:
            out = out[:, k]
        return np.ascontiguousarray(out, np.int64)

    def depth(self, n: Node) -> int:
        d = self.depth_memo.get(id(n))
        if d is not None:
            return d
        if n.kind in ("load", "iload", "tload"):
            d = max(0, len(n.attrs["axes"]) - self.A)
        elif n.kind == "param":
            v = n.attrs["values"]
            d = max(0, (v.ndim if isinstance(v, np.ndarray) else 0) - self.A)
        elif n.kind == "iter":
            d = n.attrs["loop"].axis - self.A + 1
        elif n.kind == "loopres":
            info: LoopInfo = n.attrs["loop"]
            d = max([info.axis - self.A] + [self.depth(x) for x in info.inits if isinstance(x, Node)])
            d = max(d, 0)
        else:
            d = max([0] + [self.depth(a) for a in n.args])
        self.depth_memo[id(n)] = d
        return d

    # -- helpers -------------------------------------------------------------------------------
    def fill(self, value, dtype: str, shape=()) -> Buf:
        return self.prog.emit("fill", self.prog.new(dtype, shape), (), value=value)

    def as_shape(self, b: Buf, shape) -> Buf:
        """``b`` broadcast NumPy-style (right aligned) to ``shape``; scalars stay scalars."""
        shape = tuple(shape)
        if b.elems == _prod(shape) or b.elems == 1:
            return b
        src_shape = (1,) * (len(shape) - len(b.shape)) + tuple(b.shape)
        st = _row_major_strides(src_shape)
        strides = [0 if s == 1 else t for s, t in zip(src_shape, st)]
        for s, o in zip(src_shape, shape):
            if s != 1 and s != o:
                raise Unsupported(f"cannot broadcast tile {b.shape} to {shape}")
        return self.prog.emit("map", self.prog.new(b.dtype, shape), (b,), shape=shape, strides=strides, offset=0)

    def ew(self, opname: str, dtype: str, shape, srcs: List[Buf], **attrs) -> Buf:
        srcs = [self.as_shape(s, shape) for s in srcs]
        return self.prog.emit("ew", self.prog.new(dtype, shape), srcs, op=opname, **attrs)

    def alloc_of(self, elem_addr: int, dtype: str, what: str):
        a = self.arena.find(int(elem_addr) * bytes_per_elem(dtype))
        if a is None:
            raise ValueError(f"{what} unmapped address 0x{int(elem_addr) * bytes_per_elem(dtype):x}")
        return a

    # -- evaluation ------------------------------------------------------------------------------
    def eval(self, n: Node, ks: Tuple[int, ...] = (), loops: Tuple[LoopInfo, ...] = ()) -> Buf:
        d = self.depth(n)
        key = (id(n), ks[:d])
        b = self.memo.get(key)
        if b is None:
            b = self._eval(n, ks[:d], loops[:d])
            self.memo[key] = b
        return b

    def _eval(self, n: Node, ks, loops) -> Buf:
        k = n.kind
        P = self.prog
        trips = tuple(l.trips for l in loops)
        if k == "load":
            acc: Access = n.attrs["access"]
            base = self.at_points(acc.off, ks, trips)
            rel = access_rel_offsets(acc)
            dt = acc.view.dtype
            al = self.alloc_of(base.min() if base.size else 0, dt, "Read from")
            bpe = bytes_per_elem(dt)
            self.loads.append((acc, ks, trips))
            return P.emit("load", P.new(dt, n.shape), (), base=base, rel=rel, lo=al.byte_lo // bpe, hi=al.byte_hi // bpe)
        if k == "tload":
            ta: TableAccess = n.attrs["access"]
            table = self.table_at_points(ta.addr, ks, trips)
            self.tables.append((table, ta.dtype, False))
            addr = P.emit("table", P.new("i64", (table.shape[1],)), (), values=table)
            return P.emit("gather", P.new(ta.dtype, n.shape), (addr,), lo=0, hi=ALL_MEMORY)
        if k == "iload":
            addr, al, dt = self.indirect_addresses(n.attrs["access"], ks, trips)
            bpe = bytes_per_elem(dt)
            self.indirect_reads.append(al)
            return P.emit("gather", P.new(dt, n.shape), (addr,), lo=al.byte_lo // bpe, hi=al.byte_hi // bpe)
        if k == "const":
            if n.attrs.get("list") is not None:
                table = np.asarray(n.attrs["list"]).astype(NP_DT[n.dtype]).reshape(-1)
                return P.emit("constv", P.new(n.dtype, n.shape), (), table=table)
            return self.fill(n.attrs["value"], n.dtype, ())          # a scalar; consumers broadcast it
        if k == "param":
            vals = self.at_points(n.attrs["values"], ks, trips)
            return P.emit("param", P.new(n.dtype, ()), (), values=vals.astype(NP_DT[n.dtype]))
        if k == "iota":
            return P.emit("iota", P.new("i64", n.shape), (), shape=tuple(n.shape), dim=n.attrs["dim"])
        if k in ("reshape",):
            src = self.eval(n.args[0], ks, loops)
            if src.elems == 1:
                return src
            return P.emit("ew", P.new(src.dtype, n.shape), (src,), op="mov")
        if k == "bcast":
            src = self.eval(n.args[0], ks, loops)
            if src.elems == 1:
                return src                                             # stays a scalar
            out = tuple(n.shape)
            if n.attrs.get("numpy"):
                return self.as_shape(src, out)
            dims = sorted(n.attrs.get("dims", []))
            kept = [d_ for d_ in range(len(out)) if d_ not in dims]
            sshape = tuple(n.args[0].shape)
            if len(kept) != len(sshape):
                return self.as_shape(src, out)
            st = _row_major_strides(sshape)
            strides = [0] * len(out)
            for j, d_ in enumerate(kept):
                strides[d_] = 0 if sshape[j] == 1 else st[j]
            return P.emit("map", P.new(src.dtype, out), (src,), shape=out, strides=strides, offset=0)
        if k == "transpose":
            src = self.eval(n.args[0], ks, loops)
            perm = n.attrs["perm"]
            st = _row_major_strides(n.args[0].shape)
            return P.emit("map", P.new(src.dtype, n.shape), (src,), shape=tuple(n.shape),
                          strides=[st[p] for p in perm], offset=0)
        if k == "slice":
            src = self._full(self.eval(n.args[0], ks, loops), n.args[0].shape)
            st = _row_major_strides(n.args[0].shape)
            return P.emit("map", P.new(src.dtype, n.shape), (src,), shape=tuple(n.shape), strides=list(st),
                          offset=int(n.attrs["lo"] * st[n.attrs["dim"]]))
        if k == "concat":
            a = self._full(self.eval(n.args[0], ks, loops), n.args[0].shape)
            b = self._full(self.eval(n.args[1], ks, loops), n.args[1].shape)
            d_ = n.attrs["dim"]
            return P.emit("concat", P.new(n.dtype, n.shape), (a, b), outer=_prod(n.shape[:d_]), na=int(n.args[0].shape[d_]),
                          nb=int(n.args[1].shape[d_]), inner=_prod(n.shape[d_ + 1:]))
        if k == "extract":
            src = self.eval(n.args[0], ks, loops)
            if src.elems == 1:
                return src
            st = _row_major_strides(n.args[0].shape)
            off = sum(i * s for i, s in zip(n.attrs["index"], st))
            return P.emit("map", P.new(src.dtype, ()), (src,), shape=(), strides=[], offset=int(off))
        if k == "cast":
            src = self.eval(n.args[0], ks, loops)
            return P.emit("ew", P.new(n.dtype, src.shape if src.elems > 1 else ()), (src,), op="mov")
        if k == "bitcast":
            src = self.eval(n.args[0], ks, loops)
            return P.emit("ew", P.new(n.dtype, src.shape if src.elems > 1 else ()), (src,), op="bitcast")
        if k == "ew":
            return self.eval_ew(n, ks, loops)
        if k == "reduce":
            return self.eval_reduce(n, ks, loops)
        if k == "matmul":
            return self.eval_matmul(n, ks, loops)
        if k == "ringred":
            return self.eval_ring(n, ks, loops)
        if k == "iter":
            info = n.attrs["loop"]
            return self.loop_state[(id(info), ks)][n.attrs["index"]]
        if k == "loopres":
            return self.run_loop(n.attrs["loop"], ks, loops)[n.attrs["index"]]
        raise Unsupported(f"{k} node has no device path")

    def run_loop(self, info: LoopInfo, ks, loops) -> List[Buf]:
        key = (id(info), ks)
        done = self.loop_runs.get(key)
        if done is not None:
            return done
        cur = [self.eval(x, ks, loops) for x in info.inits]
        for kk in range(info.trips):
            inner_ks, inner_loops = ks + (kk,), loops + (info,)
            self.loop_state[(id(info), inner_ks)] = cur
            cur = [self.eval(y, inner_ks, inner_loops) for y in info.yields]
        self.loop_runs[key] = cur
        return cur

    def eval_ew(self, n: Node, ks, loops) -> Buf:
        op = n.attrs["op"]
        srcs = [self.eval(a, ks, loops) for a in n.args]
        shape = tuple(n.shape) if any(s.elems > 1 for s in srcs) else ()
        if op == "arith.cmpi":
            return self.ew(_CMPI[n.attrs["pred"]], "i1", shape, srcs, cmp_int=1)
        if op == "arith.cmpf":
            pred = n.attrs["pred"]
            if pred not in _CMPF:
                raise NotImplementedError(f"arith.cmpf: unsupported predicate '{pred}'")
            return self.ew(_CMPF[pred], "i1", shape, srcs)
        if n.dtype in ("f16", "f32"):
            if op not in _FLOAT_EW:
                raise Unsupported(f"{op} on a float tile")
            # operands take the result dtype first (NumPy promotes, a scalar was coerced when traced)
            return self.ew(_FLOAT_EW[op], n.dtype, shape, srcs)
        if op == "arith.select":
            return self.ew("select", n.dtype, shape, srcs)
        if op not in _INT_EW:
            raise Unsupported(f"{op} on an integer tile")
        return self.ew(_INT_EW[op], n.dtype, shape, srcs)

    def eval_reduce(self, n: Node, ks, loops) -> Buf:
        src_node = n.args[0]
        cur = self.eval(src_node, ks, loops)
        comb = n.attrs["op"]
        code = _FLOAT_EW.get(comb) or _INT_EW.get(comb)
        if code is None:
            raise Unsupported(f"linalg.reduce with combiner {comb}")
        shape = list(src_node.shape)
        if cur.elems == 1 and _prod(shape) > 1:
            cur = self.prog.emit("map", self.prog.new(cur.dtype, shape), (cur,), shape=tuple(shape),
                                 strides=[0] * len(shape), offset=0)
        dims = n.attrs["dims"]
        if dims is None:
            shape, fold = [_prod(shape)], [0]
        else:
            fold = sorted(dims, reverse=True)
        for d in fold:
            m = shape[d]
            outer, inner = _prod(shape[:d]), _prod(shape[d + 1:])
            while m > 1:
                h = m // 2
                nm = h + (m % 2)
                lvl = list(shape)
                lvl[d] = nm
                cur = self.prog.emit("redl", self.prog.new(n.dtype, lvl), (cur,), op=code, outer=outer, n=m, inner=inner, h=h)
                m = nm
            shape[d] = 1
        if cur.elems != _prod(n.shape):
            raise Unsupported("reduce result shape mismatch")
        out = self.prog.new(n.dtype, n.shape)
        return self.prog.emit("ew", out, (cur,), op="mov")

    def eval_ring(self, n: Node, ks, loops) -> Buf:
        """``ktdp.inter_tile_reduce``: per point the fold of its partial with those of the other cores
        of its group, in ring arrival order (see ``trace_comm``).  Points are core-major, so the
        partial of core ``s`` at the same loop indices is point ``s * inner + p % inner``."""
        if n.dtype not in ("f16", "f32"):
            raise Unsupported(f"inter_tile_reduce of a {n.dtype} tile")
        axes = tuple(self.store.axes)
        P_all = _prod(axes)
        if self.prog.P != P_all:
            raise Unsupported("inter_tile_reduce evaluated on part of the grid")
        src = self._full(self.eval(n.args[0], ks, loops), n.args[0].shape)
        code = _FLOAT_EW.get(n.attrs["op"])
        if code is None:
            raise Unsupported(f"inter_tile_reduce with combiner {n.attrs['op']}")
        inner = P_all // axes[0]
        srcs, counts, groups = n.attrs["sources"], n.attrs["counts"], n.attrs["groups"]
        S = srcs.shape[1]
        core = np.arange(P_all, dtype=np.int64) // inner
        lane = np.arange(P_all, dtype=np.int64) % inner
        pts = np.where(srcs[core] >= 0, srcs[core] * inner + lane[:, None], -1)
        # one cluster per (group, loop point) when every group has the same size of at most 8 cores
        members = {int(g): np.flatnonzero(groups == g) for g in np.unique(groups)}
        sizes = {len(m) for m in members.values()}
        cluster, order, ranks = 0, None, None
        if len(sizes) == 1 and 1 < next(iter(sizes)) <= 8:
            cluster = next(iter(sizes))
            rank_of = np.zeros(axes[0], np.int64)
            for m in members.values():
                rank_of[m] = np.arange(len(m))
            same_group = (srcs < 0) | (groups[np.clip(srcs, 0, None)] == groups[:, None])
            if same_group.all():
                order = np.concatenate([(m[None, :] * inner + np.arange(inner)[:, None]).reshape(-1)
                                        for m in members.values()]).astype(np.int64)
                ranks = np.where(srcs[core] >= 0, rank_of[np.clip(srcs[core], 0, None)], -1)
            else:
                cluster = 0
        return self.prog.emit("ringred", self.prog.new(n.dtype, n.shape), (src,), op=code, swapped=bool(n.attrs["swapped"]),
                              counts=counts[core].astype(np.int64), sources=(ranks if cluster else pts).astype(np.int64),
                              cluster=cluster, order=order, S=S)

    def eval_matmul(self, n: Node, ks, loops) -> Buf:
        a_n, b_n = n.args[0], n.args[1]
        a, b = self.eval(a_n, ks, loops), self.eval(b_n, ks, loops)
        acc = self.eval(n.args[2], ks, loops) if len(n.args) > 2 else None
        if len(a_n.shape) < 2 or len(b_n.shape) < 2 or a_n.shape[-1] != b_n.shape[-2]:
            raise Unsupported(f"matmul of tiles {a_n.shape} x {b_n.shape}")
        batch = _prod(a_n.shape[:-2])
        if _prod(b_n.shape[:-2]) != batch:
            raise Unsupported("matmul with broadcast batch dimensions")
        M, K, N = a_n.shape[-2], a_n.shape[-1], b_n.shape[-1]
        a = self._full(a, a_n.shape)
        b = self._full(b, b_n.shape)
        prod_dt = a_n.dtype if a_n.dtype == b_n.dtype else "f32"
        prod = self.prog.emit("matmul", self.prog.new(prod_dt, n.shape), (a, b), batch=batch, M=M, N=N, K=K)
        if acc is None:
            return prod
        return self.ew("add", n.dtype, tuple(n.shape), [acc, prod])

    def _full(self, b: Buf, shape) -> Buf:
        if b.elems == _prod(shape):
            return b
        return self.prog.emit("map", self.prog.new(b.dtype, shape), (b,), shape=tuple(shape),
                              strides=[0] * len(shape), offset=0)

    def _indirect_affine(self, ia: IndirectAccess, ks, trips, vars_e, nv: int, E: int) -> Buf:
        """Subscripts affine in the variables: address = per-point base + per-element offset (+ lookups)."""
        from .lower_scatter import _lin
        P = self.prog
        base = self.at_points(ia.view.base, ks, trips)
        rel = np.zeros(E, np.int64)
        lookups = []
        pending_reads = []
        for sub, stride in zip(ia.subs, ia.view.strides):
            if sub["kind"] == "direct":
                c, b = _lin(sub["expr"], nv, ia.ssa)
                rel += stride * (np.asarray(c, np.int64)[:, None] * vars_e).sum(0)
                base = base + stride * self.at_points(b, ks, trips)
            else:
                iv = ia.index_views[sub["view"]]
                ibase = self.at_points(iv.base, ks, trips)
                irel = np.zeros(E, np.int64)
                for e_, s_ in zip(sub["exprs"], iv.strides):
                    c, b = _lin(e_, nv, ia.ssa)
                    irel += s_ * (np.asarray(c, np.int64)[:, None] * vars_e).sum(0)
                    ibase = ibase + s_ * self.at_points(b, ks, trips)
                ial = self.alloc_of(ibase.min() if ibase.size else 0, iv.dtype, "Read from")
                pending_reads.append(ial)
                lookups.append((iv.dtype, ibase, irel, ial, int(stride)))
        # nothing is emitted before every subscript has proved affine
        self.indirect_reads.extend(pending_reads)
        addr = P.emit("addr", P.new("i64", (E,)), (), base=base, rel=rel)
        for idt, ibase, irel, ial, stride in lookups:
            ibpe = bytes_per_elem(idt)
            idx = P.emit("load", P.new(idt, (E,)), (), base=ibase, rel=irel, lo=ial.byte_lo // ibpe, hi=ial.byte_hi // ibpe)
            addr = P.emit("idxadd", P.new("i64", (E,)), (addr, idx), stride=stride)
        return addr

    def _indirect_tabulated(self, ia: IndirectAccess, ks, trips, vars_e, E: int) -> Buf:
        """Any quasi-affine subscripts (``floordiv`` / ``mod`` of the variables — a position split into
        page and slot, ktir_cpu/ops/memory_ops.py:488-576): the host evaluates them for every point and
        element and hands the device tables of addresses."""
        from .lower_scatter import sub_values
        P = self.prog

        def at(name):
            return self.at_points(ia.ssa[name], ks, trips)
        n_pts = len(self.sel)
        table = np.broadcast_to(self.at_points(ia.view.base, ks, trips)[:, None], (n_pts, E)).astype(np.int64)
        lookups = []
        for sub, stride in zip(ia.subs, ia.view.strides):
            if sub["kind"] == "direct":
                table = table + stride * sub_values(sub["expr"], vars_e, at)
            else:
                iv = ia.index_views[sub["view"]]
                itab = np.broadcast_to(self.at_points(iv.base, ks, trips)[:, None], (n_pts, E)).astype(np.int64)
                for e_, s_ in zip(sub["exprs"], iv.strides):
                    itab = itab + s_ * sub_values(e_, vars_e, at)
                ial = self.alloc_of(itab.min() if itab.size else 0, iv.dtype, "Read from")
                self.indirect_reads.append(ial)
                lookups.append((iv.dtype, np.ascontiguousarray(itab), ial, int(stride)))
        addr = P.emit("table", P.new("i64", (E,)), (), values=np.ascontiguousarray(table))
        for idt, itab, ial, stride in lookups:
            ibpe = bytes_per_elem(idt)
            iaddr = P.emit("table", P.new("i64", (E,)), (), values=itab)
            idx = P.emit("gather", P.new(idt, (E,)), (iaddr,), lo=ial.byte_lo // ibpe, hi=ial.byte_hi // ibpe)
            addr = P.emit("idxadd", P.new("i64", (E,)), (addr, idx), stride=stride)
        return addr

    # -- indirect access tiles: one address per element, through integer steps -------------------
    def indirect_addresses(self, ia: IndirectAccess, ks, trips):
        """Element addresses ``[points, elems]`` (i64 buffer) of an indirect tile, its allocation, dtype.

        Per parent dimension the coordinate is an affine expression of the variable-space point or a
        value looked up in an index view (ktir_cpu/ops/memory_ops.py:488-576); elements are
        enumerated row-major over the (rectangular) variable space.
        """
        from .lower_scatter import _lin
        vars_e = variable_space_points(ia)
        nv, E = vars_e.shape
        P = self.prog
        dt = ia.view.dtype
        try:
            addr = self._indirect_affine(ia, ks, trips, vars_e, nv, E)
        except Unsupported:
            addr = self._indirect_tabulated(ia, ks, trips, vars_e, E)
        al = self.alloc_of(int(np.asarray(ia.view.base).reshape(-1)[0]) if np.asarray(ia.view.base).size else 0,
                           dt, "Read from")
        return addr, al, dt


def variable_space_points(ia: IndirectAccess) -> np.ndarray:
    """The points of an indirect tile's variable space as ``[n_vars, elems]``, in the order its elements
    are enumerated: row-major over the set, re-sorted by ``variables_space_order`` when that permutes
    the variables (ktir_cpu/ops/memory_ops.py:488-520)."""
    box = ia.aset.box()
    if box is not None:
        lo, hi = box
        ext = [h - l for l, h in zip(lo, hi)]
        pts = np.indices(ext, dtype=np.int64).reshape(len(ext), -1) + np.asarray(lo, np.int64)[:, None]
    else:
        lst = ia.aset.enumerate(ia.shape)
        pts = np.asarray(lst, np.int64).reshape(len(lst), len(ia.shape)).T
    if ia.order is not None and not ia.order.is_identity():
        keys = ia.order.eval(list(pts))
        keys = [np.broadcast_to(np.asarray(k_, np.int64), pts.shape[1:]) for k_ in keys]
        pts = pts[:, np.lexsort(tuple(reversed(keys)))]
    return np.ascontiguousarray(pts)


ALL_MEMORY = 1 << 60      # upper bound of a gather / scatter whose addresses the host has already checked


def table_footprints(table: np.ndarray, dtype: str, write: bool, sel, cores, arena, stmt_id: int):
    """Byte runs of a resolved access (one address per point and element, -1 = none), one Footprint
    per allocation touched."""
    from .lower import Footprint
    bpe = bytes_per_elem(dtype)
    P_, E = table.shape
    flat = table.reshape(-1)
    valid = flat >= 0
    if not valid.any():
        return []
    idx = np.flatnonzero(valid)
    a = flat[idx]
    # a run continues while the address grows by one inside the same row
    brk = np.ones(len(idx), bool)
    brk[1:] = (np.diff(a) != 1) | (np.diff(idx) != 1) | (idx[1:] // E != idx[:-1] // E)
    first = np.flatnonzero(brk)
    length = np.diff(np.append(first, len(idx)))
    starts = a[first] * bpe
    ends = starts + length * bpe
    rows = idx[first] // E
    pts = sel[rows] if len(sel) == P_ else np.full(len(rows), -1)
    crs = cores[rows] if len(cores) == P_ else np.full(len(rows), -1)
    out = []
    for al in arena.allocs:
        m = (starts >= al.byte_lo) & (starts < al.byte_hi)
        if m.any():
            out.append(Footprint(starts[m], ends[m], pts[m], crs[m], write, stmt_id))
    return out


def _runs(rel: np.ndarray):
    """Split sorted-as-given element offsets into maximal unit-stride runs: (starts, lengths)."""
    if rel.size == 0:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    brk = np.flatnonzero(np.diff(rel) != 1) + 1
    starts = np.concatenate([[0], brk])
    ends = np.concatenate([brk, [rel.size]])
    return rel[starts], (ends - starts).astype(np.int64)


def _contains_kind(root: Node, kind: str) -> bool:
    seen, stack = set(), [root]
    while stack:
        n = stack.pop()
        if id(n) in seen:
            continue
        seen.add(id(n))
        if n.kind == kind:
            return True
        stack.extend(a for a in n.args if isinstance(a, Node))
        if n.kind == "loopres":
            info = n.attrs["loop"]
            stack.extend(x for x in list(info.inits) + list(info.yields) if isinstance(x, Node))
    return False


def build_generic(store: Store, arena, sel: np.ndarray):
    """(program, written allocation names, direct footprints as (base, rel, dtype, write), indirect allocs)."""
    n_points = _prod(tuple(store.axes))
    ring = _contains_kind(store.value, "ringred")
    store_sel = sel
    if ring and len(sel) != n_points:
        # the cores that do not store still contribute their partials: evaluate everywhere and keep
        # their stores out of the allocation (writes outside are dropped)
        sel = np.arange(n_points, dtype=np.int64)
    gb = GenBuilder(store, arena, sel)
    val = gb.eval(store.value)
    tgt = store.target
    P = gb.prog
    direct = []
    written = []
    if isinstance(tgt, Access):
        dt = tgt.view.dtype
        n_el = _prod(tgt.shape) if tgt.coords is None else len(tgt.coords)
        if val.dtype != dt:
            val = P.emit("ew", P.new(dt, val.shape), (val,), op="mov")
        if val.elems != n_el:
            if val.elems != 1:
                raise ValueError(f"ktdp.store: tile of {val.elems} elements into an access tile of {n_el}")
            val = P.emit("map", P.new(dt, (n_el,)), (val,), shape=(n_el,), strides=[0], offset=0)
        base = gb.at_points(tgt.off, (), ())
        rel = access_rel_offsets(tgt)
        live = base if len(store_sel) == len(sel) else base[store_sel]
        al = gb.alloc_of(live.min() if live.size else 0, dt, "Scatter to")
        bpe = bytes_per_elem(dt)
        if len(store_sel) != len(sel):
            keep = np.zeros(len(sel), bool)
            keep[store_sel] = True
            base = np.where(keep, base, -(1 << 50))
        P.emit("store", None, (val,), base=base, rel=rel, lo=al.byte_lo // bpe, hi=al.byte_hi // bpe, dtype=dt)
        direct.append((live, rel, dt, True, al))
        written.append(al.name)
    elif isinstance(tgt, TableAccess):
        dt = tgt.dtype
        table = gb.table_at_points(tgt.addr, (), ())
        if len(store_sel) != len(sel):
            keep = np.zeros(len(sel), bool)
            keep[store_sel] = True
            table = np.where(keep[:, None], table, -1)
        E = table.shape[1]
        if val.dtype != dt:
            val = P.emit("ew", P.new(dt, val.shape), (val,), op="mov")
        if val.elems != E:
            if val.elems != 1:
                raise ValueError(f"ktdp.store: tile of {val.elems} elements into an access tile of {E}")
            val = P.emit("map", P.new(dt, (E,)), (val,), shape=(E,), strides=[0], offset=0)
        live = table[table >= 0]
        addr = P.emit("table", P.new("i64", (E,)), (), values=table)
        P.emit("scatter", None, (val, addr), lo=0, hi=ALL_MEMORY, dtype=dt,
               any_order=bool(len(np.unique(live)) == len(live)))
        gb.tables.append((table, dt, True))
        bpe = bytes_per_elem(dt)
        written.extend(a_.name for a_ in arena.allocs if ((live * bpe >= a_.byte_lo) & (live * bpe < a_.byte_hi)).any())
    else:
        addr, al, dt = gb.indirect_addresses(tgt, (), ())
        gb.indirect_reads.pop()                       # the parent allocation is written, not read
        E = addr.elems
        if val.dtype != dt:
            val = P.emit("ew", P.new(dt, val.shape), (val,), op="mov")
        if val.elems != E:
            if val.elems != 1:
                raise ValueError(f"indirect_store: source tile of {val.elems} elements does not match IAT of {E}")
            val = P.emit("map", P.new(dt, (E,)), (val,), shape=(E,), strides=[0], offset=0)
        bpe = bytes_per_elem(dt)
        P.emit("scatter", None, (val, addr), lo=al.byte_lo // bpe, hi=al.byte_hi // bpe, dtype=dt)
        written.append(al.name)
    for acc, ks, trips in gb.loads:
        lbase = gb.at_points(acc.off, ks, trips)
        direct.append((lbase, access_rel_offsets(acc), acc.view.dtype, False,
                       gb.alloc_of(lbase.min() if lbase.size else 0, acc.view.dtype, "Read from")))
    P.place()
    ind_write = None if isinstance(tgt, (Access, TableAccess)) else al
    if ind_write is not None and len(sel) > 1:
        # all points are read before any is written: a read-modify-write of the scattered tensor
        # across iteration points would lose the sequential order (the fused row scatter keeps it)
        reads = {a_.name for a_ in gb.indirect_reads}
        for acc, ks, trips in gb.loads:
            reads.add(gb.alloc_of(gb.at_points(acc.off, ks, trips).min(), acc.view.dtype, "Read from").name)
        if ind_write.name in reads:
            raise Unsupported("indirect store into a tensor the same statement reads, in a form the "
                              "ordered row scatter does not cover")
    return P, written, direct, gb.indirect_reads, ind_write, gb.tables


# ---------------------------------------------------------------------------
# The statement: steps bound to device memory
# ---------------------------------------------------------------------------
def _make_statement_class():
    import ctypes as C

    from . import runtime as R
    from .lower import Footprint, Statement, _points

    class GenericStatement(Statement):
        """One ``ktdp.store`` whose value is computed step by step on the device."""
        kind = "generic"

        def __init__(self, dev, store: Store, arena, stmt_id: int):
            sel, cores = _points(store)
            self.prog, written, direct, ind_reads, ind_write, tables = build_generic(store, arena, sel)
            self.extra_written = list(written) if ind_write is not None else []
            self._dev = dev
            self._store_points = sel if self.prog.P == len(sel) else np.arange(self.prog.P)
            self.launches = len(self.prog.ops)
            self.device_arrays: List[int] = []
            self.scratch = dev.alloc(self.prog.scratch_bytes)
            self.device_arrays.append(self.scratch)
            P = self.prog.P
            self.steps: List[R.GenOpArgs] = []
            for op in self.prog.ops:
                g = R.GenOpArgs()
                a = op.attrs
                g.kind = R.G_KINDS[op.kind]
                d = op.dst
                ref = d if d is not None else op.srcs[0]
                g.points, g.elems = P, ref.elems
                if op.kind in ("store", "scatter"):
                    g.elems = len(a["rel"]) if op.kind == "store" else op.srcs[1].elems
                if d is not None:
                    g.dt_dst = R.DTYPE_CODE[d.dtype]
                    g.dst = self.scratch + d.offset
                for slot, b in zip(("a", "b", "c"), op.srcs):
                    setattr(g, slot, self.scratch + b.offset)
                    setattr(g, "dt_" + slot, R.DTYPE_CODE[b.dtype])
                    setattr(g, "e" + slot, b.elems)
                if "base" in a:
                    g.dev_base = self._up(dev, np.ascontiguousarray(a["base"], np.int64))
                    g.dev_rel = self._up(dev, np.ascontiguousarray(a["rel"], np.int64))
                if "lo" in a:
                    g.lo, g.hi = int(a["lo"]), int(a["hi"])
                if op.kind == "constv":
                    g.dev_table = self._up(dev, np.ascontiguousarray(a["table"]))
                elif op.kind == "param":
                    g.dev_table = self._up(dev, np.ascontiguousarray(a["values"]))
                elif op.kind == "table":
                    g.dev_table = self._up(dev, np.ascontiguousarray(a["values"], np.int64))
                elif op.kind == "scatter" and a.get("any_order"):
                    g.flags = 4
                elif op.kind == "fill":
                    v = a["value"]
                    g.fimm = float(v) if d.dtype in ("f16", "f32") else 0.0
                    g.iimm = 0 if d.dtype in ("f16", "f32") else int(v)
                elif op.kind == "idxadd":
                    g.iimm = int(a["stride"])
                elif op.kind == "iota":
                    shape = a["shape"]
                    g.ndim = len(shape)
                    for i_, s_ in enumerate(shape):
                        g.shape[i_] = int(s_)
                    g.offset = int(a["dim"])
                elif op.kind == "map":
                    shape, strides = a["shape"], a["strides"]
                    if len(shape) > R.G_MAXDIM:
                        raise Unsupported(f"tile of rank {len(shape)}")
                    g.ndim = len(shape)
                    for i_, (s_, t_) in enumerate(zip(shape, strides)):
                        g.shape[i_], g.strides[i_] = int(s_), int(t_)
                    g.offset = int(a["offset"])
                elif op.kind in ("ew", "redl"):
                    g.op = EW_CODE[a["op"]]
                    g.flags = 1 if a.get("cmp_int") else 0
                    if op.kind == "redl":
                        g.outer, g.n, g.inner, g.h = int(a["outer"]), int(a["n"]), int(a["inner"]), int(a["h"])
                elif op.kind == "matmul":
                    g.batch, g.M, g.N, g.K = int(a["batch"]), int(a["M"]), int(a["N"]), int(a["K"])
                elif op.kind == "concat":
                    g.outer, g.n, g.h, g.inner = int(a["outer"]), int(a["na"]), int(a["nb"]), int(a["inner"])
                elif op.kind == "ringred":
                    g.op = EW_CODE[a["op"]]
                    g.flags = 2 if a["swapped"] else 0
                    g.n, g.h = int(a["S"]), int(a["cluster"])
                    g.dev_base = self._up(dev, np.ascontiguousarray(a["counts"], np.int64))
                    g.dev_table = self._up(dev, np.ascontiguousarray(a["sources"], np.int64))
                    if a["cluster"]:
                        g.dev_rel = self._up(dev, np.ascontiguousarray(a["order"], np.int64))
                self.steps.append(g)
            # footprints for the sequential-order check
            self.fps: List[Footprint] = []
            neg = np.array([-1])
            for base, rel, dt, write, al in direct:
                bpe = bytes_per_elem(dt)
                rs, rl = _runs(rel)
                starts = (base[:, None] + rs[None, :]).reshape(-1) * bpe
                ends = starts + np.tile(rl, len(base)) * bpe
                if len(base) == len(sel):
                    pts, crs = np.repeat(sel, len(rs)), np.repeat(cores, len(rs))
                else:
                    pts, crs = np.repeat(neg, len(starts)), np.repeat(neg, len(starts))
                # what lies outside the allocation is read as zero / not written: it touches no memory
                starts, ends = np.maximum(starts, al.byte_lo), np.minimum(ends, al.byte_hi)
                real = ends > starts
                if not real.all():
                    starts, ends, pts, crs = starts[real], ends[real], pts[real], crs[real]
                self.fps.append(Footprint(starts, ends, pts, crs, write, stmt_id))
            for table, dt, write in tables:
                self.fps.extend(table_footprints(table, dt, write, sel, cores, arena, stmt_id))
            for al in ind_reads:
                self.fps.append(Footprint(np.array([al.byte_lo]), np.array([al.byte_hi]), neg, neg, False, stmt_id))
            if ind_write is not None:
                self.fps.append(Footprint(np.array([ind_write.byte_lo]), np.array([ind_write.byte_hi]), neg, neg,
                                          True, stmt_id))
            self._bytes = sum(int((f.ends - f.starts).sum()) for f in self.fps)

        def order_points(self, rounds):
            """Several points store to the same bytes: the final store step is repeated once per round,
            each time with only that round's points inside the allocation (the others fall outside
            and are dropped), so the last point in sequential order wins."""
            last = self.steps[-1]
            op = self.prog.ops[-1]
            if op.kind != "store":
                raise Unsupported("several cores scatter to the same bytes through an indirect store")
            base = np.ascontiguousarray(op.attrs["base"], np.int64)
            pts = self._store_points
            per_point = np.array([rounds.get(int(p), 0) for p in pts], np.int64)
            self.steps = self.steps[:-1]
            for r in range(int(per_point.max()) + 1):
                g = R.GenOpArgs.from_buffer_copy(last)
                g.dev_base = self._up(self._dev, np.where(per_point == r, base, -(1 << 50)))
                self.steps.append(g)
            self.launches = len(self.steps)

        def _up(self, dev, arr: np.ndarray) -> int:
            p = dev.upload(arr if arr.size else np.zeros(1, arr.dtype))
            self.device_arrays.append(p)
            return p

        def launch(self, dev, arena_ptr):
            for g in self.steps:
                g.arena = arena_ptr
                dev.check(dev.lib.ktb_launch_generic(dev.h, C.byref(g)))

        def footprints(self):
            return self.fps

        def bytes_moved(self):
            return self._bytes

    return GenericStatement


GenericStatement = None


def generic_statement(dev, store, arena, stmt_id):
    global GenericStatement
    if GenericStatement is None:
        GenericStatement = _make_statement_class()
    return GenericStatement(dev, store, arena, stmt_id)

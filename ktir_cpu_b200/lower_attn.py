"""Lowering of the online-softmax attention loop to the fused attention kernel.

The matcher accepts the loop a KTIR flash-attention kernel carries per KV page
(examples/triton-ktir/paged_attention.mlir:183-396 of the reference, one query
head per KV head): running max ``M``, running sum ``L`` and accumulator ``acc``
as ``iter_args``; per page S = scale * (Q @ K^T), a causal ``select`` against
-inf, m = max(M, rowmax S), P = exp(S - m), alpha = exp(M - m),
acc = acc * alpha + P @ V, L = L * alpha + rowsum P; after the loop
O = acc / L truncated to f16.  K and V pages come through a block table.
Query tiles of all cores are regrouped per head, so the device kernel uses its
own 128-row query blocks whatever tile size the KTIR text used.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem
from .lower import ArenaMap, Footprint, Statement, _points, _row_broadcast, _row_reduce, strip_views
from .lower_mm import _is_zero_const, _unext
from .lower_scatter import row_form
from .trace import Access, IndirectAccess, LoopInfo, Node, Store, Unsupported, iv_bin, iv_full


def _const_value(n: Node) -> Optional[float]:
    n = strip_views(n)
    while n.kind == "bcast":
        n = strip_views(n.args[0])
    if n.kind == "const" and n.attrs.get("list") is None:
        return float(n.attrs["value"])
    return None


def _ew(n: Node, op: str) -> Optional[Node]:
    n = strip_views(n)
    return n if n.kind == "ew" and n.attrs.get("op") == op else None


def _int_affine(n: Node):
    """Integer tile expression -> (row coefficient, column coefficient, per-point constant, row divisor):
    value = (row // divisor) * row coefficient + col * column coefficient + constant.

    The divisor comes from ``arith.divui %row, %c`` on the bare row index: a tile whose rows
    interleave ``c`` query heads per position (notebooks/demo_gen_mlir.py:879-883 of the reference)."""
    n = strip_views(n)
    if n.kind == "cast":
        return _int_affine(n.args[0])
    if n.kind == "iota":
        return (1, 0, 0, 1) if n.attrs["dim"] == 0 else (0, 1, 0, 1)
    if n.kind == "param":
        return (0, 0, n.attrs["values"], 1)
    if n.kind == "const":
        return (0, 0, int(n.attrs["value"]), 1)
    if n.kind == "bcast":
        return _int_affine(n.args[0])
    if n.kind == "ew" and n.attrs["op"] in ("arith.addi", "arith.subi"):
        a, b = _int_affine(n.args[0]), _int_affine(n.args[1])
        s = 1 if n.attrs["op"] == "arith.addi" else -1
        if a[0] and b[0] and a[3] != b[3]:
            raise Unsupported("attention mask mixes row indices with different divisors")
        return (a[0] + s * b[0], a[1] + s * b[1], iv_bin(lambda x, y: x + s * y, a[2], b[2]),
                a[3] if a[0] else b[3])
    if n.kind == "ew" and n.attrs["op"] == "arith.muli":
        a, b = _int_affine(n.args[0]), _int_affine(n.args[1])
        for x, y in ((a, b), (b, a)):
            if x[0] == 0 and x[1] == 0 and isinstance(x[2], (int, np.integer)):
                k = int(x[2])
                return (y[0] * k, y[1] * k, iv_bin(lambda u, v: u * v, y[2], k), y[3])
    if n.kind == "ew" and n.attrs["op"] in ("arith.divui", "arith.divsi", "arith.floordivsi"):
        a, b = _int_affine(n.args[0]), _int_affine(n.args[1])
        if (b[0] == 0 and b[1] == 0 and isinstance(b[2], (int, np.integer)) and int(b[2]) > 0
                and a[0] == 1 and a[1] == 0 and a[3] == 1 and isinstance(a[2], (int, np.integer)) and int(a[2]) == 0):
            return (1, 0, 0, int(b[2]))
    raise Unsupported("attention mask is not an affine comparison of row and column indices")


def match_attention(value: Node):
    root = strip_views(value)
    if not (root.kind == "cast" and root.dtype == "f16" and root.args[0].dtype == "f32"):
        return None
    div = _ew(root.args[0], "arith.divf")
    if div is None:
        return None
    acc_fin = strip_views(div.args[0])
    if acc_fin.kind != "loopres" or len(acc_fin.shape) != 2:
        return None
    l_fin = _row_broadcast(div.args[1], acc_fin.shape)
    if l_fin is None or l_fin.kind != "loopres" or l_fin.attrs["loop"] is not acc_fin.attrs["loop"]:
        return None
    loop: LoopInfo = acc_fin.attrs["loop"]
    if len(loop.yields) != 3:
        return None
    ia, il = acc_fin.attrs["index"], l_fin.attrs["index"]
    im = ({0, 1, 2} - {ia, il}).pop()

    def is_iter(n, k):
        n = strip_views(n)
        return n.kind == "iter" and n.attrs.get("loop") is loop and n.attrs["index"] == k

    m_new, l_new, acc_new = (strip_views(loop.yields[k]) for k in (im, il, ia))
    if acc_new.kind != "matmul" or len(acc_new.args) != 3:
        return None
    # m_new = max(M, rowmax(masked))
    if not (m_new.kind == "ew" and m_new.attrs["op"] in ("arith.maximumf", "arith.maxnumf")):
        return None
    rmax = m_new.args[1] if is_iter(m_new.args[0], im) else (m_new.args[0] if is_iter(m_new.args[1], im) else None)
    if rmax is None:
        return None
    rr = _row_reduce(rmax, ("arith.maximumf", "arith.maxnumf"))
    if rr is None:
        return None
    masked = strip_views(rr[0])
    causal, cond, sc = False, None, masked
    sel = _ew(masked, "arith.select")
    if sel is not None:
        if _const_value(sel.args[2]) != float("-inf"):
            return None
        causal, cond, sc = True, strip_views(sel.args[0]), strip_views(sel.args[1])
    scale = 1.0
    mul = _ew(sc, "arith.mulf")
    qk = sc
    if mul is not None:
        c0, c1 = _const_value(mul.args[0]), _const_value(mul.args[1])
        if c0 is not None:
            scale, qk = c0, strip_views(mul.args[1])
        elif c1 is not None:
            scale, qk = c1, strip_views(mul.args[0])
        else:
            return None
    if qk.kind != "matmul" or not _is_zero_const(qk.args[2] if len(qk.args) > 2 else None):
        return None
    q = _unext(qk.args[0])
    kt = _unext(qk.args[1])
    if q.kind != "load" or kt.kind != "transpose" or tuple(kt.attrs["perm"]) != (1, 0):
        return None
    k = strip_views(kt.args[0])
    # P = exp(masked - m_new), V, acc * alpha
    p = _ew(acc_new.args[0], "math.exp")
    if p is None:
        return None
    sub = _ew(p.args[0], "arith.subf")
    if sub is None or strip_views(sub.args[0]) is not masked or _row_broadcast(sub.args[1], masked.shape) is not m_new:
        return None
    v = _unext(acc_new.args[1])
    scaled = _ew(acc_new.args[2], "arith.mulf")
    if scaled is None or not is_iter(scaled.args[0], ia):
        return None
    alpha = _row_broadcast(scaled.args[1], acc_new.shape)
    if alpha is None:
        return None
    aexp = _ew(alpha, "math.exp")
    asub = _ew(aexp.args[0], "arith.subf") if aexp is not None else None
    if asub is None or not is_iter(asub.args[0], im) or strip_views(asub.args[1]) is not m_new:
        return None
    # L = L * alpha + rowsum(P)
    ladd = _ew(l_new, "arith.addf")
    if ladd is None:
        return None
    lmul = _ew(ladd.args[0], "arith.mulf")
    lr = _row_reduce(ladd.args[1], ("arith.addf",))
    if lmul is None or lr is None or strip_views(lr[0]) is not p:
        return None
    if not is_iter(lmul.args[0], il) or strip_views(lmul.args[1]) is not alpha:
        return None
    m_init, l_init, acc_init = (_const_value(loop.inits[i]) for i in (im, il, ia))
    if m_init is None or l_init is None or acc_init != 0.0:
        return None
    if k.kind not in ("iload",) or v.kind not in ("iload",):
        return None
    return dict(loop=loop, q=q.attrs["access"], k=k.attrs["access"], v=v.attrs["access"], scale=scale,
                causal=causal, cond=cond, m_init=m_init, l_init=l_init, tile=masked.shape)


class AttentionStatement(Statement):
    kind = "attention_fwd"

    def __init__(self, dev: R.Device, store: Store, m: dict, arena: ArenaMap, stmt_id: int):
        loop: LoopInfo = m["loop"]
        T = loop.trips
        Q: Access = m["q"]
        O: Access = store.target
        Kc: IndirectAccess = m["k"]
        Vc: IndirectAccess = m["v"]
        tm, tn = m["tile"]
        sel, _ = _points(store)
        P = len(sel)
        for acc in (Q, O):
            if acc.coords is not None or len(acc.shape) != 3 or acc.strides[2] != 1:
                raise Unsupported("attention query/output tile must be [rows, heads, head_dim] of a [seq, heads, dim] view")
        # a tile holds bq query positions x grp query heads that share one K/V head; its rows are
        # position-major (tensor.collapse_shape [[0, 1], [2]]): tile row r = position r // grp, head r % grp
        bq, grp, hd = Q.shape
        if hd != 128 or tuple(O.shape) != tuple(Q.shape) or bq * grp != tm:
            raise Unsupported("attention kernel supports head_dim 128 with matching query/output tiles")
        if Q.view.dtype != "f16" or O.view.dtype != "f16" or Kc.view.dtype != "f16" or Vc.view.dtype != "f16":
            raise Unsupported("attention operands must be f16")
        ext = tuple(store.axes) + (T,)

        def decode(acc: Access, offs):
            rel = offs - int(np.asarray(acc.view.base).reshape(-1)[0])
            row0, rem = np.divmod(rel, acc.strides[0])
            head, rem2 = np.divmod(rem, acc.strides[1])
            if rem2.any():
                raise Unsupported("attention query/output tile not aligned to a head")
            return row0, head

        q_off = np.ascontiguousarray(iv_full(Q.off, store.axes).reshape(-1)[sel])
        o_off = np.ascontiguousarray(iv_full(O.off, store.axes).reshape(-1)[sel])
        if np.asarray(Q.view.base).size != 1 or np.asarray(O.view.base).size != 1:
            raise Unsupported("per-core query/output base pointers")
        row0, head = decode(Q, q_off)
        orow0, ohead = decode(O, o_off)
        if (row0 != orow0).any() or (head != ohead).any() or ((row0 - row0.min()) % bq).any() or (head % grp).any():
            raise Unsupported("attention output tiles do not mirror the query tiles")
        # the statement may cover a sub-range of the heads (a core slice of a sharded kernel)
        hmin = int(head.min())
        hgrp = (head - hmin) // grp                  # K/V head of the tile, relative to the first one
        ngrp = int(hgrp.max()) + 1
        heads = ngrp * grp
        rmin = int(row0.min())
        nblk = int((row0.max() - rmin) // bq) + 1
        key = ((row0 - rmin) // bq) * ngrp + hgrp
        if P != nblk * ngrp or len(np.unique(key)) != P:
            raise Unsupported("attention query tiles do not cover [rows x heads] exactly once")
        seq_q = nblk * bq

        # K / V pages: one block-table entry per loop trip, rows and head_dim direct
        flat = np.arange(int(np.prod(ext)), dtype=np.int64).reshape(-1, T)[sel].reshape(-1)
        forms = []
        for acc in (Kc, Vc):
            f = row_form(acc, ext, flat)
            if (f.rows, f.cols) != (tn, hd) or f.idx_stride != 0:
                raise Unsupported("attention K/V tile must be one [page_rows, head_dim] page per block-table entry")
            forms.append(f)
        kf, vf = forms
        if (kf.idx_dtype, kf.idx_mult, kf.pos_stride) != (vf.idx_dtype, vf.idx_mult, vf.pos_stride) or \
                not np.array_equal(kf.idx_off, vf.idx_off):
            raise Unsupported("K and V caches must share geometry and block table")
        idx = kf.idx_off.reshape(P, T)
        if (idx != idx[0:1, 0:1] + np.arange(T)[None, :]).any():
            raise Unsupported("attention loop must walk consecutive block-table entries, the same for every core")
        kview, vview = Kc.view, Vc.view
        if len(kview.shape) != 4 or kview.shape[1] != tn or tuple(kview.strides) != tuple(vview.strides) or \
                kview.strides[3] != 1:
            raise Unsupported("K/V cache must be [pages, page_rows, heads, head_dim]")
        kbase, vbase = (int(np.asarray(x.base).reshape(-1)[0]) for x in (kview, vview))
        for f, base in ((kf, kbase), (vf, vbase)):
            hh, rem = np.divmod(f.base.reshape(P, T) - base, kview.strides[2])
            if rem.any() or (hh != (hgrp + hmin // grp)[:, None]).any():
                raise Unsupported("K/V head does not follow the query head")

        delta = 0
        if m["causal"]:
            cond = m["cond"]
            if cond.kind != "ew" or cond.attrs.get("op") != "arith.cmpi" or cond.attrs.get("pred") not in ("ule", "sle"):
                raise Unsupported("attention mask must be `kv position <= query position`")
            kr, kc, kconst, _ = _int_affine(cond.args[0])
            qr, qc, qconst, qdiv = _int_affine(cond.args[1])
            if (kr, kc, qr, qc) != (0, 1, 1, 0) or qdiv != grp:
                raise Unsupported("attention mask must compare a column index with the query position of a row")
            kfull = iv_full(kconst, ext).reshape(-1, T)[sel] - np.arange(T)[None, :] * tn
            qfull = iv_full(qconst, ext).reshape(-1, T)[sel] - row0[:, None]
            d = qfull - kfull
            if (d != d.flat[0]).any():
                raise Unsupported("attention mask offset differs between cores or pages")
            delta = int(d.flat[0]) + rmin
            if delta < 0:
                raise Unsupported("attention rows that see no KV position")
        arena.check_range(int(q_off.min()), int(q_off.max()) + (bq - 1) * Q.strides[0] + (grp - 1) * Q.strides[1] + hd,
                          "f16", "Read from")
        arena.check_range(int(o_off.min()), int(o_off.max()) + (bq - 1) * O.strides[0] + (grp - 1) * O.strides[1] + hd,
                          "f16", "Scatter to")
        kalloc = arena.check_range(kbase, kbase + 1, "f16", "Read from")
        valloc = arena.check_range(vbase, vbase + 1, "f16", "Read from")
        bt_alloc = arena.check_range(int(idx.min()), int(idx.max()) + 1, kf.idx_dtype, "Read from")
        n_pages = int(kview.shape[0])

        self.args = a = R.AttnArgs()
        a.q_off = int(np.asarray(Q.view.base).reshape(-1)[0]) + rmin * Q.strides[0] + hmin * Q.strides[1]
        a.o_off = int(np.asarray(O.view.base).reshape(-1)[0]) + rmin * O.strides[0] + hmin * O.strides[1]
        a.k_off, a.v_off = kbase + (hmin // grp) * kview.strides[2], vbase + (hmin // grp) * kview.strides[2]
        a.kv_group = grp
        a.bt_off, a.bt_dtype = int(idx[0, 0]), R.DTYPE_CODE[kf.idx_dtype]
        a.seq_q, a.heads, a.head_dim = seq_q, heads, hd
        a.page, a.n_pages_total, a.num_tiles = tn, n_pages, T
        a.causal, a.causal_delta = int(m["causal"]), delta
        a.q_row_stride, a.q_head_stride = Q.strides[0], Q.strides[1]
        a.o_row_stride, a.o_head_stride = O.strides[0], O.strides[1]
        a.kv_page_stride, a.kv_row_stride, a.kv_head_stride = kview.strides[0], kview.strides[1], kview.strides[2]
        a.scale, a.m_init, a.l_init = m["scale"], m["m_init"], m["l_init"]
        self.device_arrays = []
        vis = np.minimum(T * tn, np.arange(seq_q) + 1 + delta) if m["causal"] else np.full(seq_q, T * tn)
        self.flops = int(4 * heads * hd * vis.sum())
        self._bytes = hd * 2 * (2 * heads * seq_q + 2 * ngrp * min(T, n_pages) * tn)
        neg = np.array([-1])
        rows = (np.arange(seq_q, dtype=np.int64)[:, None] * 1)
        qs = ((a.q_off + rows * Q.strides[0] + np.arange(heads)[None, :] * Q.strides[1]) * 2).reshape(-1)
        os_ = ((a.o_off + rows * O.strides[0] + np.arange(heads)[None, :] * O.strides[1]) * 2).reshape(-1)
        nr = len(qs)
        self.fps = [Footprint(qs, qs + hd * 2, np.repeat(neg, nr), np.repeat(neg, nr), False, stmt_id),
                    Footprint(os_, os_ + hd * 2, np.repeat(neg, nr), np.repeat(neg, nr), True, stmt_id)]
        for al in (kalloc, valloc, bt_alloc):
            self.fps.append(Footprint(np.array([al.byte_lo]), np.array([al.byte_hi]), neg, neg, False, stmt_id))

    def launch(self, dev, arena_ptr):
        self.args.arena = arena_ptr
        dev.check(dev.lib.ktb_launch_attention_fwd(dev.h, C.byref(self.args)))

    def split(self, piece_bytes: int):
        """Groups of heads (whole K/V heads): a group reads its columns of Q, K and V — ``seq`` rows of
        ``heads x head_dim`` elements each, one strided region per tensor — and the block table."""
        from .lower import _copy_args
        from .pipeline import Chunk, Region, chunk_count
        a = self.args
        grp = max(a.kv_group, 1)
        hd = a.head_dim
        kv_rows = a.n_pages_total * a.page
        if (a.q_head_stride != hd or a.o_head_stride != hd or a.kv_head_stride != hd
                or a.kv_page_stride != a.page * a.kv_row_stride):
            return None
        n = chunk_count(self._bytes, a.heads // grp, piece_bytes)
        bt_bpe = 4 if a.bt_dtype == R.KTB_I32 else 8
        bt = Region(a.bt_off * bt_bpe, a.num_tiles * bt_bpe)
        bounds = np.linspace(0, a.heads // grp, n + 1).astype(np.int64)
        chunks = []
        for g0, g1 in zip(bounds[:-1], bounds[1:]):
            g0, g1 = int(g0), int(g1)
            if g0 == g1:
                continue
            h0, nh = g0 * grp, (g1 - g0) * grp
            sub = _copy_args(a)
            sub.q_off, sub.o_off = a.q_off + h0 * hd, a.o_off + h0 * hd
            sub.k_off, sub.v_off = a.k_off + g0 * hd, a.v_off + g0 * hd
            sub.heads = nh
            q = Region(sub.q_off * 2, nh * hd * 2, a.seq_q, a.q_row_stride * 2)
            o = Region(sub.o_off * 2, nh * hd * 2, a.seq_q, a.o_row_stride * 2)
            k = Region(sub.k_off * 2, (g1 - g0) * hd * 2, kv_rows, a.kv_row_stride * 2)
            v = Region(sub.v_off * 2, (g1 - g0) * hd * 2, kv_rows, a.kv_row_stride * 2)
            chunks.append(Chunk(("ktb_launch_attention_fwd", sub), [bt, q, k, v], [o]))
        return chunks

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


def try_lower_attention(dev, store, arena, stmt_id):
    m = match_attention(store.value)
    if m is None:
        return None
    return AttentionStatement(dev, store, m, arena, stmt_id)

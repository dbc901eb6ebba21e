"""Lowering of K-loops around ``linalg.matmul`` to the tensor-core GEMM.

A KTIR tiled matmul keeps one bm x bn accumulator per (core, tile) and walks K
in steps of bk: per step it loads an A tile and a B tile, multiplies and
accumulates (examples/triton-ktir/matmul_fwd_ktir.mlir:33-58 of the reference).
When the tiles of all cores and outer-loop iterations form a dense grid over
row-major A[M,K], B[K,N], C[M,N], the whole statement is one GEMM and is
re-tiled for tcgen05 (128 x 256 CTA tiles) instead of being run tile by tile.

Numerics: the GEMM accumulates all of K in f32 and rounds once.  For kernels
that carry an f32 accumulator this is the reference's arithmetic up to summation
order; for the f16 form (f16 matmul per K-step added into an f16 accumulator)
the reference rounds at every K-step, so results agree to the f16 tolerance of
the matmul tests (rtol 2e-2, atol 2e-1), not bit for bit.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import runtime as R
from .dtypes import bytes_per_elem
from .lower import ArenaMap, Footprint, Statement, _points, strip_views
from .trace import Access, LoopInfo, Node, Store, Unsupported, iv_full


def _unext(n: Node) -> Node:
    n = strip_views(n)
    if n.kind == "cast" and n.dtype == "f32" and n.args[0].dtype == "f16":
        n = strip_views(n.args[0])
    return n


def _is_zero_const(n: Optional[Node]) -> bool:
    if n is None:
        return True
    n = strip_views(n)
    while n.kind == "bcast":
        n = strip_views(n.args[0])
    return n.kind == "const" and n.attrs.get("list") is None and float(n.attrs["value"]) == 0.0


def match_matmul_loop(value: Node):
    v = strip_views(value)
    if v.kind == "cast" and v.dtype == "f16" and v.args[0].dtype == "f32":
        v = strip_views(v.args[0])
    if v.kind != "loopres":
        return None
    loop: LoopInfo = v.attrs["loop"]
    if len(loop.yields) != 1:
        return None
    y = strip_views(loop.yields[0])

    def is_iter(n):
        n = strip_views(n)
        return n.kind == "iter" and n.attrs.get("loop") is loop

    mm = None
    if y.kind == "matmul" and len(y.args) == 3 and is_iter(y.args[2]):
        mm = y
    elif y.kind == "ew" and y.attrs["op"] == "arith.addf" and len(y.args) == 2:
        for p, q in ((0, 1), (1, 0)):
            cand = strip_views(y.args[q])
            if is_iter(y.args[p]) and cand.kind == "matmul" and _is_zero_const(cand.args[2] if len(cand.args) > 2 else None):
                mm = cand
    if mm is None or mm.attrs.get("batched"):
        return None
    a, b = _unext(mm.args[0]), _unext(mm.args[1])
    if a.kind != "load" or b.kind != "load" or a.dtype != "f16" or b.dtype != "f16":
        return None
    init = strip_views(loop.inits[0])
    while init.kind == "bcast":
        init = strip_views(init.args[0])
    if init.kind != "const" or init.attrs.get("list") is not None:
        return None
    return dict(loop=loop, a=a.attrs["access"], b=b.attrs["access"], c_init=float(init.attrs["value"]))


class GemmStatement(Statement):
    kind = "gemm_f16"

    def __init__(self, dev: R.Device, store: Store, m: dict, arena: ArenaMap, stmt_id: int):
        loop: LoopInfo = m["loop"]
        A: Access = m["a"]
        B: Access = m["b"]
        Cc: Access = store.target
        T = loop.trips
        for acc in (A, B, Cc):
            if acc.coords is not None or len(acc.shape) != 2 or acc.strides[1] != 1:
                raise Unsupported("matmul operand tile that is not a row-major 2-D box")
        bm, bk = A.shape
        bk2, bn = B.shape
        if bk2 != bk or tuple(Cc.shape) != (bm, bn):
            raise Unsupported("matmul tile shapes do not agree")
        lda, ldb, ldc = A.strides[0], B.strides[0], Cc.strides[0]
        sel, _ = _points(store)
        ext = tuple(store.axes) + (T,)
        a_off = iv_full(A.off, ext).reshape(-1, T)[sel]
        b_off = iv_full(B.off, ext).reshape(-1, T)[sel]
        c_off = np.ascontiguousarray(iv_full(Cc.off, store.axes).reshape(-1)[sel])
        if T > 1:
            if (np.diff(a_off, axis=1) != bk).any() or (np.diff(b_off, axis=1) != bk * ldb).any():
                raise Unsupported("matmul K-loop whose tiles do not advance contiguously along K")
        a0, b0 = a_off[:, 0], b_off[:, 0]
        amin, bmin, cmin = int(a0.min()), int(b0.min()), int(c_off.min())
        ri, rr = np.divmod(a0 - amin, bm * lda)
        cj, cr = np.divmod(b0 - bmin, bn)
        if rr.any() or cr.any():
            raise Unsupported("matmul tiles are not aligned to a tile grid")
        Mi, Nj = int(ri.max()) + 1, int(cj.max()) + 1
        key = ri * Nj + cj
        if len(key) != Mi * Nj or len(np.unique(key)) != Mi * Nj:
            raise Unsupported("matmul tiles do not cover a dense grid exactly once")
        if (c_off != cmin + ri * bm * ldc + cj * bn).any():
            raise Unsupported("matmul output tiles do not follow the operand tile grid")
        M, N, K = Mi * bm, Nj * bn, T * bk
        if N > ldb or N > ldc or K > lda:
            raise Unsupported("matmul tile grid wider than the operand rows")
        arena.check_range(amin, amin + (M - 1) * lda + K, "f16", "Read from")
        arena.check_range(bmin, bmin + (K - 1) * ldb + N, "f16", "Read from")
        arena.check_range(cmin, cmin + (M - 1) * ldc + N, Cc.view.dtype, "Scatter to")
        if A.view.dtype != "f16" or B.view.dtype != "f16" or Cc.view.dtype not in ("f16", "f32"):
            raise Unsupported("matmul operand dtypes")
        if N % 32 or K % 8 or lda % 8 or ldb % 8 or ldc % 8 or amin % 8 or bmin % 8 or cmin % 8:
            raise Unsupported("GEMM needs N % 32 == 0 and 16-byte aligned operand rows")
        self.args = a = R.GemmArgs()
        a.a_off, a.b_off, a.c_off = amin, bmin, cmin
        a.M, a.N, a.K = M, N, K
        a.lda, a.ldb, a.ldc = lda, ldb, ldc
        a.c_dtype = R.DTYPE_CODE[Cc.view.dtype]
        a.c_init = m["c_init"]
        self.device_arrays = []
        self.flops = 2 * M * N * K
        cb = bytes_per_elem(Cc.view.dtype)
        self._bytes = (M * K + K * N) * 2 + M * N * cb
        neg = np.array([-1])

        def rows(off, n, ld, width, bpe, write):
            s = (off + np.arange(n, dtype=np.int64) * ld) * bpe
            return Footprint(s, s + width * bpe, np.repeat(neg, n), np.repeat(neg, n), write, stmt_id)

        self.fps = [rows(amin, M, lda, K, 2, False), rows(bmin, K, ldb, N, 2, False),
                    rows(cmin, M, ldc, N, cb, True)]

    def launch(self, dev, arena_ptr):
        self.args.arena = arena_ptr
        dev.check(dev.lib.ktb_launch_gemm_f16(dev.h, C.byref(self.args)))

    def split(self, piece_bytes: int):
        """Row blocks of C: block [m0, m1) needs the same rows of A and all of B."""
        from .lower import _copy_args
        from .pipeline import Chunk, Region, chunk_count
        a = self.args
        cb = 2 if a.c_dtype == R.KTB_F16 else 4
        blocks = (a.M + 127) // 128                      # the kernel works in 128-row tiles
        n = chunk_count(a.M * a.K * 2 + a.M * a.N * cb, blocks, piece_bytes)

        def rows(off, r0, r1, ld, width, bpe):
            if ld == width:
                return Region((off + r0 * ld) * bpe, (r1 - r0) * width * bpe)
            return Region((off + r0 * ld) * bpe, width * bpe, r1 - r0, ld * bpe)
        b_reg = rows(a.b_off, 0, a.K, a.ldb, a.N, 2)
        bounds = np.linspace(0, blocks, n + 1).astype(np.int64) * 128
        chunks = []
        for m0, m1 in zip(bounds[:-1], bounds[1:]):
            m0, m1 = int(m0), int(min(m1, a.M))
            if m0 >= m1:
                continue
            sub = _copy_args(a)
            sub.a_off, sub.c_off, sub.M = a.a_off + m0 * a.lda, a.c_off + m0 * a.ldc, m1 - m0
            chunks.append(Chunk(("ktb_launch_gemm_f16", sub), [b_reg, rows(a.a_off, m0, m1, a.lda, a.K, 2)], [rows(a.c_off, m0, m1, a.ldc, a.N, cb)]))
        return chunks

    def footprints(self):
        return self.fps

    def bytes_moved(self):
        return self._bytes


def try_lower_matmul(dev, store, arena, stmt_id):
    m = match_matmul_loop(store.value)
    if m is None:
        return None
    return GemmStatement(dev, store, m, arena, stmt_id)

"""Chunked, overlapped execution of a launch plan: upload of chunk i+1, kernels of chunk i and
read-back of chunk i-1 run at the same time on three streams.

``KTIRInterpreter.execute_function`` of the reference copies every ndarray argument into its
simulated memory, runs, and reads every one back into a new array
(ktir_cpu/interpreter.py:156-194).  Here each ndarray argument gets one page-locked result array;
host threads copy the caller's data into it piece by piece and every piece is sent on to the
device from there (``ktb_run_pipeline``), so a single host copy yields both the upload and the fresh
array the caller receives, for page-locked and ordinary caller arrays alike.  Tensors the plan
writes are read back into the same result arrays, region by region, as soon as the chunk that
produced them has run.

A statement that can run in independent parts says so through ``Statement.split``: each part
(:class:`Chunk`) names the arena regions it reads and writes.  Plans that cannot be split run as
one chunk over whole tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class Region:
    """``height`` rows of ``width`` bytes, ``pitch`` bytes apart, first byte at arena offset ``off``."""
    off: int
    width: int
    height: int = 1
    pitch: int = 0

    @property
    def nbytes(self) -> int:
        return self.width * self.height

    @property
    def end(self) -> int:
        return self.off + (self.height - 1) * (self.pitch or self.width) + self.width


@dataclass
class Chunk:
    launch: Optional[Tuple[str, object]]   # (name of a ktb_launch_* entry point, its argument struct) or None
    reads: List[Region]
    writes: List[Region]
    uploads: List[Region] = field(default_factory=list)     # reads no earlier chunk has brought in


def merge_intervals(starts: np.ndarray, ends: np.ndarray) -> List[Tuple[int, int]]:
    if len(starts) == 0:
        return []
    order = np.argsort(starts, kind="stable")
    s, e = np.asarray(starts)[order], np.asarray(ends)[order]
    hi = np.maximum.accumulate(e)
    new = np.ones(len(s), bool)
    new[1:] = s[1:] > hi[:-1]
    first = np.flatnonzero(new)
    last = np.concatenate([first[1:] - 1, [len(s) - 1]])
    return [(int(s[a]), int(hi[b])) for a, b in zip(first, last)]


def tile_regions(offs: np.ndarray, rows: int, row_stride: int, cols: int, bpe: int, limit: int = 32) -> Optional[List[Region]]:
    """Regions covering tiles of ``rows`` x ``cols`` elements at element offsets ``offs``; None when
    they do not merge into at most ``limit`` contiguous runs."""
    offs = np.asarray(offs, np.int64)
    if rows == 1 or row_stride == cols:
        st = offs * bpe
        runs = merge_intervals(st, st + rows * cols * bpe)
    else:
        if len(offs) * rows > 1 << 20:
            return None
        st = ((offs[:, None] + np.arange(rows, dtype=np.int64)[None, :] * row_stride) * bpe).reshape(-1)
        runs = merge_intervals(st, st + cols * bpe)
    if len(runs) > limit:
        return None
    return [Region(a, b - a) for a, b in runs]


class _Covered:
    """Bytes already uploaded: exact 2-D regions plus merged 1-D intervals."""

    def __init__(self):
        self.runs: List[Tuple[int, int]] = []
        self.boxes = set()

    def missing(self, r: Region) -> List[Region]:
        if r.height > 1:
            if r in self.boxes or any(a <= r.off and r.end <= b for a, b in self.runs):
                return []
            self.boxes.add(r)
            return [r]
        out, pos = [], r.off
        for a, b in self.runs:
            if b <= pos:
                continue
            if a >= r.end:
                break
            if a > pos:
                out.append(Region(pos, a - pos))
            pos = max(pos, b)
        if pos < r.end:
            out.append(Region(pos, r.end - pos))
        if out:
            self.runs = merge_intervals(np.array([a for a, _ in self.runs] + [r.off]),
                                        np.array([b for _, b in self.runs] + [r.end]))
        return out


class TransferPlan:
    """What ``execute_function`` moves, and when, for one session.

    ``tensors``: name -> (arena offset, nbytes).  ``no_upload``: fully overwritten, never read.
    ``chunks``: the plan's parts, or None for a plan that runs as a whole.  ``written_ranges``:
    merged arena byte ranges the plan writes (read back instead of whole tensors when they are few).
    ``partial``: a rank's share of a kernel split over several GPUs — only what this rank's cores
    read is staged and only what they wrote is read back, so the result arrays are complete
    only inside this rank's slabs."""

    def __init__(self, tensors: Dict[str, Tuple[int, int]], written: Sequence[str], no_upload: Sequence[str],
                 chunks: Optional[List[Chunk]], written_ranges: Optional[Sequence[Tuple[int, int]]] = None,
                 partial: bool = False):
        self.tensors = dict(tensors)
        self.no_upload = set(no_upload)
        self.written = set(written)
        self.partial = partial
        names = sorted(self.tensors, key=lambda k: self.tensors[k][0])
        self._starts = np.array([self.tensors[k][0] for k in names], np.int64)
        self._names = names
        staged = [k for k in names if k not in self.no_upload and self.tensors[k][1] > 0]
        if chunks:
            chunks = self._complete(chunks, staged)
        if not chunks:
            whole_r = [Region(*self.tensors[k]) for k in staged]
            whole_w = [Region(*self.tensors[k]) for k in names if k in self.written and self.tensors[k][1] > 0]
            if written_ranges is not None and 0 < len(written_ranges) <= 64:
                try:
                    ranges = [Region(lo, hi - lo) for lo, hi in written_ranges]
                    for r in ranges:
                        self.owner(r)
                    whole_w = ranges
                except ValueError:
                    pass
            chunks = [Chunk(None, whole_r, whole_w, list(whole_r))]
            self.split = False
        else:
            self.split = True
        self.chunks = chunks
        up = {k: 0 for k in names}
        for c in chunks:
            for r in c.uploads:
                up[self.owner(r)] += r.nbytes
        # inputs no chunk reads: the caller still gets a copy back, the device does not need them
        self.host_only = [] if partial else [k for k in staged if up[k] == 0]
        self.h2d_bytes = sum(up.values())
        self.d2h_bytes = sum(r.nbytes for c in chunks for r in c.writes)

    def owner(self, r: Region) -> str:
        i = int(np.searchsorted(self._starts, r.off, side="right")) - 1
        name = self._names[max(i, 0)]
        off, nb = self.tensors[name]
        if not (off <= r.off and r.end <= off + nb):
            raise ValueError(f"transfer region [{r.off}, {r.end}) is not inside one tensor")
        return name

    def _complete(self, chunks: List[Chunk], staged: List[str]) -> Optional[List[Chunk]]:
        """Fill in ``uploads``; a tensor whose regions do not add up to all of it is uploaded whole
        ahead of the first chunk instead (the caller's copy must be complete either way)."""
        cov = _Covered()
        per = {k: 0 for k in self.tensors}
        try:
            for c in chunks:
                c.uploads = []
                for r in c.reads:
                    if self.owner(r) in self.no_upload:
                        continue
                    for m in cov.missing(r):
                        c.uploads.append(m)
                        per[self.owner(m)] += m.nbytes
                for r in c.writes:
                    self.owner(r)
        except ValueError:
            return None
        partial = [] if self.partial else [k for k in staged if 0 < per[k] != self.tensors[k][1]]
        if partial:
            for c in chunks:
                c.uploads = [r for r in c.uploads if self.owner(r) not in partial]
            chunks[0].uploads = [Region(*self.tensors[k]) for k in partial] + chunks[0].uploads
        # a written tensor must be read back completely unless the rest of it reaches the caller
        # through the staged copy: that holds for everything staged; unstaged (no_upload) tensors
        # are fully overwritten by definition
        return chunks


def chunk_count(total_bytes: int, units: int, piece: int = 8 << 20, most: int = 32) -> int:
    """How many parts to run ``units`` independent units in, for ``total_bytes`` of transfers."""
    n = int(min(most, units, max(1, total_bytes // piece)))
    return max(n, 1)


class BoundPipeline:
    """A :class:`TransferPlan` as the argument arrays of ``ktb_run_pipeline`` for one device arena."""

    def __init__(self, dev, arena: int, tp: TransferPlan):
        import ctypes as C

        from . import runtime as R
        self.tp = tp
        self.names = list(tp.tensors)
        index = {k: i for i, k in enumerate(self.names)}
        self._keep = []

        def regions(rs: Sequence[Tuple[Region, bool]]):
            arr = (R.PipeRegion * max(len(rs), 1))()
            for i, (r, on_device) in enumerate(rs):
                k = tp.owner(r)
                arr[i] = R.PipeRegion(index[k], 0, r.off if on_device else R.NO_DEVICE, r.off - tp.tensors[k][0],
                                      r.width, r.height, r.pitch or r.width)
            self._keep.append(arr)
            return arr

        n = len(tp.chunks)
        self.chunks = (R.PipeChunk * n)()
        self.n_chunks = n
        for i, c in enumerate(tp.chunks):
            # tensors the device never reads are copied for the caller only, ahead of everything else
            up = [(Region(*tp.tensors[k]), False) for k in tp.host_only] if i == 0 else []
            up += [(r, True) for r in c.uploads]
            down = [(r, True) for r in c.writes] if tp.split else []
            ch = self.chunks[i]
            if tp.split and c.launch is not None:
                name, args = c.launch
                args.arena = arena
                self._keep.append(args)
                ch.launch = C.cast(getattr(dev.lib, name), C.c_void_p).value
                ch.launch_args = C.addressof(args)
            ch.n_up, ch.n_down = len(up), len(down)
            ch.up, ch.down = regions(up), regions(down)
        self.ptr_t = C.c_void_p * len(self.names)

    def submit(self, dev, arena: int, host: Dict[str, np.ndarray], results: Dict[str, np.ndarray],
               snapshot_ptr: int, event_slot: int) -> int:
        """Hand the call (a plan whose parts launch through the C ABI) to the context's submission thread;
        returns the job's sequence number.  The arrays must stay alive until the job's event has completed."""
        assert self.tp.split
        pinned = self.ptr_t(*[results[k].ctypes.data for k in self.names])
        src = self.ptr_t(*[host[k].ctypes.data for k in self.names])
        return dev.submit_pipeline(arena, self.chunks, self.n_chunks, pinned, src, len(self.names), snapshot_ptr, event_slot)

    def run(self, dev, arena: int, host: Dict[str, np.ndarray], results: Dict[str, np.ndarray], whole_launch,
            after_launch=None):
        """Queue the whole call; the caller synchronises afterwards.  ``after_launch`` (plans that run
        as a whole only) is called between the launches and the read-back."""
        pinned = self.ptr_t(*[results[k].ctypes.data for k in self.names])
        src = self.ptr_t(*[host[k].ctypes.data for k in self.names])
        dev.run_pipeline(arena, self.chunks, self.n_chunks, pinned, src, len(self.names))
        if not self.tp.split:
            # a plan that runs as a whole: its launches (or their graph replay) go out from here,
            # then every written tensor comes back
            whole_launch()
            if after_launch is not None:
                after_launch()
            writes = self.tp.chunks[0].writes
            if writes:
                dev.fence(0, 2)
                for r in writes:
                    k = self.tp.owner(r)
                    dev.lane_d2h(results[k].ctypes.data + (r.off - self.tp.tensors[k][0]), arena + r.off,
                                 r.width, r.height, r.pitch)

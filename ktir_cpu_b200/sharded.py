"""One KTIR kernel split over several GPUs (one process per GPU).

The grid cores of the kernels this backend runs are independent, so rank ``r`` of ``world``
traces and launches only the cores ``[r*C/world, (r+1)*C/world)``.  Each rank then holds a
correct copy of the bytes its cores wrote ("slabs"); ``exchange`` broadcasts every rank's slabs
so that all ranks end with the complete result — the only collective on the data path.

An ordered indirect store is the exception: cores write overlapping destination rows and the
reference applies them core after core (ktir_cpu/grid.py:595-613, ktir_cpu/memory.py:281-291).
There every rank walks all cores' tiles but applies, in the global (tile, position) order,
only the updates that land in the destination rows it owns, which keeps the result bit-exact;
its slab is that row range.

Inputs are replicated: every rank uploads the same tensors.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

from .trace import IndirectAccess, Store


def core_slice(n_cores: int, rank: int, world: int) -> Tuple[int, int]:
    """Linear core ids [lo, hi) of ``rank``; sizes differ by at most one, no core is lost."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return rank * n_cores // world, (rank + 1) * n_cores // world


def needs_row_ownership(stores: Sequence[Store]) -> bool:
    """True when the kernel stores through an indirect access tile (order between cores matters)."""
    return any(isinstance(s.target, IndirectAccess) for s in stores)


def check_disjoint(ranges_per_rank: Sequence[Sequence[Tuple[int, int]]]):
    """Slabs of different ranks must not overlap, else the exchange would depend on rank order."""
    flat = sorted((lo, hi, r) for r, rs in enumerate(ranges_per_rank) for lo, hi in rs)
    for (lo0, hi0, r0), (lo1, hi1, r1) in zip(flat, flat[1:]):
        if lo1 < hi0 and r0 != r1:
            raise ValueError(f"ranks {r0} and {r1} both write bytes [{lo1:#x}, {min(hi0, hi1):#x})")


def exchange(arena, my_ranges: Sequence[Tuple[int, int]], dist, group=None) -> List[List[Tuple[int, int]]]:
    """Make every rank's slabs visible on all ranks.

    ``arena`` is a 1-D uint8 torch tensor (device memory under NCCL, host memory under gloo)
    whose byte offsets are arena offsets; ``dist`` is ``torch.distributed``.  Returns the slab
    lists of all ranks.  Runs on the current torch stream.
    """
    world = dist.get_world_size(group)
    all_ranges: List[List[Tuple[int, int]]] = [None] * world
    dist.all_gather_object(all_ranges, [tuple(r) for r in my_ranges], group=group)
    check_disjoint(all_ranges)
    broadcast_slabs(arena, all_ranges, dist, group)
    return all_ranges


def broadcast_slabs(arena, all_ranges, dist, group=None):
    """The data step of ``exchange`` alone (slab lists already known, e.g. from an earlier step).

    One equal-sized slab per rank, laid out back to back in rank order (the usual case: contiguous
    row ranges of one output) is a single in-place all-gather under NCCL; anything else is one
    broadcast per slab."""
    world = len(all_ranges)
    if world > 1 and dist.get_backend(group) == "nccl" and all(len(r) == 1 for r in all_ranges):
        los = [r[0][0] for r in all_ranges]
        n = all_ranges[0][0][1] - los[0]
        if n > 0 and all(r[0][1] - r[0][0] == n for r in all_ranges) and \
                all(b == a + n for a, b in zip(los, los[1:])):
            me = dist.get_rank(group)
            dist.all_gather_into_tensor(arena[los[0]:los[0] + world * n], arena[los[me]:los[me] + n], group=group)
            return
    me = dist.get_rank(group)
    for src, ranges in enumerate(all_ranges):
        reg = _regular(ranges)
        if reg is not None:
            # many equal fragments at a constant stride (e.g. a head range of a [seq, heads, dim]
            # output): pack, one broadcast, unpack
            lo, length, stride, count = reg
            view = arena.as_strided((count, length), (stride, 1), lo)
            buf = view.contiguous() if src == me else arena.new_empty((count, length))
            dist.broadcast(buf, src=src, group=group)
            if src != me:
                view.copy_(buf)
            continue
        for lo, hi in ranges:
            if hi > lo:
                dist.broadcast(arena[lo:hi], src=src, group=group)


def _regular(ranges):
    """(lo, length, stride, count) if ``ranges`` are > 4 equal-length runs at a constant stride."""
    if len(ranges) <= 4:
        return None
    lo0, hi0 = ranges[0]
    length, stride = hi0 - lo0, ranges[1][0] - lo0
    for i, (lo, hi) in enumerate(ranges):
        if hi - lo != length or lo != lo0 + i * stride:
            return None
    return lo0, length, stride, len(ranges)


class ShardedRun:
    """A sharded session whose arena lives in a torch tensor, so NCCL can move the slabs.

    ``interp`` is a KTIRInterpreter; the context's work is queued on torch's current stream.
    """

    def __init__(self, interp, func_name: str, rank: int, world: int, dist, **kwargs):
        import torch
        from .interpreter import Session, arena_layout
        self.dist, self.rank, self.world = dist, rank, world
        func = interp._require_module().get_function(func_name)
        tensors = [(k, tuple(v.shape), v.dtype) for k, v in kwargs.items() if isinstance(v, np.ndarray)]
        scalars = {k: v for k, v in kwargs.items() if not isinstance(v, np.ndarray)}
        layout, _ = arena_layout(tensors)
        size = max(off + nbytes for off, nbytes, _, _ in layout.values()) + 512 if layout else 512
        dev = interp.device
        self.arena_t = torch.zeros(size, dtype=torch.uint8, device=f"cuda:{dev.index}")
        dev.set_stream(torch.cuda.current_stream().cuda_stream)
        self.sess = Session(dev, func, tensors, scalars, shard=(rank, world), arena_ptr=self.arena_t.data_ptr())
        self.my_ranges = self.sess.written_ranges()
        self.all_ranges = None

    def upload(self, **arrays):
        for k, v in arrays.items():
            self.sess.upload(k, v)

    def step(self):
        """This rank's launches followed by the slab exchange."""
        self.sess.run()
        if self.world > 1:
            if self.all_ranges is None:
                self.all_ranges = exchange(self.arena_t, self.my_ranges, self.dist)
            else:
                broadcast_slabs(self.arena_t, self.all_ranges, self.dist)

    def download(self, name: str) -> np.ndarray:
        out = self.sess.download(name)
        self.sess.dev.sync()
        return out

    def close(self):
        self.sess.close()

"""ctypes binding of ``libktir_b200.so`` (declared in ``include/ktir_b200.h``).

There is no CPU fallback: if the library is missing or no CUDA device answers,
:func:`lib` / :class:`Device` raise.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libktir_b200.so")

KTB_F16, KTB_F32, KTB_I32, KTB_I64, KTB_I1 = range(5)
DTYPE_CODE = {"f16": KTB_F16, "f32": KTB_F32, "i32": KTB_I32, "i64": KTB_I64, "i1": KTB_I1, "index": KTB_I32}

VM_MAX_OPS, VM_MAX_IN, VM_REGS = 12, 4, 8
VM_OPS = ["MOV", "CONST", "ADD", "SUB", "MUL", "DIV", "MAX", "MAXNUM", "MIN", "MINNUM", "NEG", "ABS",
          "EXP", "LOG", "LOG2", "SQRT", "RSQRT", "TANH", "SIN", "COS", "FMA"]
VM = {n: i for i, n in enumerate(VM_OPS)}
VM_ROUND16 = 0x100
VM_IMM_A, VM_IMM_B = 0x200, 0x400          # row-value programs: operand a / b is the op's immediate


class Status(C.Structure):
    _fields_ = [("negative_index", C.c_int32), ("bad_index_value", C.c_int32),
                ("wait_timeout", C.c_int32), ("wait_site", C.c_int32), ("reserved", C.c_int32 * 4)]


class VmOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("dst", C.c_int32), ("a", C.c_int32), ("b", C.c_int32),
                ("c", C.c_int32), ("imm", C.c_float)]


class VmProgram(C.Structure):
    _fields_ = [("n_in", C.c_int32), ("n_ops", C.c_int32), ("result_reg", C.c_int32),
                ("reserved", C.c_int32), ("ops", VmOp * VM_MAX_OPS)]


class EwArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("dev_item_offsets", C.c_void_p), ("n_items", C.c_int64),
                ("rows", C.c_int32), ("cols", C.c_int32),
                ("row_stride", C.c_int64 * (VM_MAX_IN + 1)), ("dtype", C.c_int32 * (VM_MAX_IN + 1)),
                ("vector_ok", C.c_int32), ("program", VmProgram)]


RP_MAX_RED, RP_MAX_SCAL, RP_MAX_SIDE = 3, 4, 2
RP_OPS = {"add": 0, "max": 1, "maxnum": 2}


class RpPhase(C.Structure):
    _fields_ = [("prog", VmProgram), ("op", C.c_int32), ("round16", C.c_int32), ("load_mask", C.c_int32),
                ("blocked", C.c_int32), ("acc_round16", C.c_int32), ("acc_init", C.c_float)]


class RpScalar(C.Structure):
    _fields_ = [("prog", VmProgram), ("ready_after", C.c_int32), ("reserved", C.c_int32)]


class RpSide(C.Structure):
    _fields_ = [("prog", VmProgram), ("row_stride", C.c_int64), ("dtype", C.c_int32), ("reserved", C.c_int32)]


class RowProgArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("dev_item_offsets", C.c_void_p), ("n_items", C.c_int64),
                ("rows_per_item", C.c_int32), ("cols", C.c_int32),
                ("n_in", C.c_int32), ("n_red", C.c_int32), ("n_scal", C.c_int32), ("out_per_row", C.c_int32),
                ("row_stride", C.c_int64 * (VM_MAX_IN + 1)), ("dtype", C.c_int32 * (VM_MAX_IN + 1)),
                ("blk_stride", C.c_int64 * (VM_MAX_IN + 1)), ("n_blocks", C.c_int32), ("n_side", C.c_int32),
                ("red", RpPhase * RP_MAX_RED), ("scal", RpScalar * RP_MAX_SCAL), ("out", RpPhase),
                ("side", RpSide * RP_MAX_SIDE)]


class SoftmaxArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("dev_item_offsets", C.c_void_p), ("n_items", C.c_int64),
                ("rows_per_item", C.c_int32), ("cols", C.c_int32),
                ("in_row_stride", C.c_int64), ("out_row_stride", C.c_int64),
                ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("f16_arith", C.c_int32), ("max_is_maxnum", C.c_int32),
                ("max_init", C.c_float), ("sum_init", C.c_float)]


ROWS_MAX_IN = 3


class RowOperand(C.Structure):
    _fields_ = [("indirect", C.c_int32), ("dtype", C.c_int32), ("idx_dtype", C.c_int32),
                ("alias_dst", C.c_int32), ("dev_base", C.c_void_p), ("dev_idx_off", C.c_void_p),
                ("idx_stride", C.c_int64), ("idx_mult", C.c_int64), ("pos_stride", C.c_int64),
                ("lo", C.c_int64), ("hi", C.c_int64), ("dev_idx2_off", C.c_void_p),
                ("idx2_stride", C.c_int64), ("idx2_mult", C.c_int64), ("idx2_dtype", C.c_int32),
                ("reserved", C.c_int32)]


class RowsArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("n_tiles", C.c_int64), ("tile_rows", C.c_int32),
                ("cols", C.c_int32), ("n_in", C.c_int32), ("vector_ok", C.c_int32),
                ("inp", RowOperand * ROWS_MAX_IN), ("out", RowOperand), ("program", VmProgram),
                ("dev_rowid_scratch", C.c_void_p), ("dst_row0", C.c_int64), ("dst_rows", C.c_int64)]


class GemmArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("a_off", C.c_int64), ("b_off", C.c_int64), ("c_off", C.c_int64),
                ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("c_dtype", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("c_init", C.c_float), ("reserved", C.c_int32)]


class AttnArgs(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("q_off", C.c_int64), ("o_off", C.c_int64), ("k_off", C.c_int64),
                ("v_off", C.c_int64), ("bt_off", C.c_int64), ("bt_dtype", C.c_int32),
                ("seq_q", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
                ("page", C.c_int32), ("n_pages_total", C.c_int32), ("num_tiles", C.c_int32),
                ("causal", C.c_int32), ("causal_delta", C.c_int32),
                ("q_row_stride", C.c_int64), ("q_head_stride", C.c_int64),
                ("o_row_stride", C.c_int64), ("o_head_stride", C.c_int64),
                ("kv_page_stride", C.c_int64), ("kv_row_stride", C.c_int64), ("kv_head_stride", C.c_int64),
                ("scale", C.c_float), ("m_init", C.c_float), ("l_init", C.c_float), ("kv_group", C.c_int32)]


G_MAXDIM = 6
G_KINDS = {k: i for i, k in enumerate(["load", "addr", "idxadd", "gather", "constv", "fill", "param", "iota", "map",
                                       "ew", "redl", "matmul", "store", "scatter", "ringred", "table", "concat"])}


NO_DEVICE = (1 << 64) - 1


class PipeRegion(C.Structure):
    _fields_ = [("tensor", C.c_int32), ("reserved", C.c_int32), ("dev_off", C.c_uint64), ("rel", C.c_uint64),
                ("width", C.c_uint64), ("height", C.c_uint64), ("pitch", C.c_uint64)]


class PipeChunk(C.Structure):
    _fields_ = [("launch", C.c_void_p), ("launch_args", C.c_void_p), ("n_up", C.c_int32), ("n_down", C.c_int32),
                ("up", C.POINTER(PipeRegion)), ("down", C.POINTER(PipeRegion))]


class GenOpArgs(C.Structure):
    _fields_ = [("kind", C.c_int32), ("op", C.c_int32), ("dt_dst", C.c_int32), ("dt_a", C.c_int32),
                ("dt_b", C.c_int32), ("dt_c", C.c_int32), ("flags", C.c_int32), ("ndim", C.c_int32),
                ("points", C.c_int64), ("elems", C.c_int64), ("ea", C.c_int64), ("eb", C.c_int64), ("ec", C.c_int64),
                ("dst", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("arena", C.c_void_p),
                ("dev_base", C.c_void_p), ("dev_rel", C.c_void_p), ("dev_table", C.c_void_p),
                ("lo", C.c_int64), ("hi", C.c_int64), ("shape", C.c_int64 * G_MAXDIM),
                ("strides", C.c_int64 * G_MAXDIM), ("offset", C.c_int64), ("outer", C.c_int64), ("n", C.c_int64),
                ("inner", C.c_int64), ("h", C.c_int64), ("batch", C.c_int64), ("M", C.c_int64), ("N", C.c_int64),
                ("K", C.c_int64), ("fimm", C.c_double), ("iimm", C.c_int64)]


_lib: Optional[C.CDLL] = None

# name -> (restype, argtypes); every symbol include/ktir_b200.h declares
SYMBOLS = {
    "ktb_init": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "ktb_destroy": (C.c_int, [C.c_void_p]),
    "ktb_last_error": (C.c_char_p, [C.c_void_p]),
    "ktb_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "ktb_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ktb_alloc_host": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "ktb_free_host": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ktb_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]),
    "ktb_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ktb_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ktb_d2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ktb_sync": (C.c_int, [C.c_void_p, C.POINTER(Status)]),
    "ktb_set_stream": (C.c_int, [C.c_void_p, C.c_uint64]),
    "ktb_event_record": (C.c_int, [C.c_void_p, C.c_int]),
    "ktb_event_elapsed_ms": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "ktb_event_record_on": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "ktb_event_sync": (C.c_int, [C.c_void_p, C.c_int]),
    "ktb_status_snapshot": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ktb_flush_l2": (C.c_int, [C.c_void_p]),
    "ktb_launch_count": (C.c_int64, [C.c_void_p]),
    "ktb_graph_begin": (C.c_int, [C.c_void_p]),
    "ktb_graph_end": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "ktb_graph_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ktb_graph_destroy": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ktb_submit_pipeline": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_int, C.POINTER(C.c_uint64)]),
    "ktb_wait_submitted": (C.c_int, [C.c_void_p, C.c_uint64]),
    "ktb_lane_fence": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "ktb_run_pipeline": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "ktb_lane_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t]),
    "ktb_set_copy_threads": (C.c_int, [C.c_int]),
    "ktb_copy_threads": (C.c_int, []),
    "ktb_launch_ew_stream": (C.c_int, [C.c_void_p, C.POINTER(EwArgs)]),
    "ktb_launch_row_program": (C.c_int, [C.c_void_p, C.POINTER(RowProgArgs)]),
    "ktb_launch_row_softmax": (C.c_int, [C.c_void_p, C.POINTER(SoftmaxArgs)]),
    "ktb_launch_rows_program": (C.c_int, [C.c_void_p, C.POINTER(RowsArgs)]),
    "ktb_launch_scatter_rows": (C.c_int, [C.c_void_p, C.POINTER(RowsArgs)]),
    "ktb_scatter_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "ktb_launch_scatter_rows_static": (C.c_int, [C.c_void_p, C.POINTER(RowsArgs)]),
    "ktb_launch_generic": (C.c_int, [C.c_void_p, C.POINTER(GenOpArgs)]),
    "ktb_launch_gemm_f16": (C.c_int, [C.c_void_p, C.POINTER(GemmArgs)]),
    "ktb_launch_attention_fwd": (C.c_int, [C.c_void_p, C.POINTER(AttnArgs)]),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ktir_cpu_b200.build` "
                "(this backend has no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


class DeviceError(RuntimeError):
    pass


class DeviceIndexError(IndexError):
    pass


class Device:
    """One context on one GPU: memory, transfers, launches, events."""

    def __init__(self, device: int = 0):
        self.lib = lib()
        h = C.c_void_p()
        rc = self.lib.ktb_init(device, C.byref(h))
        if rc != 0 or not h:
            raise DeviceError(f"ktb_init(device={device}) failed (code {rc}): no usable CUDA device; "
                              "this backend has no CPU fallback")
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.ktb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc: int):
        if rc != 0:
            msg = self.lib.ktb_last_error(self.h).decode(errors="replace")
            if rc == -4 and "is negative" in msg:
                raise DeviceIndexError(msg)
            if rc == -3:
                raise NotImplementedError(msg)
            raise DeviceError(f"libktir_b200 error {rc}: {msg}")

    # memory ---------------------------------------------------------------
    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.lib.ktb_alloc(self.h, nbytes, C.byref(p)))
        return p.value

    def free(self, ptr: int):
        self.check(self.lib.ktb_free(self.h, C.c_void_p(ptr)))

    def alloc_host(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.lib.ktb_alloc_host(self.h, nbytes, C.byref(p)))
        return p.value

    def free_host(self, ptr: int):
        self.check(self.lib.ktb_free_host(self.h, C.c_void_p(ptr)))

    def memset(self, ptr: int, value: int, nbytes: int):
        self.check(self.lib.ktb_memset(self.h, C.c_void_p(ptr), value, nbytes))

    def h2d(self, dev_ptr: int, host: np.ndarray):
        host = np.ascontiguousarray(host)
        self.check(self.lib.ktb_h2d(self.h, C.c_void_p(dev_ptr), C.c_void_p(host.ctypes.data), host.nbytes))
        return host          # keep alive until the next sync

    def h2d_raw(self, dev_ptr: int, host_ptr: int, nbytes: int):
        self.check(self.lib.ktb_h2d(self.h, C.c_void_p(dev_ptr), C.c_void_p(host_ptr), nbytes))

    def d2h(self, host: np.ndarray, dev_ptr: int):
        assert host.flags["C_CONTIGUOUS"]
        self.check(self.lib.ktb_d2h(self.h, C.c_void_p(host.ctypes.data), C.c_void_p(dev_ptr), host.nbytes))

    def d2h_raw(self, host_ptr: int, dev_ptr: int, nbytes: int):
        self.check(self.lib.ktb_d2h(self.h, C.c_void_p(host_ptr), C.c_void_p(dev_ptr), nbytes))

    # pipelined transfers: lane 0 = launch stream, 1 = upload lane, 2 = read-back lane
    def fence(self, src_lane: int, dst_lane: int):
        self.check(self.lib.ktb_lane_fence(self.h, src_lane, dst_lane))

    def run_pipeline(self, arena: int, chunks, n_chunks: int, pinned, src, n_tensors: int):
        self.check(self.lib.ktb_run_pipeline(self.h, C.c_void_p(arena), chunks, n_chunks, pinned, src, n_tensors))

    def submit_pipeline(self, arena: int, chunks, n_chunks: int, pinned, src, n_tensors: int, snapshot_ptr: int,
                        event_slot: int) -> int:
        seq = C.c_uint64()
        self.check(self.lib.ktb_submit_pipeline(self.h, C.c_void_p(arena), chunks, n_chunks, pinned, src, n_tensors,
                                                C.c_void_p(snapshot_ptr), event_slot, C.byref(seq)))
        return seq.value

    def wait_submitted(self, seq: int):
        self.check(self.lib.ktb_wait_submitted(self.h, C.c_uint64(seq)))

    def lane_d2h(self, host_ptr: int, dev_ptr: int, width: int, height: int = 1, pitch: int = 0):
        self.check(self.lib.ktb_lane_d2h(self.h, C.c_void_p(host_ptr), C.c_void_p(dev_ptr), width, height,
                                         pitch or width))

    def sync(self) -> Status:
        st = Status()
        self.check(self.lib.ktb_sync(self.h, C.byref(st)))
        return st

    def upload(self, arr: np.ndarray) -> int:
        """Allocate device memory holding ``arr`` (synchronous)."""
        arr = np.ascontiguousarray(arr)
        p = self.alloc(max(arr.nbytes, 16))
        if arr.nbytes:
            self.h2d(p, arr)
            self.sync()
        return p

    def set_stream(self, cuda_stream: int):
        """Queue this context's work on an existing CUDA stream (e.g. torch's current stream)."""
        self.check(self.lib.ktb_set_stream(self.h, C.c_uint64(cuda_stream)))

    @property
    def index(self) -> int:
        return self.device

    # timing ----------------------------------------------------------------
    def record(self, slot: int):
        self.check(self.lib.ktb_event_record(self.h, slot))

    def record_on(self, slot: int, lane: int):
        self.check(self.lib.ktb_event_record_on(self.h, slot, lane))

    def event_sync(self, slot: int):
        self.check(self.lib.ktb_event_sync(self.h, slot))

    def status_snapshot(self, host_ptr: int):
        self.check(self.lib.ktb_status_snapshot(self.h, C.c_void_p(host_ptr)))

    def elapsed_ms(self, a: int, b: int) -> float:
        ms = C.c_float()
        self.check(self.lib.ktb_event_elapsed_ms(self.h, a, b, C.byref(ms)))
        return float(ms.value)

    def flush_l2(self):
        self.check(self.lib.ktb_flush_l2(self.h))

    def launch_count(self) -> int:
        return int(self.lib.ktb_launch_count(self.h))

    # graphs -----------------------------------------------------------------
    def graph_begin(self):
        self.check(self.lib.ktb_graph_begin(self.h))

    def graph_end(self) -> Optional[int]:
        g = C.c_void_p()
        rc = self.lib.ktb_graph_end(self.h, C.byref(g))
        return g.value if rc == 0 else None

    def graph_launch(self, g: int):
        self.check(self.lib.ktb_graph_launch(self.h, C.c_void_p(g)))

    def graph_destroy(self, g: int):
        self.lib.ktb_graph_destroy(self.h, C.c_void_p(g))


_devices = {}


def get_device(index: int = 0) -> Device:
    d = _devices.get(index)
    if d is None or d.h is None:
        d = _devices[index] = Device(index)
    return d


class PlanOnlyDevice:
    """Stands in for :class:`Device` when only the launch plan is wanted (no GPU needed).

    It can hold no data and launch nothing: planning code may call ``upload`` /
    ``alloc`` / ``free``; anything that would run on the GPU raises."""

    h = None
    lib = None

    def alloc(self, nbytes: int) -> int:
        return 0

    def free(self, ptr: int):
        pass

    def upload(self, arr) -> int:
        return 0

    def sync(self):
        return Status()

    def check(self, rc):
        raise DeviceError("plan-only device cannot launch kernels")

    def __getattr__(self, name):
        raise DeviceError(f"plan-only device has no '{name}'")

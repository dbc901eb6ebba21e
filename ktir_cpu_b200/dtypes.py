"""KTIR element types and their NumPy / device encodings.

Same table as the reference (ktir_cpu/dtypes.py:24-47): ``index`` tiles are
stored as 32-bit integers, ``i1`` as one byte, fp8/mxfp8 are placeholders that
raise ``NotImplementedError``.
"""
import numpy as np

_NP = {
    "f16": np.float16, "fp16": np.float16, "float16": np.float16,
    "f32": np.float32, "float32": np.float32,
    "i1": np.bool_,
    "i32": np.int32, "si32": np.int32, "index": np.int32,
    "i64": np.int64, "si64": np.int64,
}
_CANON = {"fp16": "f16", "float16": "f16", "float32": "f32", "si32": "i32", "si64": "i64"}
_PLACEHOLDER = frozenset({"fp8", "mxfp8"})
_FROM_NP = {np.dtype(np.float16): "f16", np.dtype(np.float32): "f32",
            np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}

# Device-side type codes shared with csrc/ktir_b200.h (KTB_F16 ...).
DEV_CODE = {"f16": 0, "f32": 1, "i32": 2, "i64": 3, "i1": 4, "index": 2}


def canon(dtype: str) -> str:
    return _CANON.get(dtype, dtype)


def to_np_dtype(dtype: str) -> np.dtype:
    if dtype in _PLACEHOLDER:
        raise NotImplementedError(
            f"dtype {dtype!r} is a placeholder pending hardware confirmation")
    try:
        return np.dtype(_NP[dtype])
    except KeyError:
        raise ValueError(f"Unsupported KTIR dtype: {dtype!r}")


def bytes_per_elem(dtype: str) -> int:
    return int(to_np_dtype(dtype).itemsize)


def to_ktir_dtype(np_dtype) -> str:
    try:
        return _FROM_NP[np.dtype(np_dtype)]
    except KeyError:
        raise ValueError(f"No KTIR dtype for NumPy dtype: {np.dtype(np_dtype)!r}")


def is_float(dtype: str) -> bool:
    return canon(dtype) in ("f16", "f32")

"""Host-side native helpers (``csrc/host/*.cpp`` inside the same shared library as the kernels): the multi-threaded group
quantiser the converter uses when the library has been built.  Results are bit-identical to the numpy implementation
in ``format/quantize.py``, so a converted file does not depend on which one ran."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from ..format.spec import QuantMethod
from . import build as _build

_lib: Optional[ctypes.CDLL] = None
_tried = False


def _load() -> Optional[ctypes.CDLL]:
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    try:
        if not _build.is_built():
            return None
        lib = ctypes.CDLL(_build.LIB_PATH)
        lib.zse_host_quantize_int4.restype = ctypes.c_int
        lib.zse_host_quantize_int4.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_void_p]
        lib.zse_host_quantize_int8.restype = ctypes.c_int
        lib.zse_host_quantize_int8.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p]
        lib.zse_host_bf16_to_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        lib.zse_host_bf16_to_f32.restype = None
        _lib = lib
    except (OSError, AttributeError):
        _lib = None
    return _lib


def available() -> bool:
    return _load() is not None


def quantize(values: np.ndarray, method: int, group_size: int):
    """Same return values as ``quantize_int4_arrays`` / ``quantize_int8_arrays``."""
    lib = _load()
    if lib is None:
        raise RuntimeError("native library not built")
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    groups = (v.size + group_size - 1) // group_size
    scales = np.empty(groups, dtype=np.float16)
    if int(method) == int(QuantMethod.INT8_SYM):
        q = np.empty(groups * group_size, dtype=np.int8)
        rc = lib.zse_host_quantize_int8(v.ctypes.data, v.size, group_size, q.ctypes.data, scales.ctypes.data)
        if rc != 0:
            raise ValueError("bad arguments to the native INT8 quantiser")
        return q, scales
    packed = np.empty(groups * group_size // 2, dtype=np.uint8)
    zeros = np.empty(groups, dtype=np.float16)
    rc = lib.zse_host_quantize_int4(v.ctypes.data, v.size, group_size, packed.ctypes.data, scales.ctypes.data,
                                    zeros.ctypes.data)
    if rc != 0:
        raise ValueError("bad arguments to the native INT4 quantiser")
    return packed, scales, zeros


def bf16_to_f32(raw_u16: np.ndarray) -> np.ndarray:
    lib = _load()
    src = np.ascontiguousarray(raw_u16, dtype=np.uint16).reshape(-1)
    if lib is None:
        return (src.astype(np.uint32) << 16).view(np.float32)
    out = np.empty(src.size, dtype=np.float32)
    lib.zse_host_bf16_to_f32(src.ctypes.data, out.ctypes.data, src.size)
    return out

"""The reference's fast-quantiser entry points (zse-engine/zse_engine/format/fast_quant.py:304-497) over the
quantiser of this package: raw safetensors bytes in, packed bytes out.

The reference compiles a C file with gcc at first use; here the same functions run in the C++ quantiser that is built
with the library (``csrc/host/quant.cpp`` through ``ops/host_native.py``) when it is present and in numpy otherwise -
``is_available()`` says which.  Results follow ``format/quantize.py`` (round half away from zero at .5 is "nearest";
the reference's C code rounds half up, see the rounding test in tests/test_format.py).
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

from . import quantize as Q
from .convert import _to_f32


def is_available() -> bool:
    """True when the compiled quantiser is loaded (the numpy path is used otherwise, with identical results)."""
    try:
        from ..ops import host_native
        return host_native.available()
    except Exception:
        return False


def _values(raw_data, dtype: str, num_elements: int) -> np.ndarray:
    itemsize = {"F32": 4, "F64": 8}.get(dtype, 2)
    return _to_f32(memoryview(raw_data)[: num_elements * itemsize], dtype)


def _quant(values: np.ndarray, method: int, group_size: int):
    if is_available():
        from ..ops import host_native
        return host_native.quantize(values, method, group_size)
    if method == 1:
        return Q.quantize_int4_arrays(values, group_size)
    return Q.quantize_int8_arrays(values, group_size)


def quantize_tensor_fast(raw_data, dtype: str, num_elements: int, group_size: int = 128) -> Tuple[bytes, bytes, bytes]:
    """INT4 asymmetric: ``(packed, scales fp16, zeros fp16)`` as bytes."""
    p, s, z = _quant(_values(raw_data, dtype, num_elements), 1, group_size)
    return np.asarray(p).tobytes(), np.asarray(s).tobytes(), np.asarray(z).tobytes()


def quantize_tensor_int8_fast(raw_data, dtype: str, num_elements: int, group_size: int = 128) -> Tuple[bytes, bytes]:
    """INT8 symmetric: ``(values int8, scales fp16)`` as bytes."""
    res = _quant(_values(raw_data, dtype, num_elements), 2, group_size)
    return np.asarray(res[0]).tobytes(), np.asarray(res[1]).tobytes()


def convert_to_fp16_fast(raw_data, dtype: str, num_elements: int) -> bytes:
    if dtype == "F16":
        return bytes(memoryview(raw_data)[: num_elements * 2])
    return _values(raw_data, dtype, num_elements).astype(np.float16).tobytes()


def repack_int4_tiled(packed_data, N: int, K: int) -> bytes:
    """Row-major ``[N, K/2]`` nibbles -> the reference's ``[N/64][K/16][64][8]`` tiles (its WMMA layout; the loader of
    this package reads such files back and re-tiles them for its own kernels)."""
    return Q.tile_int4_64x8(np.frombuffer(bytes(packed_data), dtype=np.uint8), N, K).tobytes()

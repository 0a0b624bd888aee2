"""Group quantisation of weight tensors (vectorised numpy; the native version lives in csrc/host).

INT4 is asymmetric: for every run of ``group_size`` values of the *flattened* tensor
``scale = (max-min)/15`` (1.0 when the range is below 1e-10), ``zero = min`` and
``q = clamp(round((v-zero)/scale), 0, 15)``; the value is rebuilt as ``q*scale + zero`` (the zero
is an fp16 *minimum*, not an integer zero point).  Two nibbles per byte, low nibble = even index.
INT8 is symmetric with ``scale = amax/127``.  Semantics:
zse-engine/zse_engine/format/quantize.py:18-235; the C fast path of the reference
(zse-engine/zse_engine/format/fast_quant.py:93-132) differs in two details that ``rounding="c"``
reproduces: round-half-up ``(int)(v+0.5)`` and truncating fp32->fp16 with subnormals flushed to zero.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np


def _as_f32(weights, keep_f64: bool = False) -> np.ndarray:
    if isinstance(weights, np.ndarray):
        if keep_f64 and weights.dtype == np.float64:
            return np.ascontiguousarray(weights).reshape(-1)
        return np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
    try:
        import torch
        if isinstance(weights, torch.Tensor):
            return weights.detach().to(torch.float32).cpu().contiguous().numpy().reshape(-1)
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(weights, dtype=np.float64 if keep_f64 else np.float32).reshape(-1)


def f32_to_f16_truncate(x: np.ndarray) -> np.ndarray:
    """fp32 -> fp16 bit pattern the way the reference's C helper does it (no rounding, FTZ)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    sign = ((bits >> 16) & 0x8000).astype(np.uint16)
    exp = ((bits >> 23) & 0xFF).astype(np.int32) - 127 + 15
    mant = (bits & 0x7FFFFF) >> 13
    out = np.where(exp <= 0, 0, np.where(exp >= 31, 0x7C00, (exp.clip(0, 31) << 10) | mant)).astype(np.uint16)
    return (sign | out).view(np.float16)


def _pad_groups(flat: np.ndarray, group_size: int) -> np.ndarray:
    rem = flat.size % group_size
    if rem:
        flat = np.concatenate([flat, np.zeros(group_size - rem, dtype=flat.dtype)])
    return flat.reshape(-1, group_size)


def quantize_int4_arrays(weights, group_size: int = 128, rounding: str = "nearest"):
    """Returns ``(packed u8 [G*gs/2], scales f16 [G], zeros f16 [G])`` as numpy arrays."""
    if rounding != "c":
        # double precision throughout, like the reference's pure-python writer
        g = _pad_groups(_as_f32(weights, keep_f64=True), group_size).astype(np.float64, copy=False)
        gmin = g.min(axis=1)
        rng = g.max(axis=1) - gmin
        scale = np.where(rng < 1e-10, 1.0, rng / 15.0)
        q = np.rint((g - gmin[:, None]) * (1.0 / scale)[:, None]).astype(np.int32)
        q = np.clip(q, 0, 15).astype(np.uint8).reshape(-1)
        return (q[0::2] | (q[1::2] << 4)).astype(np.uint8), scale.astype(np.float16), gmin.astype(np.float16)
    g = _pad_groups(_as_f32(weights), group_size)
    gmin = g.min(axis=1)
    gmax = g.max(axis=1)
    rng = gmax - gmin
    ok = rng > 1e-10
    scale = np.where(ok, rng / np.float32(15.0), np.float32(1.0)).astype(np.float32)
    inv = np.where(ok, np.float32(15.0) / np.where(ok, rng, 1), np.float32(0.0)).astype(np.float32)
    q = ((g - gmin[:, None]) * inv[:, None] + np.float32(0.5)).astype(np.int32)
    scales16, zeros16 = f32_to_f16_truncate(scale), f32_to_f16_truncate(gmin)
    q = np.clip(q, 0, 15).astype(np.uint8).reshape(-1)
    packed = (q[0::2] | (q[1::2] << 4)).astype(np.uint8)
    return packed, scales16, zeros16


def quantize_tensor(weights, group_size: int = 128, rounding: str = "nearest") -> Tuple[bytes, bytes, bytes]:
    p, s, z = quantize_int4_arrays(weights, group_size, rounding)
    return p.tobytes(), s.tobytes(), z.tobytes()


def dequantize_int4_arrays(packed, scales, zeros, num_elements: int, group_size: int = 128) -> np.ndarray:
    p = np.frombuffer(packed, dtype=np.uint8) if not isinstance(packed, np.ndarray) else packed.reshape(-1)
    s = np.frombuffer(scales, dtype=np.float16) if not isinstance(scales, np.ndarray) else scales.reshape(-1)
    z = np.frombuffer(zeros, dtype=np.float16) if not isinstance(zeros, np.ndarray) else zeros.reshape(-1)
    groups = (num_elements + group_size - 1) // group_size
    p = p[: groups * group_size // 2]
    q = np.empty(p.size * 2, dtype=np.float32)
    q[0::2] = p & 0x0F
    q[1::2] = p >> 4
    q = q.reshape(groups, group_size)
    out = q * s[:groups].astype(np.float32)[:, None] + z[:groups].astype(np.float32)[:, None]
    return out.reshape(-1)[:num_elements]


def dequantize_tensor(packed, scales, zeros, shape: Sequence[int], group_size: int = 128):
    n = int(np.prod(shape)) if len(shape) else 1
    return dequantize_int4_arrays(packed, scales, zeros, n, group_size)


def quantize_int8_arrays(weights, group_size: int = 128, rounding: str = "nearest"):
    g = _pad_groups(_as_f32(weights), group_size)
    amax = np.abs(g).max(axis=1)
    ok = amax > 1e-10
    scale = np.where(ok, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    inv = np.where(ok, np.float32(127.0) / np.where(ok, amax, 1), np.float32(0.0))
    v = g * inv[:, None]
    if rounding == "c":
        q = (v + np.where(v >= 0, np.float32(0.5), np.float32(-0.5))).astype(np.int32)
        s16 = f32_to_f16_truncate(scale)
    else:
        q = np.rint(v).astype(np.int32)
        s16 = scale.astype(np.float16)
    return np.clip(q, -128, 127).astype(np.int8).reshape(-1), s16


def quantize_tensor_int8(weights, group_size: int = 128, rounding: str = "nearest") -> Tuple[bytes, bytes]:
    q, s = quantize_int8_arrays(weights, group_size, rounding)
    return q.tobytes(), s.tobytes()


def dequantize_tensor_int8(packed, scales, shape: Sequence[int], group_size: int = 128) -> np.ndarray:
    n = int(np.prod(shape)) if len(shape) else 1
    groups = (n + group_size - 1) // group_size
    q = np.frombuffer(packed, dtype=np.int8)[: groups * group_size].astype(np.float32).reshape(groups, group_size)
    s = np.frombuffer(scales, dtype=np.float16)[:groups].astype(np.float32)
    return (q * s[:, None]).reshape(-1)[:n]


def quantize_fp16(weights) -> bytes:
    return _as_f32(weights).astype(np.float16).tobytes()


def compute_packed_size(num_elements: int, group_size: int = 128) -> Tuple[int, int, int]:
    padded = (num_elements + group_size - 1) // group_size * group_size
    groups = padded // group_size
    return padded // 2, groups * 2, groups * 2


# ---- the 64x8 re-tiling the reference's C converter applies to 2-D INT4 data --------------------
def tile_int4_64x8(packed_rowmajor, n_rows: int, k_cols: int) -> np.ndarray:
    """``[N, K/2]`` bytes -> ``[ceil(N/64)][ceil(K/16)][64][8]`` bytes, zero padded
    (zse-engine/zse_engine/format/fast_quant.py:193-225)."""
    half = k_cols // 2
    src = np.frombuffer(packed_rowmajor, dtype=np.uint8)[: n_rows * half].reshape(n_rows, half)
    nt, kt = (n_rows + 63) // 64, (k_cols + 15) // 16
    full = np.zeros((nt * 64, kt * 8), dtype=np.uint8)
    full[:n_rows, :half] = src
    return np.ascontiguousarray(full.reshape(nt, 64, kt, 8).transpose(0, 2, 1, 3)).reshape(-1)


def untile_int4_64x8(tiled, n_rows: int, k_cols: int) -> np.ndarray:
    half = k_cols // 2
    nt, kt = (n_rows + 63) // 64, (k_cols + 15) // 16
    t = np.frombuffer(tiled, dtype=np.uint8)[: nt * kt * 512].reshape(nt, kt, 64, 8)
    full = t.transpose(0, 2, 1, 3).reshape(nt * 64, kt * 8)
    return np.ascontiguousarray(full[:n_rows, :half]).reshape(-1)

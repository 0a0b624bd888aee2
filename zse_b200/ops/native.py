"""ctypes binding of ``libzse_b200.so`` (see ``csrc/api.h``) on torch tensors.

Every call launches on ``torch.cuda.current_stream()``, so the kernels order with torch ops and are captured by
``torch.cuda.graph``.  A negative return code raises ``NativeError``; device-side failures are read with
``check_status``.  On a machine with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p, POINTER, c_uint32
from typing import Optional

import torch

from . import build as _build

_ERRORS = {-1: "unsupported shape", -2: "misaligned pointer or stride", -3: "CUDA driver call failed",
           -4: "kernel launch failed", -5: "size beyond a built-in limit"}


class NativeError(RuntimeError):
    pass


class DeviceStatusError(RuntimeError):
    """A kernel reported a failure through the status word (bounded wait ran out, bad index, ...)."""


_lib: Optional[ctypes.CDLL] = None

_SIGS = {
    "zse_gemm_w4": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_void_p]),
    "zse_gemm_w4_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "zse_gemm_w4_dec": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_void_p, c_void_p, c_void_p]),
    "zse_gemm_w4_dec_qkv_rope": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                         c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                         c_void_p, c_void_p]),
    "zse_gemm_w8_dec": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_void_p, c_void_p, c_void_p]),
    "zse_gemm_w8_dec_qkv_rope": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                         c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                         c_void_p, c_void_p]),
    "zse_w8_tiled_bytes": (c_int64, [c_int, c_int]),
    "zse_repack_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "zse_dequant_w8_tiled": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "zse_gemm_w4_dec_workspace_bytes": (c_int64, [c_int]),
    "zse_gemm_w4_dec_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "zse_gemm_w4_dec_plan": (None, [c_int, c_int, c_int, c_int, POINTER(c_int)]),
    "zse_gemm_w4_dec_set_tuning": (None, [c_int, c_int]),
    "zse_gemm_f16": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p]),
    "zse_gemm_f16_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "zse_w4_tiled_bytes": (c_int64, [c_int, c_int]),
    "zse_repack_w4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "zse_dequant_w4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "zse_dequant_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "zse_quantize_w4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "zse_embedding": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "zse_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                c_void_p]),
    "zse_rmsnorm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "zse_rope_kv_write": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "zse_swiglu": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "zse_headnorm_rope_kv_write": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                           c_int, c_void_p]),
    "zse_attn_generic": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                 c_int, c_void_p]),
    "zse_norm_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_float, c_void_p]),
    "zse_softcap_f16": (c_int, [c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "zse_bias_add": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "zse_attn_decode_scratch_floats": (c_int64, [c_int, c_int, c_int, c_int]),
    "zse_attn_decode": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "zse_attn_prefill": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "zse_attn_decode_ext": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                    c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                    c_void_p]),
    "zse_attn_prefill_ext": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                     c_int, c_void_p]),
    "zse_argmax": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "zse_sample": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64,
                           c_void_p]),
    "zse_apply_repetition_penalty": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                             c_void_p]),
    "zse_lora_shrink": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "zse_attn_prefill_tc": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]),
    "zse_lora_apply": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_void_p]),
    "zse_lora_expand": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_void_p]),
    "zse_tp_ctx_create": (c_void_p, [c_int, c_int, c_int, c_int, POINTER(c_uint64), POINTER(c_uint64), c_uint64,
                                     POINTER(c_uint64), POINTER(c_uint64)]),
    "zse_tp_ctx_destroy": (None, [c_void_p]),
    "zse_tp_reduce_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float,
                                          c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_reduce_add_rmsnorm_emulated": (c_int, [c_void_p, POINTER(c_uint64), POINTER(c_uint64), c_int, c_void_p,
                                                   POINTER(c_uint64), c_int, c_float, c_int, c_void_p, c_void_p]),
    "zse_tp_reduce_scatter_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float,
                                          c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_reduce_scatter_add_rmsnorm_emulated": (c_int, [c_void_p, POINTER(c_uint64), POINTER(c_uint64), c_int, c_void_p,
                                                   POINTER(c_uint64), c_int, c_float, c_int, c_void_p, c_void_p]),
    "zse_tp_ctx_set_push": (c_int, [c_void_p, c_int, POINTER(c_uint64), c_uint64, POINTER(c_uint64), c_uint64,
                                    POINTER(c_uint64)]),
    "zse_tp_gemm_w4_push": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_void_p]),
    "zse_tp_gemm_dec_allreduce_norm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                               c_void_p]),
    "zse_tp_sum_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p,
                                       c_void_p]),
    "zse_tp_ctx_set_sp": (c_int, [c_void_p, c_int, c_int, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64),
                                  c_uint64, POINTER(c_uint64), POINTER(c_uint64)]),
    "zse_tp_gemm_w4_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p]),
    "zse_tp_gemm_w4_gathered": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_sp_sum_norm_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p,
                                          c_void_p]),
    "zse_tp_sp_sum_norm_gather_emulated": (c_int, [c_void_p, POINTER(c_uint64), c_void_p, c_int, c_float, c_int,
                                                   c_void_p, c_void_p]),
    "zse_tp_sp_wait": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_sum_add_rmsnorm_emulated": (c_int, [c_void_p, POINTER(c_uint64), c_void_p, POINTER(c_uint64), c_int,
                                                c_float, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_ctx_set_gather": (c_int, [c_void_p, c_int, c_int, POINTER(c_uint64), POINTER(c_uint64)]),
    "zse_read_probe": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_gather_rows": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_gather_rows_emulated": (c_int, [c_void_p, POINTER(c_uint64), c_int, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_argmax": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "zse_tp_argmax_emulated": (c_int, [c_void_p, POINTER(c_uint64), c_int, POINTER(c_uint64), c_int, c_int, c_int,
                                       c_int, c_void_p, c_void_p]),
    "zse_status_read": (c_int, [c_void_p, POINTER(c_uint32)]),
    "zse_device_info": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int64), POINTER(c_int64)]),
    "zse_build_info": (c_char_p, []),
    "zse_set_pdl": (None, [c_int]),
    "zse_gemm_w4_set_mode": (None, [c_int]),
    "zse_get_pdl": (c_int, []),
}


def lib_path() -> str:
    """The library this process loads: the ordinary build, or the file ZSE_NATIVE_LIB names (an instrumented variant
    built by ``python -m zse_b200.ops.build --variant NAME``)."""
    return os.environ.get("ZSE_NATIVE_LIB") or _build.LIB_PATH


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise NativeError(f"{path} is missing: run `python -m zse_b200.ops.build`")
        _build.build()
    lib = ctypes.CDLL(path)
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue   # optional entry points are looked up by their users
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def available() -> bool:
    return torch.cuda.is_available()


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = [0]      # kernels launched through this module (graph replays are accounted by the runner)


def _ck(rc: int, what: str, launches: int = 1) -> None:
    if rc < 0:
        raise NativeError(f"{what}: {_ERRORS.get(rc, rc)}")
    LAUNCHES[0] += launches


class Status:
    """The 16-byte device status word shared by all launches of one engine."""

    def __init__(self, device):
        self.buf = torch.zeros(4, dtype=torch.int32, device=device)

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def read(self):
        out = (c_uint32 * 4)()
        _ck(load().zse_status_read(self.ptr, out), "status read", 0)
        return tuple(out)

    def check(self) -> None:
        code, block, where, detail = self.read()
        if code:
            self.buf.zero_()
            kind = {1: "wait timed out", 2: "bad argument", 3: "peer wait timed out"}.get(code, f"code {code}")
            raise DeviceStatusError(f"device reported: {kind} (block {block}, site {where}, detail {detail})")


# ---- thin wrappers (shapes are checked by the callers in ops/linear.py and the model runner) -------------------
def gemm_w4(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, k_split, status):
    _ck(load().zse_gemm_w4(_p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(out), M, N, K, ldo, epilogue, k_split,
                           status, _stream()), "gemm_w4")


def gemm_w4_dec(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, workspace, status):
    """Decode-sized INT4 GEMM (M <= 64) of the persistent kernel; epilogue 0 fp16 (+bias), 1 SwiGLU, 2 fp32."""
    _ck(load().zse_gemm_w4_dec(_p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(out), M, N, K, ldo, epilogue,
                               _p(workspace), status, _stream()), "gemm_w4_dec")


def gemm_w4_dec_qkv_rope(w_tiled, x, x_rows_cap, bias, qkv_out, ldo, M, K, nh, nkv, kv_layer, block_size, positions,
                         slots, cos_sin, max_position, workspace, status):
    _ck(load().zse_gemm_w4_dec_qkv_rope(_p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(qkv_out), ldo, M, K, nh, nkv,
                                        _p(kv_layer), block_size, _p(positions), _p(slots), _p(cos_sin), max_position,
                                        _p(workspace), status, _stream()), "gemm_w4_dec_qkv_rope")


def gemm_w8_dec(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, workspace, status):
    """The decode-sized GEMM for INT8 weights tiled by ``repack_w8`` (the weights stay 8 bits wide in memory)."""
    _ck(load().zse_gemm_w8_dec(_p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(out), M, N, K, ldo, epilogue,
                               _p(workspace), status, _stream()), "gemm_w8_dec")


def gemm_w8_dec_qkv_rope(w_tiled, x, x_rows_cap, bias, qkv_out, ldo, M, K, nh, nkv, kv_layer, block_size, positions,
                         slots, cos_sin, max_position, workspace, status):
    _ck(load().zse_gemm_w8_dec_qkv_rope(_p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(qkv_out), ldo, M, K, nh, nkv,
                                        _p(kv_layer), block_size, _p(positions), _p(slots), _p(cos_sin), max_position,
                                        _p(workspace), status, _stream()), "gemm_w8_dec_qkv_rope")


def repack_w8(q, scales, out_tiled, N, K, interleave_rows=0):
    _ck(load().zse_repack_w8(_p(q), _p(scales), _p(out_tiled), N, K, interleave_rows, _stream()), "repack_w8")


def dequant_w8_tiled(tiled, out_f16, N, K, interleave_rows=0):
    _ck(load().zse_dequant_w8_tiled(_p(tiled), _p(out_f16), N, K, interleave_rows, _stream()), "dequant_w8_tiled")


def gemm_w4_dec_workspace(device, sm_count: int) -> torch.Tensor:
    """Zeroed workspace (partial sums + synchronisation words) for the persistent decode GEMM on ``device``."""
    n = int(load().zse_gemm_w4_dec_workspace_bytes(sm_count))
    return torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device=device)


def gemm_w4_dec_supported(M, N, K, epilogue) -> bool:
    return bool(load().zse_gemm_w4_dec_supported(M, N, K, epilogue))


def gemm_w4_dec_plan(N, K, epilogue, sm_count):
    out = (c_int * 2)()
    load().zse_gemm_w4_dec_plan(N, K, epilogue, sm_count, out)
    return out[0], out[1]


def gemm_f16(w, w_rows, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, k_split, status):
    _ck(load().zse_gemm_f16(_p(w), w_rows, _p(x), x_rows_cap, _p(bias), _p(out), M, N, K, ldo, epilogue, k_split,
                            status, _stream()), "gemm_f16")


def gemm_w4_splits(M, N, K, k_split) -> int:
    return load().zse_gemm_w4_splits(M, N, K, k_split)


def gemm_f16_splits(M, N, K, k_split) -> int:
    return load().zse_gemm_f16_splits(M, N, K, k_split)


def w4_tiled_bytes(N, K) -> int:
    return load().zse_w4_tiled_bytes(N, K)


def repack_w4(packed, scales, zeros, out, N, K, interleave_rows=0):
    _ck(load().zse_repack_w4(_p(packed), _p(scales), _p(zeros), _p(out), N, K, interleave_rows, _stream()),
        "repack_w4")


def dequant_w4(packed, scales, zeros, out, n_elements, group_size):
    _ck(load().zse_dequant_w4(_p(packed), _p(scales), _p(zeros), _p(out), n_elements, group_size, _stream()),
        "dequant_w4")


def dequant_w8(q, scales, out, n_elements, group_size):
    _ck(load().zse_dequant_w8(_p(q), _p(scales), _p(out), n_elements, group_size, _stream()), "dequant_w8")


def quantize_w4(w, packed, scales, zeros, n_groups):
    _ck(load().zse_quantize_w4(_p(w), _p(packed), _p(scales), _p(zeros), n_groups, _stream()), "quantize_w4")


def embedding(table, ids, out, M, H, vocab, scale, status):
    _ck(load().zse_embedding(_p(table), _p(ids), _p(out), M, H, vocab, scale, status, _stream()), "embedding")


def add_rmsnorm(residual, partials, n_partials, add_f16, weight, out, M, H, eps):
    _ck(load().zse_add_rmsnorm(_p(residual), _p(partials), n_partials, _p(add_f16), _p(weight), _p(out), M, H, eps,
                               _stream()), "add_rmsnorm")


def rmsnorm_f16(x, weight, out, M, H, eps):
    _ck(load().zse_rmsnorm_f16(_p(x), _p(weight), _p(out), M, H, eps, _stream()), "rmsnorm_f16")


def rope_kv_write(qkv, kv_layer, positions, slots, inv_freq, M, nh, nkv, hd, rotary_dim, block_size, planes=None,
                  n_planes=0, bias=None):
    _ck(load().zse_rope_kv_write(_p(qkv), _p(kv_layer), _p(positions), _p(slots), _p(inv_freq), M, nh, nkv, hd,
                                 rotary_dim, block_size, _p(planes), n_planes, _p(bias), _stream()), "rope_kv_write")


def headnorm_rope_kv_write(qkv, kv_layer, positions, slots, freqs, q_norm_w, k_norm_w, norm_v, k_is_v, eps, M, nh, nkv,
                           hd, block_size):
    """``kv_layer``: a (possibly strided) view [blocks, 2, nkv, block_size, hd] whose last three dims are packed."""
    _ck(load().zse_headnorm_rope_kv_write(_p(qkv), qkv.stride(0), _p(kv_layer), kv_layer.stride(0), kv_layer.stride(1),
                                          _p(positions), _p(slots), _p(freqs), _p(q_norm_w), _p(k_norm_w),
                                          int(norm_v), int(k_is_v), float(eps), M, nh, nkv, hd, block_size,
                                          _stream()), "headnorm_rope_kv_write")


def attn_generic(q, ldq, kv_layer, block_tables, seq_lens, cu_q, q_pos0, num_seqs, out, ldo, T, nh, nkv, hd,
                 block_size, scale, softcap=0.0, window=0):
    _ck(load().zse_attn_generic(_p(q), ldq, _p(kv_layer), kv_layer.stride(0), kv_layer.stride(1), _p(block_tables),
                                block_tables.stride(0), _p(seq_lens), _p(cu_q), _p(q_pos0), num_seqs, _p(out), ldo, T,
                                nh, nkv, hd, block_size, float(scale), float(softcap), int(window), _stream()),
        "attn_generic")


def norm_add_rmsnorm(x, w_post, residual, scalar, w_next, out, M, H, eps):
    _ck(load().zse_norm_add_rmsnorm(_p(x), _p(w_post), _p(residual), _p(scalar), _p(w_next), _p(out), M, H, float(eps),
                                    _stream()), "norm_add_rmsnorm")


def softcap(x, M, V, cap):
    _ck(load().zse_softcap_f16(_p(x), x.stride(0), M, V, float(cap), _stream()), "softcap")


def swiglu(gate_up, out, M, I, gelu=False):
    _ck(load().zse_swiglu(_p(gate_up), _p(out), M, I, int(gelu), _stream()), "swiglu")


def read_probe(buf, nbytes, repeats, ctas, sink):
    """Diagnostic: ``ctas`` CTAs read ``nbytes`` of ``buf`` ``repeats`` times (csrc/elementwise.cu)."""
    _ck(load().zse_read_probe(_p(buf), nbytes, repeats, ctas, _p(sink), _stream()), "read_probe")


def bias_add(x, bias, M, N):
    _ck(load().zse_bias_add(_p(x), _p(bias), M, N, _stream()), "bias_add")


def attn_decode_scratch_floats(num_seqs, nh, hd, max_splits) -> int:
    return load().zse_attn_decode_scratch_floats(num_seqs, nh, hd, max_splits)


def attn_decode(q, ldq, kv_layer, block_tables, max_blocks, seq_lens, out, ldo, scratch, num_seqs, nh, nkv, hd,
                block_size, num_splits, scale):
    _ck(load().zse_attn_decode(_p(q), ldq, _p(kv_layer), _p(block_tables), max_blocks, _p(seq_lens), _p(out), ldo,
                               _p(scratch), num_seqs, nh, nkv, hd, block_size, num_splits, scale, _stream()),
        "attn_decode", 2 if num_splits > 1 else 1)


def attn_decode_ext(q, ldq, kv_layer, block_tables, seq_lens, out, ldo, scratch, num_seqs, nh, nkv, hd, block_size,
                    num_splits, scale, softcap=0.0, window=0):
    """``kv_layer``: a (possibly strided) view [blocks, 2, nkv, block_size, hd] whose last three dims are packed."""
    _ck(load().zse_attn_decode_ext(_p(q), ldq, _p(kv_layer), kv_layer.stride(0), kv_layer.stride(1), _p(block_tables),
                                   block_tables.stride(0), _p(seq_lens), _p(out), ldo, _p(scratch), num_seqs, nh, nkv,
                                   hd, block_size, num_splits, float(scale), float(softcap), int(window), _stream()),
        "attn_decode_ext")


def attn_prefill_ext(q, ldq, kv_layer, block_tables, cu_q, q_pos0, out, ldo, num_seqs, max_q_len, nh, nkv, hd,
                     block_size, scale, softcap=0.0, window=0):
    _ck(load().zse_attn_prefill_ext(_p(q), ldq, _p(kv_layer), kv_layer.stride(0), kv_layer.stride(1),
                                    _p(block_tables), block_tables.stride(0), _p(cu_q), _p(q_pos0), _p(out), ldo,
                                    num_seqs, max_q_len, nh, nkv, hd, block_size, float(scale), float(softcap),
                                    int(window), _stream()), "attn_prefill_ext")


def attn_prefill(q, ldq, kv_layer, block_tables, max_blocks, cu_q, q_pos0, out, ldo, num_seqs, max_q_len, nh, nkv,
                 hd, block_size, scale):
    _ck(load().zse_attn_prefill(_p(q), ldq, _p(kv_layer), _p(block_tables), max_blocks, _p(cu_q), _p(q_pos0), _p(out),
                                ldo, num_seqs, max_q_len, nh, nkv, hd, block_size, scale, _stream()), "attn_prefill")


def attn_prefill_tc(q, ldq, total_rows, kv_layer, block_tables, cu_q, q_pos0, out, ldo, num_seqs, max_q_len, nh, nkv, hd,
                    block_size, scale, status, variant=0):
    """Chunked-prefill attention on the tcgen05 tensor cores (csrc/attention_tc.cu); head_dim 128, contiguous cache."""
    _ck(load().zse_attn_prefill_tc(_p(q), ldq, total_rows, _p(kv_layer), kv_layer.shape[0], _p(block_tables),
                                   block_tables.stride(0), _p(cu_q), _p(q_pos0), _p(out), ldo, num_seqs, max_q_len, nh,
                                   nkv, hd, block_size, float(scale), int(variant), status, _stream()),
        "attn_prefill_tc")


def argmax(logits, ld, out, M, V):
    _ck(load().zse_argmax(_p(logits), ld, _p(out), M, V, _stream()), "argmax")


def sample(logits, ld, out, M, V, temperature, top_k, top_p, seeds, step):
    _ck(load().zse_sample(_p(logits), ld, _p(out), M, V, _p(temperature), _p(top_k), _p(top_p), _p(seeds), step,
                          _stream()), "sample")


def apply_repetition_penalty(logits, ld, rows, tokens, counts, n, penalty, V):
    _ck(load().zse_apply_repetition_penalty(_p(logits), ld, _p(rows), _p(tokens), _p(counts), n, _p(penalty), V,
                                            _stream()), "repetition_penalty")


def lora_shrink(x, ldx, a, ids, tmp, M, K, rank):
    _ck(load().zse_lora_shrink(_p(x), ldx, _p(a), _p(ids), _p(tmp), M, K, rank, _stream()), "lora_shrink")


def lora_apply(x, ldx, a, b, ids, scales, y, ldy, M, K, N, rank):
    _ck(load().zse_lora_apply(_p(x), ldx, _p(a), _p(b), _p(ids), _p(scales), _p(y), ldy, M, K, N, rank, _stream()),
        "lora_apply")


def lora_expand(tmp, b, ids, scales, y, ldy, M, N, rank):
    _ck(load().zse_lora_expand(_p(tmp), _p(b), _p(ids), _p(scales), _p(y), ldy, M, N, rank, _stream()), "lora_expand")


def _u64s(vals):
    return (c_uint64 * len(vals))(*[int(v) for v in vals])


def tp_ctx_create(tp, rank, m_cap, H, data_ptrs, flag_ptrs, mc_data, xchg_ptrs, xflag_ptrs) -> int:
    ctx = load().zse_tp_ctx_create(tp, rank, m_cap, H, _u64s(data_ptrs), _u64s(flag_ptrs), int(mc_data or 0),
                                   _u64s(xchg_ptrs), _u64s(xflag_ptrs))
    if not ctx:
        raise NativeError("tp_ctx_create: unsupported tensor-parallel size")
    return ctx


def tp_ctx_destroy(ctx) -> None:
    load().zse_tp_ctx_destroy(ctx)


def tp_reduce_add_rmsnorm(ctx, residual, partials, n_planes, weight, out, M, eps, slot, use_multimem, status):
    _ck(load().zse_tp_reduce_add_rmsnorm(ctx, _p(residual), _p(partials), n_planes, _p(weight), _p(out), M, eps,
                                         slot, int(use_multimem), status, _stream()), "tp_reduce_add_rmsnorm",
        (M + 511) // 512)


def tp_reduce_add_rmsnorm_emulated(ctx, residuals, partials, n_planes, weight, outs, M, eps, slot, status):
    _ck(load().zse_tp_reduce_add_rmsnorm_emulated(ctx, _u64s([t.data_ptr() for t in residuals]),
                                                  _u64s([t.data_ptr() for t in partials]), n_planes, _p(weight),
                                                  _u64s([t.data_ptr() for t in outs]), M, eps, slot, status,
                                                  _stream()), "tp_reduce_add_rmsnorm_emulated")


def tp_reduce_scatter_add_rmsnorm(ctx, residual, partials, n_planes, weight, out, M, eps, slot, use_multimem, status):
    _ck(load().zse_tp_reduce_scatter_add_rmsnorm(ctx, _p(residual), _p(partials), n_planes, _p(weight), _p(out), M, eps,
                                         slot, int(use_multimem), status, _stream()), "tp_reduce_scatter_add_rmsnorm",
        (M + 511) // 512)


def tp_reduce_scatter_add_rmsnorm_emulated(ctx, residuals, partials, n_planes, weight, outs, M, eps, slot, status):
    _ck(load().zse_tp_reduce_scatter_add_rmsnorm_emulated(ctx, _u64s([t.data_ptr() for t in residuals]),
                                                  _u64s([t.data_ptr() for t in partials]), n_planes, _p(weight),
                                                  _u64s([t.data_ptr() for t in outs]), M, eps, slot, status,
                                                  _stream()), "tp_reduce_scatter_add_rmsnorm_emulated")


def tp_ctx_set_push(ctx, push_m_cap, inbox_ptrs, mc_inbox, arrive_ptrs, mc_arrive, state_ptrs):
    _ck(load().zse_tp_ctx_set_push(ctx, push_m_cap, _u64s(inbox_ptrs), int(mc_inbox), _u64s(arrive_ptrs), int(mc_arrive),
                                   _u64s(state_ptrs)), "tp_ctx_set_push", 0)


def tp_gemm_w4_push(ctx, w_tiled, x, x_rows_cap, M, N, K, slot, use_multimem, status, rank_override=-1) -> int:
    """Row-parallel INT4 GEMM whose epilogue sends the partial rows to every rank.  Returns its CTA count."""
    rc = load().zse_tp_gemm_w4_push(ctx, _p(w_tiled), _p(x), x_rows_cap, M, N, K, slot, int(use_multimem),
                                    rank_override, status, _stream())
    if rc < 0:
        _ck(rc, "tp_gemm_w4_push")
    LAUNCHES[0] += 1
    return rc


def tp_gemm_dec_allreduce_norm(ctx, w_tiled, int8_weights, x, x_rows_cap, M, N, K, slot, use_multimem, residual,
                               norm_w, xnorm, eps, workspace, status, rank_override=-1):
    """Row-parallel projection + all-reduce + residual add + RMSNorm in one kernel (csrc/gemm_w4_dec.cu)."""
    _ck(load().zse_tp_gemm_dec_allreduce_norm(ctx, _p(w_tiled), int(int8_weights), _p(x), x_rows_cap, M, N, K, slot,
                                              int(use_multimem), rank_override, _p(residual), _p(norm_w), _p(xnorm),
                                              eps, _p(workspace), status, _stream()), "tp_gemm_dec_allreduce_norm")


def tp_ctx_set_sp(ctx, own_cap, nblk_cap, inbox_ptrs, arrive_ptrs, xg_ptrs, mc_xg, gflag_ptrs, state_ptrs):
    _ck(load().zse_tp_ctx_set_sp(ctx, own_cap, nblk_cap, _u64s(inbox_ptrs), _u64s(arrive_ptrs), _u64s(xg_ptrs),
                                 int(mc_xg), _u64s(gflag_ptrs), _u64s(state_ptrs)), "tp_ctx_set_sp", 0)


def tp_gemm_w4_scatter(ctx, w_tiled, x, x_rows_cap, M, N, K, slot, status, rank_override=-1):
    """Row-parallel INT4 GEMM whose epilogue is the reduce-scatter: each 64-row block of partial sums goes to the rank
    that owns it (csrc/gemm_w4.cu, kEpiScatterF16)."""
    _ck(load().zse_tp_gemm_w4_scatter(ctx, _p(w_tiled), _p(x), x_rows_cap, M, N, K, slot, rank_override, status,
                                      _stream()), "tp_gemm_w4_scatter")


def tp_gemm_w4_gathered(ctx, w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, k_split, status,
                        rank_override=-1):
    """zse_gemm_w4 on the gathered activation buffer: the activation producer waits for the row blocks of its token
    tile to arrive from their owners before it loads them (the all-gather's receiving side)."""
    _ck(load().zse_tp_gemm_w4_gathered(ctx, _p(w_tiled), _p(x), x_rows_cap, _p(bias), _p(out), M, N, K, ldo, epilogue,
                                       k_split, rank_override, status, _stream()), "tp_gemm_w4_gathered")


def tp_sp_sum_norm_gather(ctx, residual, weight, M, eps, slot, use_multimem, status):
    _ck(load().zse_tp_sp_sum_norm_gather(ctx, _p(residual), _p(weight), M, eps, slot, int(use_multimem), status,
                                         _stream()), "tp_sp_sum_norm_gather")


def tp_sp_sum_norm_gather_emulated(ctx, residuals, weight, M, eps, slot, status):
    _ck(load().zse_tp_sp_sum_norm_gather_emulated(ctx, _u64s([t.data_ptr() for t in residuals]), _p(weight), M, eps,
                                                  slot, status, _stream()), "tp_sp_sum_norm_gather_emulated")


def tp_sp_wait(ctx, M, status, rank_override=-1):
    _ck(load().zse_tp_sp_wait(ctx, M, rank_override, status, _stream()), "tp_sp_wait")


def tp_sum_add_rmsnorm(ctx, residual, weight, out, M, eps, slot, expected_add, status):
    _ck(load().zse_tp_sum_add_rmsnorm(ctx, _p(residual), _p(weight), _p(out), M, eps, slot, expected_add, status,
                                      _stream()), "tp_sum_add_rmsnorm")


def tp_sum_add_rmsnorm_emulated(ctx, residuals, weight, outs, M, eps, slot, expected_add, status):
    _ck(load().zse_tp_sum_add_rmsnorm_emulated(ctx, _u64s([t.data_ptr() for t in residuals]), _p(weight),
                                               _u64s([t.data_ptr() for t in outs]), M, eps, slot, expected_add,
                                               status, _stream()), "tp_sum_add_rmsnorm_emulated")


def tp_ctx_set_gather(ctx, rows_cap, width, buf_ptrs, flag_ptrs):
    _ck(load().zse_tp_ctx_set_gather(ctx, rows_cap, width, _u64s(buf_ptrs), _u64s(flag_ptrs)), "tp_ctx_set_gather", 0)


def tp_gather_rows(ctx, logits, ld, M, slot, status):
    """All-gather of vocabulary-sharded logits rows into this rank's symmetric buffer (csrc/comm.cu)."""
    _ck(load().zse_tp_gather_rows(ctx, _p(logits), ld, M, slot, status, _stream()), "tp_gather_rows")


def tp_gather_rows_emulated(ctx, logits, ld, M, slot, status):
    _ck(load().zse_tp_gather_rows_emulated(ctx, _u64s([t.data_ptr() for t in logits]), ld, M, slot, status, _stream()),
        "tp_gather_rows_emulated")


def tp_argmax(ctx, logits, ld, out, M, V_local, vocab_stride, slot, status):
    _ck(load().zse_tp_argmax(ctx, _p(logits), ld, _p(out), M, V_local, vocab_stride, slot, status, _stream()),
        "tp_argmax")


def tp_argmax_emulated(ctx, logits, ld, outs, M, V_local, vocab_stride, slot, status):
    _ck(load().zse_tp_argmax_emulated(ctx, _u64s([t.data_ptr() for t in logits]), ld,
                                      _u64s([t.data_ptr() for t in outs]), M, V_local, vocab_stride, slot,
                                      status, _stream()), "tp_argmax_emulated")


def device_info() -> dict:
    sm, maj, mnr, tot, free = c_int(), c_int(), c_int(), c_int64(), c_int64()
    _ck(load().zse_device_info(sm, maj, mnr, tot, free), "device_info", 0)
    return {"sm_count": sm.value, "cc": (maj.value, mnr.value), "total_mem": tot.value, "free_mem": free.value}


def gemm_w4_set_mode(mode: int) -> None:
    """Tuning hook for the INT4 GEMM: 0 = the planner picks the CTA shape, 1 = wide CTAs only, 2 = narrow CTAs (two per
    SM) wherever they are allowed."""
    load().zse_gemm_w4_set_mode(int(mode))


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch between the kernels of a step (on by default, ``ZSE_PDL=0`` switches it off)."""
    load().zse_set_pdl(1 if on else 0)


def pdl_enabled() -> bool:
    return bool(load().zse_get_pdl())


def build_info() -> str:
    return load().zse_build_info().decode()

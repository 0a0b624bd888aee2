"""Binding of the native step driver (``csrc/step.cu``): one C call launches every kernel of a decoder pass.

``NativeStep`` mirrors the ``ZseStepModel`` / ``ZseStepBuffers`` structs of ``csrc/step.h`` with ctypes, fills them
from a loaded ``DecoderModel`` and its ``StepBuffers`` and keeps the arrays alive.  The driver covers the
single-GPU path without adapters; ``DecoderModel.forward`` keeps its Python wiring for everything else (tensor
parallelism needs host logic between kernels, LoRA patches the projections).  ``ZSE_NATIVE_STEP=0`` switches the
driver off.  Counterpart in the reference: the embedded C launcher ``fast_decode_m1``
(zse-engine/zse_engine/orchestrator/fast_dispatch.py:341-609), which is disabled there.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_int32, c_int64, c_void_p
from typing import Optional

import torch

from ..ops import native
from ..utils import env

KIND = {"w4t": 0, "f16": 1}


class _Linear(Structure):
    _fields_ = [("kind", c_int32), ("N", c_int32), ("K", c_int32), ("reserved", c_int32), ("data", c_void_p),
                ("bias", c_void_p)]


class _Layer(Structure):
    _fields_ = [("qkv", _Linear), ("o", _Linear), ("gate_up", _Linear), ("down", _Linear), ("ln1", c_void_p),
                ("ln2", c_void_p)]


class _Model(Structure):
    _fields_ = [(n, c_int32) for n in ("num_layers", "hidden", "num_heads", "num_kv_heads", "head_dim", "inter",
                                       "vocab_rows", "rotary_dim", "sm_count", "attn_tc")] + \
               [(n, c_float) for n in ("eps", "scale", "embed_scale", "reserved_f")] + \
               [("embed", c_void_p), ("final_norm", c_void_p), ("inv_freq", c_void_p), ("lm_head", _Linear),
                ("layers", POINTER(_Layer)), ("rope_table", c_void_p), ("max_position", c_int32),
                ("dec_mode", c_int32)]


class _Buffers(Structure):
    _fields_ = [(n, c_int32) for n in ("max_tokens", "max_blocks", "qkv_plane_rows", "qkv_max_planes", "max_planes",
                                       "logits_rows_cap", "logits_ld", "reserved")] + \
               [(n, c_void_p) for n in ("ids", "positions", "slots", "block_tables", "seq_lens", "cu_q", "q_pos0",
                                        "logit_rows", "residual", "xnorm", "qkv", "attn_out", "qkv_planes", "act",
                                        "gate_up_tmp", "partials", "xsel", "logits", "attn_scratch", "status",
                                        "dec_ws", "norm_ctx")]


def _linear(w) -> _Linear:
    return _Linear(KIND[w.kind], w.N, w.K, 0, w.data.data_ptr(), None if w.bias is None else w.bias.data_ptr())


def enabled() -> bool:
    return env.flag("ZSE_NATIVE_STEP")


class NativeStep:
    """The structs for one (model, step buffers) pair."""

    def __init__(self, model, buffers):
        lib = native.load()
        lib.zse_step_supported.restype = c_int
        lib.zse_step_supported.argtypes = [POINTER(_Model), POINTER(_Buffers)]
        lib.zse_step_forward.restype = c_int
        lib.zse_step_forward.argtypes = [POINTER(_Model), POINTER(_Buffers), c_void_p, c_int64, c_int, c_int, c_int,
                                         c_int, c_int, c_int, c_int, c_void_p, POINTER(c_int)]
        self._lib = lib
        c, p, b = model.config, model.plan, buffers
        kinds = {w.kind for L in model.layers for w in (L.qkv, L.o, L.gate_up, L.down)} | {model.lm_head.kind}
        if not kinds <= set(KIND):
            raise ValueError(f"weights of kind {sorted(kinds - set(KIND))} have no native path")
        self._layers = (_Layer * len(model.layers))()
        for i, L in enumerate(model.layers):
            self._layers[i] = _Layer(_linear(L.qkv), _linear(L.o), _linear(L.gate_up), _linear(L.down),
                                     L.ln1.data_ptr(), L.ln2.data_ptr())
        self._model = _Model(
            num_layers=len(model.layers), hidden=c.hidden_size, num_heads=p.num_heads, num_kv_heads=p.num_kv_heads,
            head_dim=c.head_dim, inter=p.inter_size, vocab_rows=model.embed.shape[0],
            rotary_dim=model.inv_freq.numel() * 2, sm_count=model.ops.sm_count,
            attn_tc=int(bool(getattr(model.ops, "attn_prefill_tc", False))), eps=c.rms_norm_eps, scale=model.scale,
            embed_scale=model.embed_scale, embed=model.embed.data_ptr(), final_norm=model.norm.data_ptr(),
            inv_freq=model.inv_freq.data_ptr(), lm_head=_linear(model.lm_head), layers=self._layers,
            rope_table=None if model.rope_table is None else model.rope_table.data_ptr(),
            max_position=0 if model.rope_table is None else model.rope_table.shape[0],
            dec_mode=int(getattr(model.ops, "dec_mode", 0)))
        dense_gate_up = any(L.gate_up.kind != "w4t" for L in model.layers)
        self._gate_up_tmp = (torch.empty(b.max_tokens, 2 * p.inter_size, dtype=torch.float16, device=model.device)
                             if dense_gate_up else None)
        ptr = lambda t: None if t is None else t.data_ptr()
        self._buffers = _Buffers(
            max_tokens=b.max_tokens, max_blocks=b.block_tables.stride(0), qkv_plane_rows=b.qkv_plane_rows,
            qkv_max_planes=b.qkv_planes.shape[0], max_planes=b.partials.shape[0], logits_rows_cap=b.xsel.shape[0],
            logits_ld=b.logits.stride(0), ids=ptr(b.ids), positions=ptr(b.positions), slots=ptr(b.slots),
            block_tables=ptr(b.block_tables), seq_lens=ptr(b.seq_lens), cu_q=ptr(b.cu_q), q_pos0=ptr(b.q_pos0),
            logit_rows=ptr(b.logit_rows), residual=ptr(b.residual), xnorm=ptr(b.xnorm), qkv=ptr(b.qkv),
            attn_out=ptr(b.attn_out), qkv_planes=ptr(b.qkv_planes), act=ptr(b.act), gate_up_tmp=ptr(self._gate_up_tmp),
            partials=ptr(b.partials), xsel=ptr(b.xsel), logits=ptr(b.logits), attn_scratch=ptr(b.attn_scratch),
            status=model.ops.status.ptr, dec_ws=model.ops.dec_ws.data_ptr() if model.ops.dec_mode else None,
            norm_ctx=model.ops.norm_ctx(model.config.hidden_size) if (model.ops.dec_mode & 8) else None)
        self._keep = (model, buffers)            # the structs hold raw pointers into these
        self._launches = c_int(0)
        if not lib.zse_step_supported(byref(self._model), byref(self._buffers)):
            raise ValueError("the native step driver does not support this model")

    def forward(self, kv: torch.Tensor, M: int, decode: bool, num_seqs: int, max_q_len: int, n_logit_rows: int,
                attn_splits: int) -> None:
        rc = self._lib.zse_step_forward(byref(self._model), byref(self._buffers), kv.data_ptr(), kv.stride(0),
                                        kv.shape[4], M, int(decode), num_seqs, max_q_len, n_logit_rows, attn_splits,
                                        torch.cuda.current_stream().cuda_stream, byref(self._launches))
        native._ck(rc, "step_forward", self._launches.value)


def try_build(model, buffers) -> Optional[NativeStep]:
    """A driver for this pair, or None when it does not apply (CPU, tensor parallelism, unsupported weights)."""
    if not enabled() or model.device.type != "cuda" or model.plan.tp_size != 1 or type(model).__name__ != "DecoderModel":
        return None
    if getattr(model, "window", 0):          # the C++ driver calls the attention entry points without a window
        return None
    try:
        return NativeStep(model, buffers)
    except (ValueError, AttributeError):
        return None
class FastDecoder:
    """The reference's handle on its C decode launcher (zse-engine/zse_engine/orchestrator/fast_dispatch.py:405-609):
    ``compile()`` once, ``setup(...)`` with the model state, then ``decode_step(...)`` per token; ``available`` says
    whether the native path can be used.  Here the launcher is the step driver of the native library:

        fd = FastDecoder()
        fd.compile()                       # loads (and if needed builds) the library
        fd.setup(model, buffers)           # a DecoderModel and its StepBuffers
        fd.decode_step(kv_slab, num_seqs)  # one decode pass over the staged batch; 0 on success

    ``FastDecoder(model, buffers)`` does the first three at once."""

    def __init__(self, model=None, buffers=None):
        self._step: Optional[NativeStep] = None
        self._compiled = False
        if model is not None:
            self.compile()
            self.setup(model, buffers)

    def compile(self) -> bool:
        try:
            native.load()
            self._compiled = True
        except Exception:
            self._compiled = False
        return self._compiled

    @property
    def available(self) -> bool:
        return self._step is not None

    def setup(self, model, buffers=None, *_, **__) -> bool:
        """``model`` / ``buffers`` as ``ModelRunner`` holds them (``runner.model``, ``runner.buf``).  Models the driver
        does not cover (CPU, tensor parallelism, adapters, sliding windows) leave ``available`` False."""
        self._step = try_build(model, buffers) if (self._compiled and buffers is not None) else None
        return self.available

    def decode_step(self, kv: "torch.Tensor", num_seqs: int, attn_splits: int = 1) -> int:
        """One decode pass for the ``num_seqs`` rows staged in the step buffers; 0 on success, -1 when the native path
        is not available (the caller then uses ``DecoderModel.forward``)."""
        if self._step is None:
            return -1
        self._step.forward(kv, num_seqs, True, num_seqs, 1, num_seqs, attn_splits)
        return 0

    def forward(self, *args, **kwargs) -> None:
        if self._step is None:
            raise RuntimeError("the native step driver is not available for this model")
        self._step.forward(*args, **kwargs)

"""The op set the decoder is written against, with two implementations.

``CudaOps``  - the hand-written sm_100a kernels in ``libzse_b200.so`` (fails loudly when the library is missing).
``TorchOps`` - ``ops.reference`` on any device; runs the engine on CPU-only machines and serves as the oracle.

Both work in place on caller-owned buffers so that a step allocates nothing and can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from . import reference as ref

EPI_F16, EPI_SWIGLU, EPI_PARTIAL = 0, 1, 2


@dataclass
class LinearWeight:
    """One (possibly fused / sharded) linear layer ready for the device."""
    kind: str                  # "w4t" tiled INT4 | "w8t" tiled INT8 | "f16" dense fp16 | "ref" fp32 (TorchOps)
    N: int                     # output rows as the kernel sees them (gate+up counted together for swiglu)
    K: int
    data: torch.Tensor
    bias: Optional[torch.Tensor] = None
    swiglu: bool = False       # rows are gate/up interleaved in 64-row halves (w4t) or [gate; up] stacked (f16/ref)
    nbytes: int = 0


def _np_to_dev(a: np.ndarray, device) -> torch.Tensor:
    """Host array -> tensor on ``device``.  Arrays that view a read-only file mapping are copied on the CPU path so
    the tensor never aliases the mapping."""
    if isinstance(a, torch.Tensor):
        return a.to(device)
    a = np.ascontiguousarray(a)
    if torch.device(device).type == "cpu" or not a.flags.writeable:
        a = np.array(a, copy=True)
    return torch.from_numpy(a).to(device, non_blocking=False)


np_to_dev = _np_to_dev


class TorchOps:
    name = "torch"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.status = None

    # ---- weights --------------------------------------------------------------------------------------
    def make_linear(self, parts, K: int, group_size: int, bias=None, swiglu: bool = False) -> LinearWeight:
        """``parts``: list of dicts {dtype, data(np), scales(np), zeros(np), shape, row_major_group_ok}; rows are
        concatenated in order (q,k,v or gate,up)."""
        ws = []
        for p in parts:
            ws.append(_dense_f32(p, group_size, self.device))
        w = torch.cat(ws, dim=0) if len(ws) > 1 else ws[0]
        b = None if bias is None else _np_to_dev(bias, self.device)
        return LinearWeight("ref", w.shape[0], K, w, b, swiglu, w.numel() * 4)

    def check(self):
        pass

    # ---- ops ------------------------------------------------------------------------------------------
    def linear(self, w: LinearWeight, x, M, out, x_cap=None, gather=None):
        out[:M, : w.N] = ref.linear(x[:M], w.data, w.bias)

    def linear_swiglu(self, w: LinearWeight, x, M, out, x_cap=None, gelu=False, gather=None):
        y = x[:M].float() @ w.data.T
        half = w.N // 2
        out[:M, :half] = ref.swiglu(y[:, :half], y[:, half:], gelu)

    def linear_partial(self, w: LinearWeight, x, M, partials, k_split=1, x_cap=None) -> int:
        # planes are laid out [plane][M rows][N] with the *actual* M as the row count, like the CUDA kernels do
        partials.view(-1)[: M * w.N].view(M, w.N).copy_(x[:M].float() @ w.data.T)
        return 1

    def embedding(self, table, ids, out, M, scale=1.0):
        out[:M] = table[ids[:M].long()].float() * scale

    def add_rmsnorm(self, residual, partials, n_partials, add_f16, weight, out, M, eps):
        H = residual.shape[1]
        if n_partials:
            residual[:M] += partials.view(-1)[: n_partials * M * H].view(n_partials, M, H).sum(0)
        if add_f16 is not None:
            residual[:M] += add_f16[:M].float()
        if out is not None:
            out[:M] = ref.rmsnorm(residual[:M], weight, eps)

    def qkv_rope_fused_ok(self, w: LinearWeight, M: int, hd: int, kv_layer) -> bool:
        """Whether ``qkv_rope_fused`` takes this pass (the torch implementation never does: it has the unfused ops)."""
        return False

    def residual_norm_fused_ok(self, w: LinearWeight, M: int, H: int) -> bool:
        """Whether ``linear_residual_norm`` (projection + residual add + RMSNorm in one kernel) takes this layer."""
        return False

    def rope_kv_write(self, qkv, kv_layer, positions, slots, inv_freq, M, nh, nkv, hd, block_size, planes=None,
                      n_planes=0, bias=None):
        if planes is not None:
            ld = qkv.shape[1]
            full = planes.view(-1)[: n_planes * M * ld].view(n_planes, M, ld).sum(0)
            if bias is not None:
                full = full + bias.float()
            qkv[:M] = full.clamp(-65504, 65504).to(qkv.dtype)
        ref.rope_kv_write(qkv[:M], kv_layer, positions[:M], slots[:M], inv_freq, nh, nkv, hd, block_size)

    def attn_decode(self, qkv, kv_layer, block_tables, seq_lens, out, S, nh, nkv, hd, block_size, scale, scratch=None,
                    num_splits=1, softcap=0.0, window=0):
        out[:S, : nh * hd] = ref.attn_decode(qkv[:S, : nh * hd], kv_layer, block_tables[:S], seq_lens[:S], nh, nkv, hd,
                                             block_size, scale, softcap, window)

    def attn_prefill(self, qkv, kv_layer, block_tables, cu_q, q_pos0, out, num_seqs, total_q, max_q_len, nh, nkv, hd,
                     block_size, scale, softcap=0.0, window=0):
        out[:total_q, : nh * hd] = ref.attn_prefill(qkv[:total_q, : nh * hd], kv_layer, block_tables[:num_seqs],
                                                    cu_q[: num_seqs + 1], q_pos0[:num_seqs], nh, nkv, hd, block_size,
                                                    scale, softcap, window)

    # ---- Gemma-family ops ---------------------------------------------------------------------------
    def headnorm_rope_kv_write(self, qkv, kv_layer, positions, slots, freqs, q_norm_w, k_norm_w, norm_v, k_is_v, eps,
                               M, nh, nkv, hd, block_size):
        ref.headnorm_rope_kv_write(qkv[:M], kv_layer, positions[:M], slots[:M], freqs, q_norm_w, k_norm_w, norm_v,
                                   k_is_v, eps, nh, nkv, hd, block_size)

    def norm_add_rmsnorm(self, x, w_post, residual, scalar, w_next, out, M, eps):
        y = ref.norm_add_rmsnorm(x[:M], w_post, residual[:M], scalar, w_next, eps)
        if out is not None and y is not None:
            out[:M] = y

    def glu(self, gate_up, out, M, I, gelu=False):
        out[:M, :I] = ref.swiglu(gate_up[:M, :I], gate_up[:M, I: 2 * I], gelu)

    def softcap(self, logits, M, cap):
        logits[:M] = ref.softcap(logits[:M], cap)

    def argmax(self, logits, out, M):
        out[:M] = logits[:M].float().argmax(dim=-1).to(out.dtype)

    def sample(self, logits, out, M, temperature, top_k, top_p, seeds, step):
        for r in range(M):
            t = float(temperature[r])
            if t <= 0 or int(top_k[r]) == 1:
                out[r] = int(logits[r].float().argmax())
                continue
            p = ref.filtered_probs(logits[r], t, int(top_k[r]), float(top_p[r]))
            # the row's own seed and nothing about its place in the batch (same rule as the CUDA kernel)
            g = torch.Generator(device="cpu").manual_seed((int(seeds[r]) * 1000003 + int(step) * 7919) % (2 ** 63))
            out[r] = int(torch.multinomial(p.cpu(), 1, generator=g))

    def apply_repetition_penalty(self, logits, rows, tokens, counts, n, penalty):
        for i in range(n):
            r, t, c = int(rows[i]), int(tokens[i]), int(counts[i])
            pen = float(penalty[r])
            if c > 0 and pen != 1.0:
                f = pen ** (1.0 + float(np.log2(c)))
                v = float(logits[r, t])
                logits[r, t] = v / f if v > 0 else v * f

    def lora_apply(self, x, a_table, b_table, ids, scales, y, M, K, N, rank, tmp=None, y_col0=0):
        for t in range(M):
            a = int(ids[t])
            if a >= 0:
                d = ref.lora_delta(x[t: t + 1, :K], a_table[a], b_table[a], float(scales[a]))
                y[t, y_col0: y_col0 + N] = (y[t, y_col0: y_col0 + N].float() + d[0]).clamp(-65504, 65504).to(y.dtype)


def _dense_f32(p: dict, group_size: int, device) -> torch.Tensor:
    shape = tuple(p["shape"])
    if p["dtype"] == "float16":
        return _np_to_dev(p["data"], device).reshape(shape).float()
    if p["dtype"] == "int8":
        return ref.dequant_int8(_np_to_dev(p["data"], device), _np_to_dev(p["scales"], device), shape, group_size)
    if "flat_data" in p:   # a column slice of a tensor whose flat groups straddle rows: dequantise whole, slice
        full = ref.dequant_int4(_np_to_dev(p["flat_data"], device), _np_to_dev(p["flat_scales"], device),
                                _np_to_dev(p["flat_zeros"], device), p["flat_shape"], group_size)
        (r0, r1), (c0, c1) = p["rows"], p["cols"]
        return full[r0:r1, c0:c1].contiguous()
    return ref.dequant_int4(_np_to_dev(p["data"], device), _np_to_dev(p["scales"], device),
                            _np_to_dev(p["zeros"], device), shape, group_size)


class CudaOps(TorchOps):
    name = "cuda"

    def __init__(self, device="cuda"):
        from . import native
        if not torch.cuda.is_available():
            raise RuntimeError("CudaOps needs a CUDA device")
        self.n = native
        native.load(build_if_missing=True)
        self.device = torch.device(device)
        self.status = native.Status(self.device)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # decode-sized passes (<= 64 tokens) of the INT4 layers: bit 0 = gate/up + SwiGLU, bit 1 = fused QKV + bias +
        # RoPE + KV-cache write, bit 2 = every other INT4 linear, through the persistent kernel (csrc/gemm_w4_dec.cu)
        from ..utils import env
        self.dec_mode = env.integer("ZSE_W4_DEC")
        self._dec_ws = None
        # INT8 weights stay INT8 on the device (ZSE_W8_RESIDENT=0: expanded to fp16 at load, twice the memory)
        self.int8_resident = env.flag("ZSE_W8_RESIDENT")
        self._w8_scratch = None
        self._norm_ctx = None
        self.attn_prefill_tc = env.flag("ZSE_ATTN_PREFILL_TC")

    def _w8_dense(self, w: "LinearWeight") -> torch.Tensor:
        """fp16 [N, K] view of an INT8 weight in the scratch buffer that all layers share (rows: gate then up for a
        fused gate/up tensor).  Valid until the next call."""
        need = w.N * w.K
        if self._w8_scratch is None or self._w8_scratch.numel() < need:
            self._w8_scratch = torch.empty(need, dtype=torch.float16, device=self.device)
        dense = self._w8_scratch[:need].view(w.N, w.K)
        self.n.dequant_w8_tiled(w.data, dense, w.N, w.K, w.N // 2 if w.swiglu else 0)
        return dense

    def norm_ctx(self, H: int) -> int:
        """A one-rank tensor-parallel context: lets a single GPU use the kernel that does a row-parallel projection,
        the residual add and the next RMSNorm in one launch (there is simply no peer to exchange with)."""
        if self._norm_ctx is None or self._norm_ctx[1] != H:
            z = lambda n, dt: torch.zeros(n, dtype=dt, device=self.device)
            keep = [z(8, torch.float16), z(8, torch.int32), z(8, torch.int64), z(8, torch.int32),
                    z(2 * 64 * H, torch.float16), z(2, torch.int32), z(4, torch.int32)]
            p = [t.data_ptr() for t in keep]
            ctx = self.n.tp_ctx_create(1, 0, 64, H, [p[0]], [p[1]], 0, [p[2]], [p[3]])
            self.n.tp_ctx_set_push(ctx, 64, [p[4]], 0, [p[5]], 0, [p[6]])
            self._norm_ctx = (ctx, H, keep)
        return self._norm_ctx[0]

    def residual_norm_fused_ok(self, w, M: int, H: int) -> bool:
        return bool((self.dec_mode & 8) and w.kind in ("w4t", "w8t") and M <= 64 and w.N == H and w.bias is None
                    and self.n.gemm_w4_dec_supported(M, w.N, w.K, 4)
                    and self.n.gemm_w4_dec_plan(w.N, w.K, 4, self.sm_count)[1] > 0)

    def linear_residual_norm(self, w, x, M: int, residual, norm_w, out, eps: float, slot: int) -> None:
        """residual += x W^T; out = RMSNorm(residual) * norm_w, one kernel (decode-sized passes, single GPU)."""
        self.n.tp_gemm_dec_allreduce_norm(self.norm_ctx(w.N), w.data, w.kind == "w8t", x, x.shape[0], M, w.N, w.K,
                                          slot & 1, False, residual, norm_w, out, float(eps), self.dec_ws,
                                          self.status.ptr)

    @property
    def dec_ws(self) -> torch.Tensor:
        if self._dec_ws is None:
            self._dec_ws = self.n.gemm_w4_dec_workspace(self.device, self.sm_count)
        return self._dec_ws

    def check(self):
        self.status.check()

    # ---- weights --------------------------------------------------------------------------------------
    def make_linear(self, parts, K: int, group_size: int, bias=None, swiglu: bool = False) -> LinearWeight:
        n = self.n
        b = None if bias is None else _np_to_dev(bias, self.device)
        tiled_ok = (K % 128 == 0 and group_size == 128
                    and all(p["dtype"] == "int4" and "flat_data" not in p for p in parts))
        if swiglu and tiled_ok:
            tiled_ok = len(parts) == 2 and parts[0]["shape"][0] == parts[1]["shape"][0]
        if tiled_ok:
            packed = torch.cat([_np_to_dev(p["data"], self.device).reshape(p["shape"][0], K // 2) for p in parts])
            scales = torch.cat([_np_to_dev(p["scales"], self.device).reshape(p["shape"][0], K // 128) for p in parts])
            zeros = torch.cat([_np_to_dev(p["zeros"], self.device).reshape(p["shape"][0], K // 128) for p in parts])
            N = packed.shape[0]
            inter = N // 2 if swiglu else 0
            n_tiles = (inter + 63) // 64 if swiglu else (N + 127) // 128
            out = torch.empty(n_tiles * (K // 128) * 8704, dtype=torch.uint8, device=self.device)
            n.repack_w4(packed, scales, zeros, out, N, K, inter)
            return LinearWeight("w4t", N, K, out, b, swiglu, out.numel())
        # INT8 (symmetric groups of 128): kept 8 bits wide, tiled for the decode kernel.  Passes of more than 64 tokens
        # expand the tensor into a scratch buffer that all layers share and run the fp16 GEMM on it.
        w8_ok = (K % 128 == 0 and group_size == 128 and all(p["dtype"] == "int8" and "scales" in p for p in parts)
                 and self.int8_resident)
        if swiglu and w8_ok:
            w8_ok = len(parts) == 2 and parts[0]["shape"][0] == parts[1]["shape"][0]
        if w8_ok:
            q = torch.cat([_np_to_dev(p["data"], self.device).reshape(p["shape"][0], K) for p in parts]).contiguous()
            sc = torch.cat([_np_to_dev(p["scales"], self.device).reshape(p["shape"][0], K // 128)
                            for p in parts]).contiguous()
            N = q.shape[0]
            inter = N // 2 if swiglu else 0
            n_tiles = (inter + 63) // 64 if swiglu else (N + 127) // 128
            out = torch.empty(n_tiles * (K // 128) * 16640, dtype=torch.uint8, device=self.device)
            n.repack_w8(q.view(torch.int8) if q.dtype != torch.int8 else q, sc, out, N, K, inter)
            return LinearWeight("w8t", N, K, out, b, swiglu, out.numel())
        # anything else becomes dense fp16 for the SS-mode kernel
        if all(p["dtype"] == "float16" for p in parts):      # already fp16: one copy, no fp32 round trip
            ws = [_np_to_dev(p["data"], self.device).reshape(tuple(p["shape"])) for p in parts]
            w = torch.cat(ws, dim=0) if len(ws) > 1 else ws[0].clone(memory_format=torch.contiguous_format)
            return LinearWeight("f16", w.shape[0], K, w, b, swiglu, w.numel() * 2)
        ws = [_dense_f32(p, group_size, self.device).to(torch.float16) for p in parts]
        w = torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0].contiguous()
        return LinearWeight("f16", w.shape[0], K, w, b, swiglu, w.numel() * 2)

    # ---- ops ------------------------------------------------------------------------------------------
    def linear(self, w, x, M, out, x_cap=None, gather=None):
        """``gather``: a tensor-parallel context whose gathered activation buffer ``x`` is - the GEMM then waits, tile
        by tile, for the rows to arrive from the ranks that own them (INT4 weights, more than 64 rows)."""
        cap = x.shape[0] if x_cap is None else x_cap
        if gather is not None:
            if w.kind != "w4t" or M <= 64:
                raise NotImplementedError("a gathered activation buffer is read by the wide INT4 GEMM only")
            self.n.tp_gemm_w4_gathered(gather, w.data, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, 0,
                                       self.status.ptr)
        elif w.kind == "w8t":
            if M <= 64 and out.stride(0) % 8 == 0 and self.n.gemm_w4_dec_supported(M, w.N, w.K, EPI_F16):
                self.n.gemm_w8_dec(w.data, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, self.dec_ws,
                                   self.status.ptr)
            else:
                self.n.gemm_f16(self._w8_dense(w), w.N, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, 1,
                                self.status.ptr)
        elif (w.kind == "w4t" and (self.dec_mode & 4) and M <= 64 and out.stride(0) % 8 == 0
                and self.n.gemm_w4_dec_supported(M, w.N, w.K, EPI_F16)):
            self.n.gemm_w4_dec(w.data, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, self.dec_ws,
                               self.status.ptr)
        elif w.kind == "w4t":
            self.n.gemm_w4(w.data, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, 0, self.status.ptr)
        else:
            self.n.gemm_f16(w.data, w.N, x, cap, w.bias, out, M, w.N, w.K, out.stride(0), EPI_F16, 1, self.status.ptr)

    def linear_swiglu(self, w, x, M, out, x_cap=None, gelu=False, tmp=None, gather=None):
        cap = x.shape[0] if x_cap is None else x_cap
        if gather is not None:
            if w.kind != "w4t" or M <= 64 or gelu:
                raise NotImplementedError("a gathered activation buffer is read by the wide INT4 GEMM only")
            self.n.tp_gemm_w4_gathered(gather, w.data, x, cap, None, out, M, w.N, w.K, out.stride(0), EPI_SWIGLU, 0,
                                       self.status.ptr)
        elif w.kind == "w8t":
            if (not gelu and M <= 64 and out.stride(0) % 8 == 0
                    and self.n.gemm_w4_dec_supported(M, w.N, w.K, EPI_SWIGLU)):
                self.n.gemm_w8_dec(w.data, x, cap, None, out, M, w.N, w.K, out.stride(0), EPI_SWIGLU, self.dec_ws,
                                   self.status.ptr)
            else:
                gu = torch.empty(M, w.N, dtype=torch.float16, device=self.device) if tmp is None else tmp
                self.n.gemm_f16(self._w8_dense(w), w.N, x, cap, None, gu, M, w.N, w.K, gu.stride(0), EPI_F16, 1,
                                self.status.ptr)
                self.n.swiglu(gu, out, M, w.N // 2, gelu)
        elif (w.kind == "w4t" and not gelu and (self.dec_mode & 1) and M <= 64 and out.stride(0) % 8 == 0
                and self.n.gemm_w4_dec_supported(M, w.N, w.K, EPI_SWIGLU)):
            self.n.gemm_w4_dec(w.data, x, cap, None, out, M, w.N, w.K, out.stride(0), EPI_SWIGLU, self.dec_ws,
                               self.status.ptr)
        elif w.kind == "w4t" and not gelu:
            self.n.gemm_w4(w.data, x, cap, None, out, M, w.N, w.K, out.stride(0), EPI_SWIGLU, 0, self.status.ptr)
        else:
            if w.kind == "w4t":
                raise NotImplementedError("GeGLU needs the dense path")
            gu = torch.empty(M, w.N, dtype=torch.float16, device=self.device) if tmp is None else tmp
            self.n.gemm_f16(w.data, w.N, x, cap, None, gu, M, w.N, w.K, gu.stride(0), EPI_F16, 1, self.status.ptr)
            self.n.swiglu(gu, out, M, w.N // 2, gelu)

    def pick_k_split(self, w, M) -> int:
        """fp16 kernel only (the INT4 kernel plans its own on-chip split): planes so that the grid fills the GPU."""
        n_tiles = (w.N + 127) // 128
        nt = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
        ctas = n_tiles * ((M + nt - 1) // nt)
        want = max(1, (self.sm_count * (2 if nt <= 64 else 1)) // max(1, ctas))
        return max(1, min(want, 8, (w.K // 64) // 4 or 1))

    def linear_partial(self, w, x, M, partials, k_split=None, x_cap=None) -> int:
        """fp32 result planes in ``partials`` [planes, M, N] (plane stride M*N); returns how many planes were written.
        The consumer (``add_rmsnorm`` / the tensor-parallel reduce) adds them in plane order."""
        cap = x.shape[0] if x_cap is None else x_cap
        if w.kind == "w8t":
            if M <= 64 and self.n.gemm_w4_dec_supported(M, w.N, w.K, EPI_PARTIAL):
                # one fp32 plane (row stride N): the decode kernel adds its K splits on chip
                self.n.gemm_w8_dec(w.data, x, cap, None, partials, M, w.N, w.K, w.N, EPI_PARTIAL, self.dec_ws,
                                   self.status.ptr)
                return 1
            dense = self._w8_dense(w)
            dw = LinearWeight("f16", w.N, w.K, dense, None, False, 0)
            return self.linear_partial(dw, x, M, partials, k_split, x_cap)
        if w.kind == "w4t":
            ks = 0 if k_split is None else min(k_split, partials.shape[0])
            planes = self.n.gemm_w4_splits(M, w.N, w.K, ks)
            if planes > partials.shape[0]:
                ks = partials.shape[0]
                planes = self.n.gemm_w4_splits(M, w.N, w.K, ks)
            self.n.gemm_w4(w.data, x, cap, None, partials, M, w.N, w.K, partials.stride(1), EPI_PARTIAL, ks,
                           self.status.ptr)
            return planes
        ks = self.pick_k_split(w, M) if k_split is None else k_split
        ks = min(ks, partials.shape[0])
        planes = self.n.gemm_f16_splits(M, w.N, w.K, ks)
        self.n.gemm_f16(w.data, w.N, x, cap, None, partials, M, w.N, w.K, partials.stride(1), EPI_PARTIAL, ks,
                        self.status.ptr)
        return planes

    def embedding(self, table, ids, out, M, scale=1.0):
        self.n.embedding(table, ids, out, M, table.shape[1], table.shape[0], float(scale), self.status.ptr)

    def add_rmsnorm(self, residual, partials, n_partials, add_f16, weight, out, M, eps):
        # partial planes are laid out [plane][M rows][H]: the plane stride the kernel assumes is M*H
        self.n.add_rmsnorm(residual, partials, n_partials, add_f16, weight, out, M, residual.shape[1], float(eps))

    def rope_kv_write(self, qkv, kv_layer, positions, slots, inv_freq, M, nh, nkv, hd, block_size, planes=None,
                      n_planes=0, bias=None):
        self.n.rope_kv_write(qkv, kv_layer, positions, slots, inv_freq, M, nh, nkv, hd, inv_freq.numel() * 2,
                             block_size, planes, n_planes, bias)

    def qkv_rope_fused_ok(self, w, M, hd, kv_layer) -> bool:
        ok_kind = w.kind == "w8t" or (w.kind == "w4t" and (self.dec_mode & 2))
        return bool(ok_kind and M <= 64 and hd == 128 and kv_layer.is_contiguous()
                    and self.n.gemm_w4_dec_supported(M, w.N, w.K, 3))

    def qkv_rope_fused(self, w, x, M, qkv, kv_layer, positions, slots, cos_sin, nh, nkv, block_size, x_cap=None):
        """One kernel: fused QKV projection + bias + rotate-half RoPE + K/V rows into the paged cache; ``qkv`` gets
        the rotated q heads.  head_dim 128, full rotary, ``cos_sin`` [max_position, 64, 2] fp32."""
        cap = x.shape[0] if x_cap is None else x_cap
        fn = self.n.gemm_w8_dec_qkv_rope if w.kind == "w8t" else self.n.gemm_w4_dec_qkv_rope
        fn(w.data, x, cap, w.bias, qkv, qkv.stride(0), M, w.K, nh, nkv, kv_layer, block_size, positions, slots, cos_sin,
           cos_sin.shape[0], self.dec_ws, self.status.ptr)

    @staticmethod
    def _tensor_core_attention(kv_layer, hd, nh, nkv, block_size) -> bool:
        """The tensor-core attention kernels cover head_dim 64/128/256 with up to 16 query heads per kv head; other
        shapes (Gemma-4 global layers with head_dim 512) take the CUDA-core kernel."""
        return (hd in (64, 128, 256) and nh // nkv <= 16 and block_size % 16 == 0 and kv_layer.stride(0) % 8 == 0
                and kv_layer.stride(1) % 8 == 0 and kv_layer.data_ptr() % 16 == 0)

    def attn_decode(self, qkv, kv_layer, block_tables, seq_lens, out, S, nh, nkv, hd, block_size, scale, scratch=None,
                    num_splits=1, softcap=0.0, window=0):
        if not self._tensor_core_attention(kv_layer, hd, nh, nkv, block_size):
            self.n.attn_generic(qkv, qkv.stride(0), kv_layer, block_tables, seq_lens, None, None, S, out,
                                out.stride(0), S, nh, nkv, hd, block_size, scale, softcap, window)
            return
        if scratch is None or scratch.numel() < S * nh * num_splits * (hd + 2):
            num_splits = 1
        self.n.attn_decode_ext(qkv, qkv.stride(0), kv_layer, block_tables, seq_lens, out, out.stride(0), scratch, S,
                               nh, nkv, hd, block_size, num_splits, scale, softcap, window)

    def attn_prefill(self, qkv, kv_layer, block_tables, cu_q, q_pos0, out, num_seqs, total_q, max_q_len, nh, nkv, hd,
                     block_size, scale, softcap=0.0, window=0):
        if not self._tensor_core_attention(kv_layer, hd, nh, nkv, block_size):
            self.n.attn_generic(qkv, qkv.stride(0), kv_layer, block_tables, None, cu_q, q_pos0, num_seqs, out,
                                out.stride(0), total_q, nh, nkv, hd, block_size, scale, softcap, window)
            return
        if (self.attn_prefill_tc and hd == 128 and softcap == 0.0 and window == 0 and kv_layer.is_contiguous()
                and kv_layer.shape[1:] == (2, nkv, block_size, hd)):
            self.n.attn_prefill_tc(qkv, qkv.stride(0), total_q, kv_layer, block_tables, cu_q, q_pos0, out,
                                   out.stride(0), num_seqs, max_q_len, nh, nkv, hd, block_size, scale,
                                   self.status.ptr)
            return
        self.n.attn_prefill_ext(qkv, qkv.stride(0), kv_layer, block_tables, cu_q, q_pos0, out, out.stride(0),
                                num_seqs, max_q_len, nh, nkv, hd, block_size, scale, softcap, window)

    def headnorm_rope_kv_write(self, qkv, kv_layer, positions, slots, freqs, q_norm_w, k_norm_w, norm_v, k_is_v, eps,
                               M, nh, nkv, hd, block_size):
        self.n.headnorm_rope_kv_write(qkv, kv_layer, positions, slots, freqs, q_norm_w, k_norm_w, norm_v, k_is_v, eps,
                                      M, nh, nkv, hd, block_size)

    def norm_add_rmsnorm(self, x, w_post, residual, scalar, w_next, out, M, eps):
        self.n.norm_add_rmsnorm(x, w_post, residual, scalar, w_next, out, M, residual.shape[1], eps)

    def glu(self, gate_up, out, M, I, gelu=False):
        self.n.swiglu(gate_up, out, M, I, gelu)

    def softcap(self, logits, M, cap):
        self.n.softcap(logits, M, logits.shape[1], cap)

    def argmax(self, logits, out, M):
        self.n.argmax(logits, logits.stride(0), out, M, logits.shape[1])

    def sample(self, logits, out, M, temperature, top_k, top_p, seeds, step):
        self.n.sample(logits, logits.stride(0), out, M, logits.shape[1], temperature, top_k, top_p, seeds, int(step))

    def apply_repetition_penalty(self, logits, rows, tokens, counts, n, penalty):
        self.n.apply_repetition_penalty(logits, logits.stride(0), rows, tokens, counts, n, penalty, logits.shape[1])

    def lora_apply(self, x, a_table, b_table, ids, scales, y, M, K, N, rank, tmp=None, y_col0=0):
        yv = y[:, y_col0:]
        if rank % 2 == 0 and rank <= 64 and K % 8 == 0 and K * 2 + 256 <= 200 * 1024:
            # one launch: the token's activation row is read once, nothing passes through global memory in between
            self.n.lora_apply(x, x.stride(0), a_table, b_table, ids, scales, yv, y.stride(0), M, K, N, rank)
            return
        if tmp is None:
            tmp = torch.empty(M, rank, dtype=torch.float32, device=self.device)
        self.n.lora_shrink(x, x.stride(0), a_table, ids, tmp, M, K, rank)
        self.n.lora_expand(tmp, b_table, ids, scales, yv, y.stride(0), M, N, rank)


def make_ops(device) -> TorchOps:
    device = torch.device(device)
    if device.type == "cuda":
        return CudaOps(device)
    return TorchOps(device)

"""Llama / Mistral / Qwen2 / Phi-3 decoder over the paged KV cache (the Gemma family lives in ``gemma.py``).

One ``DecoderModel`` lives on one device and holds this rank's shard of the weights.  ``forward`` runs a pass over
``M`` packed tokens that are already in the persistent step buffers (token ids, positions, cache slots, block
tables...), so a pass allocates nothing and can be replayed from a CUDA graph.  The same pass serves prefill,
chunked prefill, speculative verification (``mode="prefill"``: causal attention over the cache) and batched decode
(``mode="decode"``: one token per sequence).

Launch sequence per layer (tp = 1): add+RMSNorm -> fused QKV GEMM (+bias) -> RoPE + KV write -> attention ->
o_proj (split-K fp32 partials) -> add+RMSNorm (reduces the partials into the fp32 residual) -> gate/up GEMM with
SwiGLU epilogue -> down_proj (split-K partials).  Decode-sized passes (<= 64 tokens, head_dim 128) do QKV, bias,
RoPE and the cache write in ONE kernel.  That is 7-8 launches where the reference issues about 18
(zse-engine/zse_engine/orchestrator/model_runner.py:1299-1474), with an fp32 residual stream like the reference.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..format.loader import ZSELoader
from ..format.config import ModelConfig
from ..ops import reference as ref
from ..ops.backend import LinearWeight, TorchOps, make_ops, np_to_dev
from ..parallel.shard_plan import ShardPlan, make_plan

SUPPORTED_ARCHS = ("llama", "mistral", "qwen2", "phi3", "gemma2", "gemma4")


def _entry_part(loader: ZSELoader, name: str, rows=None, cols=None, mirror=None) -> dict:
    """Views of one stored tensor, optionally restricted to a row range and/or a column (K) range: numpy views of the
    file mapping, or (with ``mirror``, a DeviceMirror of the weight section) device views."""
    e = loader.weight_index.find(name)
    if e is None:
        raise KeyError(name)
    N, K = e.shape
    r0, r1 = rows if rows is not None else (0, N)
    c0, c1 = cols if cols is not None else (0, K)
    gs = e.group_size
    if mirror is not None:
        if e.dtype == "float16":
            t = mirror.view(e.data_offset, e.data_nbytes, "float16").reshape(N, K)
            return {"dtype": "float16", "data": t[r0:r1, c0:c1], "shape": (r1 - r0, c1 - c0)}
        if (e.dtype == "int4" and loader.int4_layout_of(e) == "rowmajor" and K % gs == 0 and c0 % gs == 0
                and c1 % gs == 0):
            p = mirror.view(e.data_offset, N * K // 2).reshape(N, K // 2)[r0:r1, c0 // 2: c1 // 2]
            s = mirror.view(e.scale_offset, N * (K // gs) * 2, "float16").reshape(N, K // gs)[r0:r1, c0 // gs: c1 // gs]
            z = mirror.view(e.zeros_offset, N * (K // gs) * 2, "float16").reshape(N, K // gs)[r0:r1, c0 // gs: c1 // gs]
            return {"dtype": "int4", "data": p, "scales": s, "zeros": z, "shape": (r1 - r0, c1 - c0)}
        # anything else (INT8, tiled INT4 files, groups that straddle rows) takes the host path below
    if e.dtype == "float16":
        return {"dtype": "float16", "data": loader.view_data(e)[r0:r1, c0:c1], "shape": (r1 - r0, c1 - c0)}
    if e.dtype == "int8":
        if K % gs or c0 % gs or c1 % gs:
            full = loader.get_weight_as_float(e)[r0:r1, c0:c1].astype(np.float16)
            return {"dtype": "float16", "data": full, "shape": full.shape}
        q = loader.view_data(e).reshape(N, K)[r0:r1, c0:c1]
        s = loader.view_scales(e).reshape(N, K // gs)[r0:r1, c0 // gs: c1 // gs]
        return {"dtype": "int8", "data": q, "scales": s, "shape": (r1 - r0, c1 - c0)}
    packed = loader.int4_rowmajor(e)
    if K % gs == 0 and c0 % gs == 0 and c1 % gs == 0:
        p = packed.reshape(N, K // 2)[r0:r1, c0 // 2: c1 // 2]
        s = loader.view_scales(e).reshape(N, K // gs)[r0:r1, c0 // gs: c1 // gs]
        z = loader.view_zeros(e).reshape(N, K // gs)[r0:r1, c0 // gs: c1 // gs]
        return {"dtype": "int4", "data": p, "scales": s, "zeros": z, "shape": (r1 - r0, c1 - c0)}
    # groups of the flattened tensor straddle rows: keep the whole tensor and slice after dequantisation
    return {"dtype": "int4", "flat_data": packed, "flat_scales": loader.view_scales(e),
            "flat_zeros": loader.view_zeros(e), "flat_shape": (N, K), "rows": (r0, r1), "cols": (c0, c1),
            "shape": (r1 - r0, c1 - c0)}


def _vec(loader: ZSELoader, name: str, rows=None) -> Optional[np.ndarray]:
    e = loader.weight_index.find(name)
    if e is None:
        return None
    v = loader.view_data(e).reshape(-1)
    return v if rows is None else v[rows[0]: rows[1]]


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: LinearWeight
    o: LinearWeight
    gate_up: LinearWeight
    down: LinearWeight


class StepBuffers:
    """Persistent device tensors one pass reads and writes."""

    def __init__(self, c: ModelConfig, plan: ShardPlan, device, max_tokens: int, max_seqs: int, max_blocks: int,
                 max_planes: int, logits_rows: int, attn_splits: int):
        f16, f32, i32, i64 = torch.float16, torch.float32, torch.int32, torch.int64
        H = c.hidden_size
        z = lambda *s, dt: torch.zeros(*s, dtype=dt, device=device)
        self.max_tokens, self.max_seqs, self.max_blocks = max_tokens, max_seqs, max_blocks
        self.ids = z(max_tokens, dt=i32)
        self.positions = z(max_tokens, dt=i32)
        self.slots = torch.full((max_tokens,), -1, dtype=i64, device=device)
        self.block_tables = torch.full((max_seqs, max_blocks), -1, dtype=i32, device=device)
        self.seq_lens = z(max_seqs, dt=i32)
        self.cu_q = z(max_seqs + 1, dt=i32)
        self.q_pos0 = z(max_seqs, dt=i32)
        self.logit_rows = z(logits_rows, dt=i64)
        self.residual = z(max_tokens, H, dt=f32)
        self.xnorm = z(max_tokens, H, dt=f16)
        self.qkv = z(max_tokens, plan.q_dim + 2 * plan.kv_dim, dt=f16)
        self.attn_out = z(max_tokens, plan.q_dim, dt=f16)
        # decode-sized passes take QKV as fp32 split-K planes (summed, biased and rotated by the RoPE kernel)
        self.qkv_plane_rows = min(max_tokens, 256)
        self.qkv_planes = z(8, self.qkv_plane_rows, plan.q_dim + 2 * plan.kv_dim, dt=f32)
        self.act = z(max_tokens, plan.inter_size, dt=f16)
        self.partials = z(max_planes, max_tokens, H, dt=f32)
        self.xsel = z(logits_rows, H, dt=f16)
        self.logits = z(logits_rows, plan.vocab_size, dt=f16)
        self.out_tokens = z(logits_rows, dt=i32)
        self.attn_splits = attn_splits
        self.attn_scratch = z(max(1, max_seqs * plan.num_heads * attn_splits * (c.head_dim + 2)), dt=f32)
        # sampling parameters per logits row
        self.temperature = torch.ones(logits_rows, dtype=f32, device=device)
        self.top_k = z(logits_rows, dt=i32)
        self.top_p = torch.ones(logits_rows, dtype=f32, device=device)
        self.seeds = z(logits_rows, dt=i64)
        # LoRA routing
        self.adapter_ids = torch.full((max_tokens,), -1, dtype=i32, device=device)
        self.lora_tmp = z(max_tokens, 64, dt=f32)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in vars(self).values() if isinstance(t, torch.Tensor))


class DecoderModel:
    def __init__(self, config: ModelConfig, plan: ShardPlan, ops: TorchOps):
        self.config, self.plan, self.ops = config, plan, ops
        self.device = ops.device
        self.layers: List[LayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[LinearWeight] = None
        self.inv_freq: Optional[torch.Tensor] = None
        self.scale = 1.0 / math.sqrt(config.head_dim)
        self.comm = None            # parallel.comm.TPComm when tp_size > 1
        # a uniform sliding window (Mistral, Phi-3): a token sees the last ``window`` positions, itself included; the
        # cache lets blocks that fell out of every window go, attention masks inside the oldest block that is left
        self.window = int(config.sliding_window or 0) if not config.layer_types else 0
        self.lora = None            # lora.manager.LoRAManager
        self.weight_bytes = 0
        self.load_stats: Dict[str, float] = {}
        self.embed_scale = math.sqrt(config.hidden_size) if config.embed_scale else 1.0

    # ---- loading --------------------------------------------------------------------------------------
    @classmethod
    def from_loader(cls, loader: ZSELoader, device="cpu", tp_size: int = 1, rank: int = 0, ops=None,
                    progress=None) -> "DecoderModel":
        c = loader.config
        if c.arch not in SUPPORTED_ARCHS:
            raise NotImplementedError(f"architecture '{c.arch}' has a converter but no runtime here yet "
                                      f"(supported: {', '.join(SUPPORTED_ARCHS)})")
        plan = make_plan(c, tp_size, rank)
        if c.is_gemma and cls is DecoderModel:
            from .gemma import GemmaDecoderModel
            cls = GemmaDecoderModel
        m = cls(c, plan, ops or make_ops(device))
        m._load(loader, progress)
        return m

    def _load(self, loader: ZSELoader, progress=None) -> None:
        c, p, ops, dev = self.config, self.plan, self.ops, self.device
        gs = c.quant.group_size
        has = lambda n: loader.weight_index.find(n) is not None
        to_dev = lambda a: np_to_dev(a, dev)
        mirror = None
        # the weight section goes to the device in one streamed pass (every tensor-parallel rank mirrors the section and
        # cuts its shard out on the device: the page cache serves all ranks, and a rank's shard of a row-parallel
        # projection is a column range that no contiguous read could deliver anyway)
        if dev.type == "cuda":
            from ..runtime.weight_stream import open_mirror
            mirror = open_mirror(loader, dev, self.load_stats)       # None: switched off, or failed -> per-tensor copies
        _part = lambda name, rows=None, cols=None: _entry_part(loader, name, rows, cols, mirror)
        e_embed = loader.weight_index.find("embed_tokens.weight")
        if mirror is not None and e_embed.dtype == "float16":
            self.embed = mirror.view(e_embed.data_offset, e_embed.data_nbytes, "float16").reshape(
                e_embed.shape).clone()
        else:
            self.embed = to_dev(loader.view_data(e_embed))
        self.norm = to_dev(_vec(loader, "norm.weight"))
        self.weight_bytes += self.embed.numel() * 2
        q_dim_full = c.num_heads * c.head_dim
        kv_dim_full = c.num_kv_heads * c.head_dim
        for i in range(c.num_layers):
            pre = f"layers.{i}."
            if has(pre + "self_attn.qkv_proj.weight"):     # Phi-3: [q; k; v] stacked in one tensor
                n = pre + "self_attn.qkv_proj.weight"
                qp = _part(n, rows=p.q_rows)
                kp = _part(n, rows=(q_dim_full + p.kv_rows[0], q_dim_full + p.kv_rows[1]))
                vp = _part(n, rows=(q_dim_full + kv_dim_full + p.kv_rows[0],
                                                  q_dim_full + kv_dim_full + p.kv_rows[1]))
                bias = None
            else:
                qp = _part(pre + "self_attn.q_proj.weight", rows=p.q_rows)
                kp = _part(pre + "self_attn.k_proj.weight", rows=p.kv_rows)
                vp = _part(pre + "self_attn.v_proj.weight", rows=p.kv_rows)
                bq = _vec(loader, pre + "self_attn.q_proj.bias", p.q_rows)
                bias = None
                if bq is not None:
                    bias = np.concatenate([bq, _vec(loader, pre + "self_attn.k_proj.bias", p.kv_rows),
                                           _vec(loader, pre + "self_attn.v_proj.bias", p.kv_rows)])
            qkv = ops.make_linear([qp, kp, vp], c.hidden_size, gs, bias)
            o = ops.make_linear([_part(pre + "self_attn.o_proj.weight", cols=p.q_rows)], p.q_dim, gs)
            if has(pre + "mlp.gate_up_proj.weight"):       # Phi-3: [gate; up]
                n = pre + "mlp.gate_up_proj.weight"
                I = c.intermediate_size
                gp = _part(n, rows=p.inter)
                up = _part(n, rows=(I + p.inter[0], I + p.inter[1]))
            else:
                gp = _part(pre + "mlp.gate_proj.weight", rows=p.inter)
                up = _part(pre + "mlp.up_proj.weight", rows=p.inter)
            gate_up = ops.make_linear([gp, up], c.hidden_size, gs, swiglu=True)
            down = ops.make_linear([_part(pre + "mlp.down_proj.weight", cols=p.inter)], p.inter_size, gs)
            self.layers.append(LayerWeights(to_dev(_vec(loader, pre + "input_layernorm.weight")),
                                            to_dev(_vec(loader, pre + "post_attention_layernorm.weight")),
                                            qkv, o, gate_up, down))
            self.weight_bytes += qkv.nbytes + o.nbytes + gate_up.nbytes + down.nbytes
            if progress:
                progress(i + 1, c.num_layers)
        head_name = "lm_head.weight" if has("lm_head.weight") else "embed_tokens.weight"   # tied embeddings
        self.lm_head = ops.make_linear([_part(head_name, rows=p.vocab)], c.hidden_size, gs)
        self.weight_bytes += self.lm_head.nbytes
        if mirror is not None:
            mirror.release()
        rot = c.head_dim
        if c.partial_rotary_factor and not c.is_gemma:       # the leading part of each head rotates, the rest passes
            rot = 2 * int(c.partial_rotary_factor * c.head_dim // 2)
        self.inv_freq = ref.inv_freq(rot, c.rope_theta, c.rope_scaling).to(dev)
        # cos / sin of every (position, frequency) for the fused QKV epilogue of decode-sized passes (head_dim 128, full
        # rotary): [max_seq_len, 64, 2] fp32, computed once with the same fp32 arithmetic as the oracle
        self.rope_table = None
        if dev.type == "cuda" and c.head_dim == 128 and rot == 128 and not c.is_gemma:
            pos = torch.arange(max(int(c.max_seq_len), 1), dtype=torch.float32, device=dev)
            ang = pos[:, None] * self.inv_freq[None, :]
            self.rope_table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()

    # ---- buffers --------------------------------------------------------------------------------------
    def make_buffers(self, max_tokens: int, max_seqs: int, max_blocks: int, logits_rows: Optional[int] = None,
                     max_planes: int = 8, attn_splits: int = 1) -> StepBuffers:
        b = StepBuffers(self.config, self.plan, self.device, max_tokens, max_seqs, max_blocks, max_planes,
                        logits_rows or max_seqs, attn_splits)
        sp = getattr(self.comm, "sp_xnorm", None)
        if sp is not None and sp.shape[0] >= max_tokens and sp.shape[1] == self.config.hidden_size:
            # the normalised activations live in the symmetric buffer other ranks store gathered rows into
            b.xnorm = sp[:max_tokens]
        return b

    @property
    def _sp_weights_ok(self) -> bool:
        """The row-block exchange handles a pass only as a whole: every projection INT4, no bias on o / down."""
        ok = getattr(self, "_sp_ok_cache", None)
        if ok is None:
            ok = all(L.qkv.kind == L.o.kind == L.gate_up.kind == L.down.kind == "w4t" and L.o.bias is None
                     and L.down.bias is None and L.gate_up.swiglu for L in self.layers) and not self.config.is_gemma
            self._sp_ok_cache = ok
        return ok

    # ---- forward --------------------------------------------------------------------------------------
    def _add_norm(self, b: StepBuffers, planes: int, weight: torch.Tensor, M: int, add=None) -> None:
        """residual += (row-parallel output summed over split-K planes and, with tensor parallelism, over ranks)
        [+ ``add``: an fp16 addend, the LoRA update of that projection; single GPU only];
        xnorm = RMSNorm(residual) * weight."""
        ops, eps = self.ops, self.config.rms_norm_eps
        if planes is None:               # the projection's own kernel reduced, added and normalised already
            return
        if add is not None and self.comm is not None and planes > 0:
            # tensor parallelism: the adapter update of a row-parallel projection is a partial sum like the projection's
            # own output (its A is sharded by columns), so it joins plane 0 and the exchange below sums both
            H = b.partials.shape[-1]
            b.partials.view(-1)[: M * H].view(M, H).add_(add[:M])
            add = None
        if add is not None:
            if self.comm is not None:
                raise RuntimeError("an adapter update without a projection output to join")
            ops.add_rmsnorm(b.residual, b.partials, planes, add, weight, b.xnorm, M, eps)
        elif planes < 0:                 # the GEMM pushed its rows to every rank itself (-planes = its CTA count)
            self.comm.sum_add_rmsnorm(ops, b.residual, weight, b.xnorm, M, eps, -planes)
        elif self.comm is None or planes == 0:
            ops.add_rmsnorm(b.residual, b.partials, planes, None, weight, b.xnorm, M, eps)
        elif self.comm.fused_norm:
            self.comm.reduce_add_rmsnorm(ops, b.residual, b.partials, planes, weight, b.xnorm, M, eps)
        elif self.comm.use_sequence_parallel(M):
            self.comm.reduce_scatter_add_rmsnorm(ops, b.residual, b.partials, planes, weight, b.xnorm, M, eps)
        else:
            planes = self.comm.all_reduce_partials(b.partials, planes, M)
            ops.add_rmsnorm(b.residual, b.partials, planes, None, weight, b.xnorm, M, eps)

    def _row_parallel(self, w: LinearWeight, x: torch.Tensor, M: int, b: StepBuffers, norm_w=None, add=None):
        """Row-parallel projection.  Returns the number of fp32 planes written to ``b.partials``, or - when the
        tensor-parallel exchange ran inside the GEMM - minus the CTA count the consumer has to wait for, or None when
        one kernel did the projection, the all-reduce, the residual add and the RMSNorm with ``norm_w``."""
        comm = self.comm
        if (comm is not None and norm_w is not None and add is None and self.lora is None
                and getattr(comm, "sp_xnorm", None) is not None and b.xnorm.data_ptr() == comm.sp_xnorm.data_ptr()
                and self._sp_weights_ok and comm.can_sp(w, M)):
            # many rows: reduce-scatter in the GEMM's epilogue, reduce + norm on the owner, gather into every rank's
            # b.xnorm; the GEMMs that read b.xnorm next wait for their rows themselves (self._sp_live)
            comm.linear_scatter_norm(self.ops, w, x, M, b.residual, norm_w, self.config.rms_norm_eps)
            self._sp_live = True
            return None
        if (comm is not None and norm_w is not None and add is None and getattr(comm, "fused_k1", False)
                and comm.can_fuse_k1(self.ops, w, M)):
            comm.linear_allreduce_norm(self.ops, w, x, M, b.residual, norm_w, b.xnorm, self.config.rms_norm_eps)
            return None
        if (comm is None and norm_w is not None and add is None
                and self.ops.residual_norm_fused_ok(w, M, self.config.hidden_size)):
            self.ops.linear_residual_norm(w, x, M, b.residual, norm_w, b.xnorm, self.config.rms_norm_eps,
                                          self._local_calls)
            self._local_calls += 1
            return None
        if (comm is not None and add is None and getattr(comm, "push", False) and w.K in self._uniform_shard_k()
                and comm.can_push(w, M)):
            return -comm.linear_push(self.ops, w, x, M)
        return self.ops.linear_partial(w, x, M, b.partials)

    def forward(self, b: StepBuffers, kv: torch.Tensor, M: int, mode: str, num_seqs: int, max_q_len: int = 1,
                n_logit_rows: int = 0, attn_splits: int = 1) -> None:
        """Runs the stack over tokens ``b.ids[:M]``; leaves fp16 logits of rows ``b.logit_rows[:n_logit_rows]`` in
        ``b.logits``.  ``kv``: [layers, blocks, 2, nkv_local, block_size, hd]."""
        c, p, ops = self.config, self.plan, self.ops
        bs = kv.shape[4]
        if self.comm is None and self.lora is None:
            step = self._native_step_for(b)
            if step is not None:       # one C call launches the whole pass (csrc/step.cu)
                step.forward(kv, M, mode == "decode", num_seqs, max_q_len, n_logit_rows, attn_splits)
                return
        if self.comm is not None and self.comm.fused_norm:
            self.comm.begin_pass()
        ops.embedding(self.embed, b.ids, b.residual, M, self.embed_scale)
        planes, add = 0, None
        lora = self.lora
        self._local_calls = 0
        self._sp_live = False          # b.xnorm currently arrives from other ranks (sequence-parallel exchange)
        for li, L in enumerate(self.layers):
            self._add_norm(b, planes, L.ln1, M, add)
            gather = self.comm._ctx if self._sp_live else None
            if gather is not None:
                ops.linear(L.qkv, b.xnorm, M, b.qkv, gather=gather)
                ops.rope_kv_write(b.qkv, kv[li], b.positions, b.slots, self.inv_freq, M, p.num_heads,
                                  p.num_kv_heads, c.head_dim, bs)
            elif (self.lora is None and self.rope_table is not None
                    and ops.qkv_rope_fused_ok(L.qkv, M, c.head_dim, kv[li])):
                ops.qkv_rope_fused(L.qkv, b.xnorm, M, b.qkv, kv[li], b.positions, b.slots, self.rope_table,
                                   p.num_heads, p.num_kv_heads, bs)
            elif self.lora is None and M <= b.qkv_plane_rows and L.qkv.kind == "w4t":
                n_q = ops.linear_partial(L.qkv, b.xnorm, M, b.qkv_planes)
                ops.rope_kv_write(b.qkv, kv[li], b.positions, b.slots, self.inv_freq, M, p.num_heads, p.num_kv_heads,
                                  c.head_dim, bs, planes=b.qkv_planes, n_planes=n_q, bias=L.qkv.bias)
            else:
                ops.linear(L.qkv, b.xnorm, M, b.qkv)
                if self.lora is not None:
                    self.lora.apply_qkv(li, b, M)
                ops.rope_kv_write(b.qkv, kv[li], b.positions, b.slots, self.inv_freq, M, p.num_heads,
                                  p.num_kv_heads, c.head_dim, bs)
            if mode == "decode":
                ops.attn_decode(b.qkv, kv[li], b.block_tables, b.seq_lens, b.attn_out, num_seqs, p.num_heads,
                                p.num_kv_heads, c.head_dim, bs, self.scale, b.attn_scratch, attn_splits,
                                window=self.window)
            else:
                ops.attn_prefill(b.qkv, kv[li], b.block_tables, b.cu_q, b.q_pos0, b.attn_out, num_seqs, M, max_q_len,
                                 p.num_heads, p.num_kv_heads, c.head_dim, bs, self.scale, window=self.window)
            add = lora.delta(li, "o_proj", b.attn_out, b, M) if lora is not None else None
            planes = self._row_parallel(L.o, b.attn_out, M, b, L.ln2, add)
            self._add_norm(b, planes, L.ln2, M, add)
            if lora is not None and (lora.has(li, "gate_proj") or lora.has(li, "up_proj")):
                self._mlp_in_with_lora(li, L, b, M)
            else:
                ops.linear_swiglu(L.gate_up, b.xnorm, M, b.act, gather=self.comm._ctx if self._sp_live else None)
            add = lora.delta(li, "down_proj", b.act, b, M) if lora is not None else None
            next_norm = self.layers[li + 1].ln1 if li + 1 < len(self.layers) else self.norm
            planes = self._row_parallel(L.down, b.act, M, b, next_norm, add)
        self._add_norm(b, planes, self.norm, M, add)
        if self._sp_live:              # the final normalised rows come from their owners: wait for all of them
            self.comm.sp_wait(ops, M)
            self._sp_live = False
        if n_logit_rows:
            torch.index_select(b.xnorm, 0, b.logit_rows[:n_logit_rows], out=b.xsel[:n_logit_rows])
            ops.linear(self.lm_head, b.xsel, n_logit_rows, b.logits)

    def _mlp_in_with_lora(self, li: int, L: LayerWeights, b: StepBuffers, M: int) -> None:
        """act = silu(x Wg^T + dg) * (x Wu^T + du) without the fused SwiGLU epilogue: the projection is written out,
        the adapters' updates are added and the activation is applied on top."""
        ops, lora, p = self.ops, self.lora, self.plan
        I = p.inter_size
        gu = lora._scratch(b, "lora_gate_up", L.gate_up.N)
        plain = LinearWeight(L.gate_up.kind, L.gate_up.N, L.gate_up.K, L.gate_up.data, None, False, L.gate_up.nbytes)
        ops.linear(plain, b.xnorm, M, gu)
        if L.gate_up.kind in ("w4t", "w8t") and L.gate_up.swiglu:   # tiles of 64 gate rows followed by their 64 up rows
            if I % 64:
                raise NotImplementedError("LoRA on gate/up needs an intermediate size that is a multiple of 64")
            t = gu[:M].view(M, I // 64, 2, 64)
            g, u = t[:, :, 0, :].reshape(M, I).float(), t[:, :, 1, :].reshape(M, I).float()
        else:
            g, u = gu[:M, :I].float(), gu[:M, I: 2 * I].float()
        dg = lora.delta(li, "gate_proj", b.xnorm, b, M)
        du = lora.delta(li, "up_proj", b.xnorm, b, M)
        if dg is not None:
            g = g + dg[:M].float()
        if du is not None:
            u = u + du[:M].float()
        b.act[:M, :I] = ref.swiglu(g, u)

    def _uniform_shard_k(self) -> set:
        """Input widths of the row-parallel projections that are the same on every rank.  The exchange inside the GEMM
        counts CTAs, and every rank must launch the same number: shards of unequal width (group-aligned splits of an
        intermediate size that does not divide evenly, e.g. 13824 over 8 ranks) plan differently and stay on the
        pull path."""
        ok = self.__dict__.get("_uniform_k")
        if ok is None:
            plans = [make_plan(self.config, self.plan.tp_size, r) for r in range(self.plan.tp_size)]
            ok = set()
            if len({pl.q_dim for pl in plans}) == 1:
                ok.add(self.plan.q_dim)
            if len({pl.inter_size for pl in plans}) == 1:
                ok.add(self.plan.inter_size)
            self._uniform_k = ok
        return ok

    def _native_step_for(self, b: StepBuffers):
        """The native step driver bound to these buffers (built on first use), or None where it does not apply."""
        cache = self.__dict__.setdefault("_native_steps", {})
        key = id(b)
        if key not in cache:
            from ..runtime import step_driver
            cache[key] = step_driver.try_build(self, b)
        return cache[key]

    def hidden_rows(self, b: StepBuffers, rows: int) -> torch.Tensor:
        """Final-norm hidden states of the first ``rows`` tokens of the last pass (for embeddings / RAG)."""
        return b.xnorm[:rows]

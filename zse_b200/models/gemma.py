"""Gemma-2 and Gemma-4 (text) decoder over the paged KV cache.

Same pass contract as ``DecoderModel`` (packed tokens in persistent step buffers, prefill / chunked prefill /
verification / batched decode from one ``forward``), different block (``csrc/gemma.cu``):

    x   = RMSNorm(h) * w_in                       (fused into the previous layer's last kernel)
    qkv = x W_qkv                                 [q | k | v], or [q | k] on layers without v_proj
    head norms (q, k learned; v plain), RoPE with the layer's base and rotary fraction, cache write      1 kernel
    a   = attention(q, cache)                     soft-capped scores, sliding window on local layers
    h   = h + RMSNorm(a W_o) * w_post_attn ;  x = RMSNorm(h) * w_pre_ffn                                1 kernel
    m   = (gelu_tanh(x W_gate) * x W_up) W_down
    h   = (h + RMSNorm(m) * w_post_ffn) * layer_scalar ;  x = RMSNorm(h) * w_in(next layer)             1 kernel

The reference runs this family through a dedicated prefill-only path with separate launches for every step and no
KV cache (zse-engine/zse_engine/orchestrator/model_runner.py:386-580); here it decodes, batches and shares the
scheduler with every other model.  Layers of a model may differ in head_dim and kv heads (Gemma-4 local / global
layers): the KV pool is allocated with rows of the widest layer and each layer addresses its own packing inside the
row through strides.  Tensor parallelism splits heads and the MLP like the other families, with a plain fp16
all-reduce after the two row-parallel projections (no fused exchange kernel for this family).
"""
from __future__ import annotations

import math
import os
import dataclasses
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..format.config import LayerSpec, ModelConfig
from ..format.loader import ZSELoader
from ..ops.backend import LinearWeight, np_to_dev
from .decoder import DecoderModel, StepBuffers, _entry_part, _vec


@dataclass
class GemmaLayerWeights:
    spec: LayerSpec
    ln_in: torch.Tensor
    ln_post_attn: torch.Tensor
    ln_pre_ffn: torch.Tensor
    ln_post_ffn: torch.Tensor
    q_norm: Optional[torch.Tensor]
    k_norm: Optional[torch.Tensor]
    scalar: Optional[torch.Tensor]
    freqs: torch.Tensor
    qkv: LinearWeight
    o: LinearWeight
    gate_up: LinearWeight
    down: LinearWeight

    @property
    def qkv_width(self) -> int:
        return self.qkv.N


def rope_table(head_dim: int, theta: float, rotary_dim: int) -> torch.Tensor:
    """fp32 [head_dim/2]: theta^(-2i/head_dim) for the rotated pairs (i, i + head_dim/2), 0 for the others."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / head_dim)
    f[rotary_dim // 2:] = 0.0
    return f.to(torch.float32)


class GemmaDecoderModel(DecoderModel):
    def _load(self, loader: ZSELoader, progress=None) -> None:
        c, p, ops, dev = self.config, self.plan, self.ops, self.device
        tp, rank = p.tp_size, p.rank
        gs = c.quant.group_size
        has = lambda n: loader.weight_index.find(n) is not None
        off = c.norm_weight_offset

        def norm_w(name: str) -> Optional[torch.Tensor]:
            v = _vec(loader, name)
            if v is None:
                return None
            if off:
                v = (np.asarray(v, dtype=np.float32) + off).astype(np.float16)
            return np_to_dev(v, dev)

        mirror = None
        if dev.type == "cuda" and tp == 1:
            from ..runtime.weight_stream import open_mirror
            mirror = open_mirror(loader, dev, self.load_stats)       # None: switched off, or failed -> per-tensor copies
        part = lambda name, rows=None, cols=None: _entry_part(loader, name, rows, cols, mirror)
        self.embed = np_to_dev(loader.view_data(loader.weight_index.find("embed_tokens.weight")), dev)
        self.norm = norm_w("norm.weight")
        self.weight_bytes += self.embed.numel() * 2
        tables: Dict[tuple, torch.Tensor] = {}
        self.gelu = (c.hidden_activation or "gelu_pytorch_tanh").startswith("gelu")
        for i in range(c.num_layers):
            pre = f"layers.{i}."
            full = c.layer_spec(i)
            # this rank's heads: query heads and kv heads are split evenly (column-parallel q/k/v, row-parallel o)
            sp = dataclasses.replace(full, num_kv_heads=full.num_kv_heads // tp)
            hd = sp.head_dim
            q_rows = (rank * p.num_heads * hd, (rank + 1) * p.num_heads * hd)
            kv_rows = (rank * sp.num_kv_heads * hd, (rank + 1) * sp.num_kv_heads * hd)
            parts = [part(pre + "self_attn.q_proj.weight", rows=q_rows),
                     part(pre + "self_attn.k_proj.weight", rows=kv_rows)]
            if not sp.k_is_v:
                parts.append(part(pre + "self_attn.v_proj.weight", rows=kv_rows))
            qkv = ops.make_linear(parts, c.hidden_size, gs)
            o = ops.make_linear([part(pre + "self_attn.o_proj.weight", cols=q_rows)], p.num_heads * hd, gs)
            gate_up = ops.make_linear([part(pre + "mlp.gate_proj.weight", rows=p.inter),
                                       part(pre + "mlp.up_proj.weight", rows=p.inter)], c.hidden_size, gs)
            down = ops.make_linear([part(pre + "mlp.down_proj.weight", cols=p.inter)], p.inter_size, gs)
            key = (sp.head_dim, sp.rope_theta, sp.rotary_dim)
            if key not in tables:
                tables[key] = rope_table(*key).to(dev)
            scalar = None
            if has(pre + "layer_scalar"):
                scalar = np_to_dev(np.asarray(_vec(loader, pre + "layer_scalar"), dtype=np.float16).reshape(1), dev)
            self.layers.append(GemmaLayerWeights(
                sp, norm_w(pre + "input_layernorm.weight"), norm_w(pre + "post_attention_layernorm.weight"),
                norm_w(pre + "pre_feedforward_layernorm.weight"), norm_w(pre + "post_feedforward_layernorm.weight"),
                norm_w(pre + "self_attn.q_norm.weight") if sp.qk_norm else None,
                norm_w(pre + "self_attn.k_norm.weight") if sp.qk_norm else None, scalar, tables[key], qkv, o, gate_up,
                down))
            self.weight_bytes += qkv.nbytes + o.nbytes + gate_up.nbytes + down.nbytes
            if progress:
                progress(i + 1, c.num_layers)
        head_name = "lm_head.weight" if has("lm_head.weight") else "embed_tokens.weight"
        self.lm_head = ops.make_linear([part(head_name, rows=p.vocab)], c.hidden_size, gs)
        self.weight_bytes += self.lm_head.nbytes
        if mirror is not None:
            mirror.release()
        self.final_softcap = float(c.final_logit_softcapping or 0.0)
        self._kv_views: Dict[tuple, torch.Tensor] = {}

    # ---- buffers --------------------------------------------------------------------------------------
    def make_buffers(self, max_tokens: int, max_seqs: int, max_blocks: int, logits_rows: Optional[int] = None,
                     max_planes: int = 8, attn_splits: int = 1) -> StepBuffers:
        c = self.config
        b = StepBuffers(c, self.plan, self.device, max_tokens, max_seqs, max_blocks, 1, logits_rows or max_seqs,
                        attn_splits)
        f16 = torch.float16
        qkv_w = max(L.qkv_width for L in self.layers)
        attn_w = max(self.plan.num_heads * L.spec.head_dim for L in self.layers)
        b.qkv = torch.zeros(max_tokens * qkv_w, dtype=f16, device=self.device)
        b.attn_out = torch.zeros(max_tokens * attn_w, dtype=f16, device=self.device)
        b.qkv_planes = torch.zeros(1, dtype=torch.float32, device=self.device)
        b.partials = torch.zeros(1, 1, c.hidden_size, dtype=torch.float32, device=self.device)
        max_hd = max(L.spec.head_dim for L in self.layers)
        b.attn_scratch = torch.zeros(max(1, max_seqs * self.plan.num_heads * attn_splits * (max_hd + 2)),
                                     dtype=torch.float32,
                                     device=self.device)
        b.gate_up = torch.zeros(max_tokens, 2 * self.plan.inter_size, dtype=f16, device=self.device)
        b.sub_out = torch.zeros(max_tokens, c.hidden_size, dtype=f16, device=self.device)
        # per-width 2-D views of the flat q/k/v and attention buffers (a layer's row length is its own)
        b.qkv_views = {w: b.qkv[: max_tokens * w].view(max_tokens, w) for w in {L.qkv_width for L in self.layers}}
        b.attn_views = {w: b.attn_out[: max_tokens * w].view(max_tokens, w)
                        for w in {self.plan.num_heads * L.spec.head_dim for L in self.layers}}
        return b

    def _kv_view(self, kv: torch.Tensor, li: int, sp: LayerSpec) -> torch.Tensor:
        """This layer's [blocks, 2, kv_heads, block_size, head_dim] inside the pool ``[layers, blocks, 2, n, bs, d]``
        (the pool's rows are as wide as the widest layer; a narrower layer packs its heads at the front)."""
        key = (kv.data_ptr(), li)
        v = self._kv_views.get(key)
        if v is None:
            layer = kv[li]
            blocks, _, n, bs, d = layer.shape
            if (n, d) == (sp.num_kv_heads, sp.head_dim):
                v = layer
            else:
                if sp.num_kv_heads * sp.head_dim > n * d:
                    raise ValueError("KV pool rows are narrower than this layer")
                v = layer.as_strided((blocks, 2, sp.num_kv_heads, bs, sp.head_dim),
                                     (layer.stride(0), layer.stride(1), bs * sp.head_dim, sp.head_dim, 1),
                                     layer.storage_offset())
            self._kv_views[key] = v
        return v

    # ---- forward --------------------------------------------------------------------------------------
    def forward(self, b: StepBuffers, kv: torch.Tensor, M: int, mode: str, num_seqs: int, max_q_len: int = 1,
                n_logit_rows: int = 0, attn_splits: int = 1) -> None:
        c, ops = self.config, self.ops
        eps, nh, I = c.rms_norm_eps, self.plan.num_heads, self.plan.inter_size
        comm = self.comm
        bs = kv.shape[4]
        ops.embedding(self.embed, b.ids, b.residual, M, self.embed_scale)
        ops.add_rmsnorm(b.residual, b.partials, 0, None, self.layers[0].ln_in, b.xnorm, M, eps)
        for li, L in enumerate(self.layers):
            sp = L.spec
            hd, nkv = sp.head_dim, sp.num_kv_heads
            qkv = b.qkv_views[L.qkv_width]
            attn_out = b.attn_views[nh * hd]
            kvv = self._kv_view(kv, li, sp)
            ops.linear(L.qkv, b.xnorm, M, qkv)
            ops.headnorm_rope_kv_write(qkv, kvv, b.positions, b.slots, L.freqs, L.q_norm, L.k_norm, sp.qk_norm,
                                       sp.k_is_v, eps, M, nh, nkv, hd, bs)
            if mode == "decode":
                ops.attn_decode(qkv, kvv, b.block_tables, b.seq_lens, attn_out, num_seqs, nh, nkv, hd, bs, sp.scale,
                                b.attn_scratch, attn_splits, softcap=sp.softcap, window=sp.window)
            else:
                ops.attn_prefill(qkv, kvv, b.block_tables, b.cu_q, b.q_pos0, attn_out, num_seqs, M, max_q_len, nh,
                                 nkv, hd, bs, sp.scale, softcap=sp.softcap, window=sp.window)
            ops.linear(L.o, attn_out, M, b.sub_out)
            if comm is not None:                    # row-parallel: sum the ranks' partial outputs (fp16, as the
                comm.all_reduce(b.sub_out[:M])      # reference does after o_proj and down_proj)
            ops.norm_add_rmsnorm(b.sub_out, L.ln_post_attn, b.residual, None, L.ln_pre_ffn, b.xnorm, M, eps)
            ops.linear(L.gate_up, b.xnorm, M, b.gate_up)
            ops.glu(b.gate_up, b.act, M, I, self.gelu)
            ops.linear(L.down, b.act, M, b.sub_out)
            if comm is not None:
                comm.all_reduce(b.sub_out[:M])
            nxt = self.layers[li + 1].ln_in if li + 1 < len(self.layers) else self.norm
            ops.norm_add_rmsnorm(b.sub_out, L.ln_post_ffn, b.residual, L.scalar, nxt, b.xnorm, M, eps)
        if n_logit_rows:
            torch.index_select(b.xnorm, 0, b.logit_rows[:n_logit_rows], out=b.xsel[:n_logit_rows])
            ops.linear(self.lm_head, b.xsel, n_logit_rows, b.logits)
            if self.final_softcap:
                ops.softcap(b.logits, n_logit_rows, self.final_softcap)

"""fp32 reference forward pass of a ``.zse`` decoder (the oracle every other path is checked against).

Weights are dequantised to fp32 exactly as the file defines them (INT4: ``nibble*scale + zero`` per run of
``group_size`` values of the flattened tensor; zse-engine/zse_engine/format/quantize.py:89-128) and the
Llama/Qwen2 block is evaluated in fp32 with the numerics contract of the reference runner
(zse-engine/zse_engine/orchestrator/model_runner.py:1123-1297): RMSNorm ``x*rsqrt(mean(x^2)+eps)*w``, rotate-half
RoPE with ``freq_i = theta^(-2i/hd)``, GQA ``kv = head // (nh/nkv)``, scale ``1/sqrt(hd)``, causal softmax,
``down(silu(gate)*up)``.  Gemma-2 / Gemma-4 layers follow HuggingFace transformers (and the reference's Gemma-4
path, model_runner.py:428-540).  Nothing here is rounded to 16 bits.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..format.loader import ZSELoader


def load_fp32_weights(loader: ZSELoader) -> Dict[str, torch.Tensor]:
    out = {}
    for e in loader.weight_index:
        out[e.name] = torch.from_numpy(np.ascontiguousarray(loader.get_weight_as_float(e)))
    return out


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 rope_scaling: Optional[dict] = None):
    """cos/sin [T, head_dim/2]; pairs beyond ``rotary_dim/2`` get angle 0 (they pass through unrotated).
    ``rope_scaling`` of kind ``linear`` (all frequencies divided by the factor) and ``llama3`` (long wavelengths
    divided by the factor, short ones kept, a smooth blend between) changes the frequencies, as in transformers."""
    half = head_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    kind = (rope_scaling or {}).get("rope_type", (rope_scaling or {}).get("type"))
    if kind == "linear":
        inv = inv / float(rope_scaling["factor"])
    elif kind == "llama3":
        factor = float(rope_scaling["factor"])
        low, high = float(rope_scaling.get("low_freq_factor", 1.0)), float(rope_scaling.get("high_freq_factor", 4.0))
        old = float(rope_scaling.get("original_max_position_embeddings", 8192))
        scaled = []
        for f in inv.tolist():
            wavelen = 2 * math.pi / f
            if wavelen < old / high:
                scaled.append(f)
            elif wavelen > old / low:
                scaled.append(f / factor)
            else:
                t = (old / wavelen - low) / (high - low)
                scaled.append((1 - t) * f / factor + t * f)
        inv = torch.tensor(scaled, dtype=torch.float64)
    if rotary_dim is not None and rotary_dim < head_dim:
        inv[rotary_dim // 2:] = 0.0
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).float(), torch.sin(ang).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hd]; pairs (i, i+hd/2)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


class OracleModel:
    def __init__(self, loader: ZSELoader):
        self.config = loader.config
        self.w = load_fp32_weights(loader)
        if "lm_head.weight" not in self.w:
            self.w["lm_head.weight"] = self.w["embed_tokens.weight"]
        c = self.config
        for i in range(c.num_layers):               # Phi-3 stores [q; k; v] and [gate; up] stacked
            p = f"layers.{i}."
            qkv = self.w.pop(p + "self_attn.qkv_proj.weight", None)
            if qkv is not None:
                Q, KV = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
                for n, t in zip("qkv", torch.split(qkv, [Q, KV, KV], dim=0)):
                    self.w[p + f"self_attn.{n}_proj.weight"] = t
            gu = self.w.pop(p + "mlp.gate_up_proj.weight", None)
            if gu is not None:
                self.w[p + "mlp.gate_proj.weight"], self.w[p + "mlp.up_proj.weight"] = torch.chunk(gu, 2, dim=0)
        off = self.config.norm_weight_offset
        if off:
            for name in self.w:
                if name.endswith("norm.weight"):
                    self.w[name] = self.w[name] + off

    def _get(self, name: str) -> Optional[torch.Tensor]:
        return self.w.get(name)

    @torch.no_grad()
    def forward(self, token_ids, return_hidden: bool = False) -> torch.Tensor:
        """Full causal forward of one sequence; returns logits ``[T, vocab]`` (fp32).

        Gemma-family layers (zse-engine/zse_engine/orchestrator/model_runner.py:428-540): four norms per layer (the
        sub-layer output is normalised before it joins the residual), GeGLU, per-layer head_dim / kv heads / RoPE,
        q/k/v head norms, V = un-normalised K on layers without ``v_proj``, a learned per-layer scalar, soft-capped
        scores and logits, sliding-window layers."""
        c = self.config
        ids = torch.as_tensor(token_ids, dtype=torch.long)
        T = ids.numel()
        h = self.w["embed_tokens.weight"][ids]
        if c.embed_scale:
            h = h * (c.hidden_size ** 0.5)
        gemma = c.is_gemma
        gelu = (c.hidden_activation or "").startswith("gelu")
        pos = torch.arange(T)
        causal = pos[None, :] > pos[:, None]
        for i in range(c.num_layers):
            p = f"layers.{i}."
            sp = c.layer_spec(i) if gemma else None
            hd = sp.head_dim if sp else c.head_dim
            nkv = sp.num_kv_heads if sp else c.num_kv_heads
            lead = hd                  # Phi-style partial rotary: only the first ``lead`` dims of a head rotate
            if not gemma and c.partial_rotary_factor:
                lead = 2 * int(c.partial_rotary_factor * hd // 2)
            cos, sin = rope_cos_sin(pos, lead, sp.rope_theta if sp else c.rope_theta, sp.rotary_dim if sp else None,
                                    None if gemma else c.rope_scaling)
            x = rmsnorm(h, self.w[p + "input_layernorm.weight"], c.rms_norm_eps)
            q = x @ self.w[p + "self_attn.q_proj.weight"].T
            k = x @ self.w[p + "self_attn.k_proj.weight"].T
            v = k.clone() if (sp and sp.k_is_v) else x @ self.w[p + "self_attn.v_proj.weight"].T
            for t, name in ((q, "q"), (k, "k"), (v, "v")):
                b = self._get(p + f"self_attn.{name}_proj.bias")
                if b is not None:
                    t += b
            q, k, v = q.view(T, c.num_heads, hd), k.view(T, nkv, hd), v.view(T, nkv, hd)
            if sp and sp.qk_norm:
                q = rmsnorm(q, self.w[p + "self_attn.q_norm.weight"], c.rms_norm_eps)
                k = rmsnorm(k, self.w[p + "self_attn.k_norm.weight"], c.rms_norm_eps)
                v = rmsnorm(v, None, c.rms_norm_eps)
            if lead < hd:
                q = torch.cat([apply_rope(q[..., :lead], cos, sin), q[..., lead:]], dim=-1)
                k = torch.cat([apply_rope(k[..., :lead], cos, sin), k[..., lead:]], dim=-1)
            else:
                q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            rep = c.num_heads // nkv
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
            s = torch.einsum("thd,shd->hts", q, k) * (sp.scale if sp else hd ** -0.5)
            if sp and sp.softcap:
                s = torch.tanh(s / sp.softcap) * sp.softcap
            hidden = causal
            win = sp.window if sp else (int(c.sliding_window or 0) if not c.layer_types else 0)
            if win:
                hidden = causal | (pos[None, :] <= pos[:, None] - win)
            s = s.masked_fill(hidden[None], float("-inf"))
            a = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), v).reshape(T, c.num_heads * hd)
            a = a @ self.w[p + "self_attn.o_proj.weight"].T
            if gemma:
                h = h + rmsnorm(a, self.w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
                x = rmsnorm(h, self.w[p + "pre_feedforward_layernorm.weight"], c.rms_norm_eps)
            else:
                h = h + a
                x = rmsnorm(h, self.w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            g = x @ self.w[p + "mlp.gate_proj.weight"].T
            u = x @ self.w[p + "mlp.up_proj.weight"].T
            act = torch.nn.functional.gelu(g, approximate="tanh") if gelu else torch.nn.functional.silu(g)
            m = (act * u) @ self.w[p + "mlp.down_proj.weight"].T
            if gemma:
                h = h + rmsnorm(m, self.w[p + "post_feedforward_layernorm.weight"], c.rms_norm_eps)
                ls = self._get(p + "layer_scalar")
                if ls is not None:
                    h = h * ls.reshape(-1)[0]
            else:
                h = h + m
        hn = rmsnorm(h, self.w["norm.weight"], c.rms_norm_eps)
        if return_hidden:
            return hn
        logits = hn @ self.w["lm_head.weight"].T
        if c.final_logit_softcapping:
            logits = torch.tanh(logits / c.final_logit_softcapping) * c.final_logit_softcapping
        return logits

    @torch.no_grad()
    def greedy(self, prompt: List[int], max_new_tokens: int) -> List[int]:
        ids = list(prompt)
        for _ in range(max_new_tokens):
            ids.append(int(self.forward(ids)[-1].argmax()))
        return ids[len(prompt):]

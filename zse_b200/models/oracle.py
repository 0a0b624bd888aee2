"""fp32 reference forward pass of a ``.zse`` decoder (the oracle every other path is checked against).

Weights are dequantised to fp32 exactly as the file defines them (INT4: ``nibble*scale + zero`` per run of
``group_size`` values of the flattened tensor; zse-engine/zse_engine/format/quantize.py:89-128) and the
Llama/Qwen2 block is evaluated in fp32 with the numerics contract of the reference runner
(zse-engine/zse_engine/orchestrator/model_runner.py:1123-1297): RMSNorm ``x*rsqrt(mean(x^2)+eps)*w``, rotate-half
RoPE with ``freq_i = theta^(-2i/hd)``, GQA ``kv = head // (nh/nkv)``, scale ``1/sqrt(hd)``, causal softmax,
``down(silu(gate)*up)``.  Nothing here is rounded to 16 bits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..format.loader import ZSELoader


def load_fp32_weights(loader: ZSELoader) -> Dict[str, torch.Tensor]:
    out = {}
    for e in loader.weight_index:
        out[e.name] = torch.from_numpy(np.ascontiguousarray(loader.get_weight_as_float(e)))
    return out


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    half = head_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).float(), torch.sin(ang).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hd]; pairs (i, i+hd/2)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


class OracleModel:
    def __init__(self, loader: ZSELoader):
        self.config = loader.config
        self.w = load_fp32_weights(loader)
        if "lm_head.weight" not in self.w:
            self.w["lm_head.weight"] = self.w["embed_tokens.weight"]

    def _get(self, name: str) -> Optional[torch.Tensor]:
        return self.w.get(name)

    @torch.no_grad()
    def forward(self, token_ids, return_hidden: bool = False) -> torch.Tensor:
        """Full causal forward of one sequence; returns logits ``[T, vocab]`` (fp32)."""
        c = self.config
        ids = torch.as_tensor(token_ids, dtype=torch.long)
        T = ids.numel()
        h = self.w["embed_tokens.weight"][ids]
        cos, sin = rope_cos_sin(torch.arange(T), c.head_dim, c.rope_theta)
        mask = torch.full((T, T), float("-inf")).triu(1)
        rep = c.num_heads // c.num_kv_heads
        for i in range(c.num_layers):
            p = f"layers.{i}."
            x = rmsnorm(h, self.w[p + "input_layernorm.weight"], c.rms_norm_eps)
            q = x @ self.w[p + "self_attn.q_proj.weight"].T
            k = x @ self.w[p + "self_attn.k_proj.weight"].T
            v = x @ self.w[p + "self_attn.v_proj.weight"].T
            for t, name in ((q, "q"), (k, "k"), (v, "v")):
                b = self._get(p + f"self_attn.{name}_proj.bias")
                if b is not None:
                    t += b
            q = apply_rope(q.view(T, c.num_heads, c.head_dim), cos, sin)
            k = apply_rope(k.view(T, c.num_kv_heads, c.head_dim), cos, sin)
            v = v.view(T, c.num_kv_heads, c.head_dim)
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
            s = torch.einsum("thd,shd->hts", q, k) / (c.head_dim ** 0.5) + mask
            a = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), v).reshape(T, c.q_dim)
            h = h + a @ self.w[p + "self_attn.o_proj.weight"].T
            x = rmsnorm(h, self.w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            g = x @ self.w[p + "mlp.gate_proj.weight"].T
            u = x @ self.w[p + "mlp.up_proj.weight"].T
            h = h + (torch.nn.functional.silu(g) * u) @ self.w[p + "mlp.down_proj.weight"].T
        hn = rmsnorm(h, self.w["norm.weight"], c.rms_norm_eps)
        if return_hidden:
            return hn
        return hn @ self.w["lm_head.weight"].T

    @torch.no_grad()
    def greedy(self, prompt: List[int], max_new_tokens: int) -> List[int]:
        ids = list(prompt)
        for _ in range(max_new_tokens):
            ids.append(int(self.forward(ids)[-1].argmax()))
        return ids[len(prompt):]

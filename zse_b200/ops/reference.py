"""Plain PyTorch restatement of every device op (fp32 math on whatever device the tensors live on).

Two jobs: the execution path on machines without a GPU (the tiny CPU configuration), and the oracle that the
numerics tests compare each CUDA kernel against.  Semantics follow the reference runner's numerics contract
(zse-engine/zse_engine/orchestrator/kernels.py, see the per-function notes); accumulation is fp32 and results are
rounded to fp16 where the CUDA kernels round.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def dequant_int4(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, shape, group_size: int = 128):
    """Flat-group dequantisation: element i belongs to group i // group_size of the flattened tensor."""
    n = int(math.prod(shape))
    groups = (n + group_size - 1) // group_size
    p = packed.reshape(-1)[: groups * group_size // 2]
    q = torch.stack([p & 0xF, p >> 4], dim=-1).reshape(groups, group_size).to(torch.float32)
    w = q * scales.reshape(-1)[:groups].float()[:, None] + zeros.reshape(-1)[:groups].float()[:, None]
    return w.reshape(-1)[:n].reshape(shape)


def dequant_int8(q: torch.Tensor, scales: torch.Tensor, shape, group_size: int = 128):
    n = int(math.prod(shape))
    groups = (n + group_size - 1) // group_size
    v = q.reshape(-1)[: groups * group_size].to(torch.float32).reshape(groups, group_size)
    return (v * scales.reshape(-1)[:groups].float()[:, None]).reshape(-1)[:n].reshape(shape)


def linear(x: torch.Tensor, w_f32: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 accumulate, clamp to the fp16 range, round to fp16 (kernels.py:1984-1987)."""
    y = x.float() @ w_f32.T
    if bias is not None:
        y = y + bias.float()
    return y.clamp(-65504, 65504).to(torch.float16)


def swiglu(gate: torch.Tensor, up: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    g, u = gate.float(), up.float()
    act = torch.nn.functional.gelu(g, approximate="tanh") if gelu else g / (1 + torch.exp(-g))
    return (act * u).clamp(-65504, 65504).to(torch.float16)


def rmsnorm(x_f32: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = x_f32.float()
    return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(torch.float16)


def inv_freq(rotary_dim: int, theta: float, rope_scaling: Optional[dict] = None) -> torch.Tensor:
    """theta^(-2i/rotary_dim) in float64, rounded to fp32.  ``linear`` and ``llama3`` scaling are applied here so
    the kernels only ever see a frequency table."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / rotary_dim)
    if rope_scaling:
        kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
        factor = float(rope_scaling.get("factor", 1.0))
        if kind == "linear":
            f = f / factor
        elif kind == "llama3":
            lo, hi = float(rope_scaling.get("low_freq_factor", 1.0)), float(rope_scaling.get("high_freq_factor", 4.0))
            old = float(rope_scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / f
            smooth = ((old / wavelen) - lo) / (hi - lo)
            mid = (1 - smooth) * f / factor + smooth * f
            f = torch.where(wavelen < old / hi, f, torch.where(wavelen > old / lo, f / factor, mid))
    return f.to(torch.float32)


def rope_(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on x [T, heads, hd] (pairs (i, i + rot/2) of the first ``2*len(freqs)`` dims)."""
    rot = freqs.numel() * 2
    ang = positions.to(torch.float32)[:, None] * freqs.to(positions.device)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    xf = x.float()
    a, b = xf[..., : rot // 2], xf[..., rot // 2: rot]
    out = xf.clone()
    out[..., : rot // 2] = a * c - b * s
    out[..., rot // 2: rot] = b * c + a * s
    return out.to(x.dtype)


def rope_kv_write(qkv: torch.Tensor, kv_layer: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                  freqs: torch.Tensor, nh: int, nkv: int, hd: int, block_size: int) -> None:
    """In place: rotates q and k inside ``qkv`` [M, (nh+2nkv)*hd], scatters k/v into ``kv_layer``
    [blocks, 2, nkv, block_size, hd] at ``slots`` (-1 = do not store)."""
    M = qkv.shape[0]
    q = qkv[:, : nh * hd].view(M, nh, hd)
    k = qkv[:, nh * hd: (nh + nkv) * hd].view(M, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(M, nkv, hd)
    q.copy_(rope_(q, positions, freqs))
    k.copy_(rope_(k, positions, freqs))
    ok = slots >= 0
    if ok.any():
        blk, off = slots[ok] // block_size, slots[ok] % block_size
        kv_layer[blk, 0, :, off, :] = k[ok].to(kv_layer.dtype)
        kv_layer[blk, 1, :, off, :] = v[ok].to(kv_layer.dtype)


def headnorm_rope_kv_write(qkv: torch.Tensor, kv_layer: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                           freqs: torch.Tensor, q_norm_w, k_norm_w, norm_v: bool, k_is_v: bool, eps: float, nh: int,
                           nkv: int, hd: int, block_size: int) -> None:
    """Gemma-family variant of ``rope_kv_write``: per-head RMSNorm of q and k (weights [hd] or None) and of v (no
    weight), RoPE with a full-length frequency table (0 = pair not rotated), V = raw k projection when ``k_is_v``
    (zse-engine/zse_engine/orchestrator/model_runner.py:455-486).  q is rotated in place; k and v only go to the
    cache."""
    M = qkv.shape[0]

    def hnorm(x, w):
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return y if w is None else y * w.float()

    q = qkv[:, : nh * hd].view(M, nh, hd)
    k_raw = qkv[:, nh * hd: (nh + nkv) * hd].float().view(M, nkv, hd)
    v = k_raw if k_is_v else qkv[:, (nh + nkv) * hd: (nh + 2 * nkv) * hd].float().view(M, nkv, hd)
    qf = q.float()
    if q_norm_w is not None:
        qf = hnorm(qf, q_norm_w)
    kf = hnorm(k_raw, k_norm_w) if k_norm_w is not None else k_raw
    if norm_v:
        v = hnorm(v, None)
    q.copy_(rope_(qf, positions, freqs).clamp(-65504, 65504).to(q.dtype))
    kf = rope_(kf, positions, freqs)
    ok = slots >= 0
    if ok.any():
        blk, off = slots[ok] // block_size, slots[ok] % block_size
        kv_layer[blk, 0, :, off, :] = kf[ok].clamp(-65504, 65504).to(kv_layer.dtype)
        kv_layer[blk, 1, :, off, :] = v[ok].clamp(-65504, 65504).to(kv_layer.dtype)


def norm_add_rmsnorm(x: torch.Tensor, w_post: torch.Tensor, residual: torch.Tensor, scalar, w_next, eps: float):
    """residual (fp32, in place) = (residual + RMSNorm(x)*w_post) * scalar; returns RMSNorm(residual)*w_next in fp16
    (or None without ``w_next``)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w_post.float()
    residual.add_(y)
    if scalar is not None:
        residual.mul_(float(scalar.reshape(-1)[0]))
    return None if w_next is None else rmsnorm(residual, w_next, eps)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return (cap * torch.tanh(x.float() / cap)).to(x.dtype)


def _gather_kv(kv_layer: torch.Tensor, table: torch.Tensor, length: int, block_size: int):
    """K, V [length, nkv, hd] plus a bool mask of positions that sit in holes (block id -1)."""
    nblk = (length + block_size - 1) // block_size
    ids = table[:nblk].long()
    hole = ids < 0
    safe = ids.clamp(min=0)
    k = kv_layer[safe, 0].permute(0, 2, 1, 3).reshape(nblk * block_size, kv_layer.shape[2], kv_layer.shape[4])
    v = kv_layer[safe, 1].permute(0, 2, 1, 3).reshape(nblk * block_size, kv_layer.shape[2], kv_layer.shape[4])
    mask = hole.repeat_interleave(block_size)[:length]
    return k[:length].float(), v[:length].float(), mask


def attn_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                nh: int, nkv: int, hd: int, block_size: int, scale: float, softcap: float = 0.0,
                window: int = 0) -> torch.Tensor:
    """q [S, nh*hd] -> out [S, nh*hd] fp16; sequence s attends to its first seq_lens[s] cached tokens."""
    S = q.shape[0]
    out = torch.zeros(S, nh * hd, dtype=torch.float16, device=q.device)
    rep = nh // nkv
    for s in range(S):
        n = int(seq_lens[s])
        if n == 0:
            continue
        k, v, hole = _gather_kv(kv_layer, block_tables[s], n, block_size)
        qs = q[s].float().view(nh, hd)
        sc = torch.einsum("hd,thd->ht", qs, k.repeat_interleave(rep, dim=1)) * scale
        if softcap:
            sc = softcap * torch.tanh(sc / softcap)
        if window:
            hole = hole | (torch.arange(n, device=q.device) < n - window)
        sc = sc.masked_fill(hole[None, :], float("-inf"))
        p = torch.softmax(sc, dim=-1).nan_to_num(0.0)
        out[s] = torch.einsum("ht,thd->hd", p, v.repeat_interleave(rep, dim=1)).reshape(-1).to(torch.float16)
    return out


def attn_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_tables: torch.Tensor, cu_q: torch.Tensor,
                 q_pos0: torch.Tensor, nh: int, nkv: int, hd: int, block_size: int, scale: float,
                 softcap: float = 0.0, window: int = 0) -> torch.Tensor:
    """Packed causal attention: query row r of sequence s sits at cache position q_pos0[s] + r and sees every
    cached token at or before it."""
    out = torch.zeros(q.shape[0], nh * hd, dtype=torch.float16, device=q.device)
    rep = nh // nkv
    for s in range(cu_q.numel() - 1):
        a, b = int(cu_q[s]), int(cu_q[s + 1])
        if b <= a:
            continue
        p0 = int(q_pos0[s])
        n = p0 + (b - a)
        k, v, hole = _gather_kv(kv_layer, block_tables[s], n, block_size)
        qs = q[a:b].float().view(b - a, nh, hd)
        sc = torch.einsum("qhd,thd->hqt", qs, k.repeat_interleave(rep, dim=1)) * scale
        if softcap:
            sc = softcap * torch.tanh(sc / softcap)
        pos_q = torch.arange(p0, n, device=q.device)[:, None]
        pos_k = torch.arange(n, device=q.device)[None, :]
        hidden = (pos_k > pos_q) | hole[None, :]
        if window:
            hidden = hidden | (pos_k <= pos_q - window)
        sc = sc.masked_fill(hidden[None], float("-inf"))
        p = torch.softmax(sc, dim=-1).nan_to_num(0.0)
        out[a:b] = torch.einsum("hqt,thd->qhd", p, v.repeat_interleave(rep, dim=1)).reshape(b - a, -1).to(torch.float16)
    return out


def apply_repetition_penalty(logits: torch.Tensor, counts: dict, penalty: float) -> torch.Tensor:
    """``counts``: token -> occurrences.  positive logits are divided, negative multiplied by
    ``penalty^(1+log2(count))`` (zse-engine/zse_engine/orchestrator/sampler.py:64-80)."""
    out = logits.clone().float()
    for tok, c in counts.items():
        if c > 0 and 0 <= tok < out.numel():
            f = penalty ** (1.0 + math.log2(c))
            out[tok] = out[tok] / f if out[tok] > 0 else out[tok] * f
    return out


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """The distribution the sampler draws from: temperature, then keep values >= the k-th largest, then the smallest
    sorted prefix whose softmax mass reaches top_p (ties at the cut are kept), renormalised."""
    x = logits.float() / max(temperature, 1e-6)
    if 0 < top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        x = torch.where(x >= kth, x, torch.full_like(x, float("-inf")))
    p = torch.softmax(x, dim=-1)
    if top_p < 1.0:
        sp, idx = torch.sort(p, descending=True)
        cum = torch.cumsum(sp, dim=-1)
        cut = int((cum < top_p).sum().item())
        thr = sp[min(cut, sp.numel() - 1)]
        p = torch.where(p >= thr, p, torch.zeros_like(p))
        p = p / p.sum()
    return p


def lora_delta(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scaling: float) -> torch.Tensor:
    """x [M, K], a [r, K], b [N, r] -> scaling * (x a^T) b^T in fp32."""
    return scaling * ((x.float() @ a.float().T) @ b.float().T)

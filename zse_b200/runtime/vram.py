"""Device memory plan: how much goes to weights, step buffers and the KV cache
(zse-engine/zse_engine/orchestrator/vram_allocator.py:19-336).

Budget rule of the reference: total - 400 MB context - 5 %; the KV cache is sized by demand
(``max_batch_seqs * max_seq_len * bytes/token * 1.5``, floor 256 MB), capped by what remains and by
``free - 1 GB``.  Here the plan is computed for this rank's shard (local kv heads, sharded weights) and B200-sized
defaults apply: with 180 GB per GPU the KV cache takes whatever the demand rule asks for, up to the cap.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..format.config import ModelConfig

MB = 1 << 20
GB = 1 << 30


@dataclass
class VRAMPlan:
    total_bytes: int
    free_bytes: int
    usable_bytes: int
    weight_bytes: int
    scratch_bytes: int
    kv_cache_bytes: int
    kv_blocks: int
    block_size: int
    max_seq_len: int
    max_batch_seqs: int

    # the reference's field names (zse-engine/zse_engine/orchestrator/vram_allocator.py:20-29)
    @property
    def total_vram(self) -> int:
        return self.total_bytes

    @property
    def available_vram(self) -> int:
        return self.total_bytes - VRAMAllocator.CONTEXT_RESERVE

    @property
    def reserved_bytes(self) -> int:
        return self.available_vram - self.usable_bytes

    @property
    def max_batch_tokens(self) -> int:
        return self.kv_blocks * self.block_size

    @property
    def utilization_pct(self) -> float:
        used = self.weight_bytes + self.scratch_bytes + self.kv_cache_bytes
        return 100.0 * used / self.total_bytes if self.total_bytes else 0.0

    def summary(self) -> str:
        g = lambda b: f"{b / GB:.2f} GB"
        return (f"VRAM plan: total {g(self.total_bytes)}, free {g(self.free_bytes)}, weights {g(self.weight_bytes)}, "
                f"scratch {g(self.scratch_bytes)}, KV {g(self.kv_cache_bytes)} = {self.kv_blocks} blocks x "
                f"{self.block_size} tokens (max_seq_len {self.max_seq_len}, {self.max_batch_seqs} sequences)")


@dataclass
class ScratchBuffers:
    """Activation buffers of one pass of at most ``max_seq_len`` tokens, under the reference's field names
    (zse-engine/zse_engine/orchestrator/vram_allocator.py:48-85).  The engine itself runs on ``models.decoder.
    StepBuffers`` (which adds the split-K planes, index tensors and sampling outputs the fused kernels need); this set is
    for code that drives individual kernels the way the reference's runner does."""
    hidden: Optional[object] = None          # [S, hidden] fp16
    residual: Optional[object] = None
    qkv: Optional[object] = None             # [S, (heads + 2 kv heads) * head_dim] fp16
    attn_out: Optional[object] = None
    mlp_gate: Optional[object] = None        # [S, intermediate] fp16
    mlp_up: Optional[object] = None
    mlp_out: Optional[object] = None
    logits: Optional[object] = None          # [min(S, 64), vocab] fp16
    norm_out: Optional[object] = None
    hidden_f32: Optional[object] = None      # fp32 residual stream
    residual_f32: Optional[object] = None
    total_bytes: int = 0

    FIELDS = ("hidden", "residual", "qkv", "attn_out", "mlp_gate", "mlp_up", "mlp_out", "logits", "norm_out",
              "hidden_f32", "residual_f32")

    def destroy(self, gpu_mem=None) -> None:
        for name in self.FIELDS:
            setattr(self, name, None)
        self.total_bytes = 0


class VRAMAllocator:
    CONTEXT_RESERVE = 400 * MB
    SAFETY_FRACTION = 0.05
    KV_FLOOR = 256 * MB
    FREE_MARGIN = 1 * GB
    CUDA_CONTEXT_BYTES = CONTEXT_RESERVE          # the reference's names for the two constants
    SAFETY_MARGIN_PCT = SAFETY_FRACTION

    def __init__(self, total_bytes: int, free_bytes: Optional[int] = None, device=None):
        self.total_bytes = total_bytes
        self.free_bytes = total_bytes if free_bytes is None else free_bytes
        self.device = device
        self._allocated_bytes = 0
        self._weight_bytes = 0

    # ---- accounting (vram_allocator.py:306-336 of the reference) ------------------------------------------------
    def track_weight_upload(self, nbytes: int) -> None:
        self._weight_bytes += int(nbytes)
        self._allocated_bytes += int(nbytes)

    @property
    def allocated_bytes(self) -> int:
        return self._allocated_bytes

    @property
    def weight_bytes(self) -> int:
        return self._weight_bytes

    def utilization(self) -> dict:
        total, free = self.total_bytes, self.free_bytes
        if self.device is not None:
            import torch
            if torch.cuda.is_available() and torch.device(self.device).type == "cuda":
                free, total = torch.cuda.mem_get_info(self.device)
        used = total - free if self.device is not None else self._allocated_bytes
        return {"total_bytes": total, "used_bytes": used, "free_bytes": free, "weight_bytes": self._weight_bytes,
                "utilization_pct": (used / total * 100) if total > 0 else 0}

    @staticmethod
    def scratch_shapes(config: ModelConfig, max_seq_len: int = 2048) -> dict:
        """name -> (shape, bytes per element).  Widths follow the widest layer (Gemma-4 full-attention layers have
        heads * head_dim above the hidden size)."""
        S, h, inter = max_seq_len, config.hidden_size, config.intermediate_size
        specs = [config.layer_spec(i) for i in range(config.num_layers)] if hasattr(config, "layer_spec") else []
        q_w = max([config.num_heads * sp.head_dim for sp in specs] or [config.num_heads * config.head_dim])
        kv_w = max([sp.num_kv_heads * sp.head_dim for sp in specs] or [config.num_kv_heads * config.head_dim])
        attn_w = max(h, q_w)
        return {"hidden": ((S, h), 2), "residual": ((S, h), 2), "qkv": ((S, q_w + 2 * kv_w), 2),
                "attn_out": ((S, attn_w), 2), "mlp_gate": ((S, inter), 2), "mlp_up": ((S, inter), 2),
                "mlp_out": ((S, max(h, kv_w)), 2), "logits": ((min(S, 64), config.vocab_size), 2),
                "norm_out": ((S, attn_w), 2), "hidden_f32": ((S, h), 4), "residual_f32": ((S, h), 4)}

    def allocate_scratch(self, config: ModelConfig, max_seq_len: int = 2048, device=None) -> ScratchBuffers:
        import torch
        dev = device if device is not None else (self.device if self.device is not None else "cpu")
        out = ScratchBuffers()
        for name, (shape, esz) in self.scratch_shapes(config, max_seq_len).items():
            setattr(out, name, torch.empty(shape, dtype=torch.float16 if esz == 2 else torch.float32, device=dev))
            out.total_bytes += shape[0] * shape[1] * esz
        self._allocated_bytes += out.total_bytes
        return out

    @classmethod
    def for_device(cls, device) -> "VRAMAllocator":
        import torch
        free, total = torch.cuda.mem_get_info(device)
        return cls(total, free, device)

    @property
    def usable_bytes(self) -> int:
        return int((self.total_bytes - self.CONTEXT_RESERVE) * (1 - self.SAFETY_FRACTION))

    def plan_allocation(self, config: ModelConfig, weight_bytes: int, scratch_bytes: int, block_size: int,
                        max_seq_len: int, max_batch_seqs: int, tp_size: int = 1,
                        kv_fraction: Optional[float] = None) -> VRAMPlan:
        """``weight_bytes`` / ``scratch_bytes``: what this rank has (or will have) resident besides the KV cache.
        ``kv_fraction`` overrides the demand rule with a share of what is left."""
        per_token = config.total_kv_cache_bytes_per_token // tp_size
        remaining = min(self.usable_bytes - weight_bytes - scratch_bytes,
                        self.free_bytes - self.FREE_MARGIN - scratch_bytes)
        if remaining < per_token * block_size:
            raise MemoryError(f"no room for a KV cache: {remaining / GB:.2f} GB left after weights "
                              f"({weight_bytes / GB:.2f} GB) and scratch ({scratch_bytes / GB:.2f} GB)")
        if kv_fraction is not None:
            kv = int(remaining * kv_fraction)
        else:
            kv = max(self.KV_FLOOR, int(max_batch_seqs * max_seq_len * per_token * 1.5))
        kv = min(kv, remaining)
        block_bytes = per_token * block_size
        blocks = kv // block_bytes
        return VRAMPlan(self.total_bytes, self.free_bytes, self.usable_bytes, weight_bytes, scratch_bytes,
                        blocks * block_bytes, blocks, block_size, max_seq_len, max_batch_seqs)

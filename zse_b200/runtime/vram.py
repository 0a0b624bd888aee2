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

    def summary(self) -> str:
        g = lambda b: f"{b / GB:.2f} GB"
        return (f"VRAM plan: total {g(self.total_bytes)}, free {g(self.free_bytes)}, weights {g(self.weight_bytes)}, "
                f"scratch {g(self.scratch_bytes)}, KV {g(self.kv_cache_bytes)} = {self.kv_blocks} blocks x "
                f"{self.block_size} tokens (max_seq_len {self.max_seq_len}, {self.max_batch_seqs} sequences)")


class VRAMAllocator:
    CONTEXT_RESERVE = 400 * MB
    SAFETY_FRACTION = 0.05
    KV_FLOOR = 256 * MB
    FREE_MARGIN = 1 * GB

    def __init__(self, total_bytes: int, free_bytes: Optional[int] = None):
        self.total_bytes = total_bytes
        self.free_bytes = total_bytes if free_bytes is None else free_bytes

    @classmethod
    def for_device(cls, device) -> "VRAMAllocator":
        import torch
        free, total = torch.cuda.mem_get_info(device)
        return cls(total, free)

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

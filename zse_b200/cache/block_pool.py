"""Fixed-size KV block pool over one device slab.

The slab is a single fp16 tensor ``[layers, blocks, 2 (K,V), kv_heads, block_size, head_dim]``: per layer every
block's K (and V) for one kv head is a contiguous ``block_size*head_dim`` run, which is what the attention kernels
stream.  Bookkeeping (free list, reference counts for shared/forked blocks) is host-side, as in
zse-engine/zse_engine/cache/block_pool.py:18-282; with ``device=None`` the pool only does bookkeeping, which is
how the CPU tests and the scheduler simulations use it.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, Optional

import torch


@dataclass
class Block:
    block_id: int
    ref_count: int = 1
    content_hash: Optional[int] = None
    seq_id: Optional[int] = None
    token_start: int = 0
    num_tokens: int = 0

    layer_block_bytes: int = 0       # bytes of this block inside one layer's section of the slab (K and V)

    @property
    def is_shared(self) -> bool:
        return self.ref_count > 1

    @property
    def gpu_offset(self) -> int:
        """Byte offset of the block inside a layer's section of the slab (the slab is layer-major, so a block has
        one such run per layer, all at this offset from their layer's start)."""
        return self.block_id * self.layer_block_bytes


class BlockPool:
    def __init__(self, num_blocks: int, block_size_tokens: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 device=None, dtype=torch.float16):
        if num_blocks <= 0:
            raise ValueError("the KV budget is smaller than one block")
        self._num_blocks = num_blocks
        self._block_size = block_size_tokens
        self._shape = (num_layers, num_blocks, 2, num_kv_heads, block_size_tokens, head_dim)
        self._bytes_per_token = num_layers * 2 * num_kv_heads * head_dim * 2
        self._free: Deque[int] = deque(range(num_blocks))
        self._blocks: Dict[int, Block] = {}
        self.slab: Optional[torch.Tensor] = None
        if device is not None:
            # zeros: masked-out tail tokens of a block are multiplied by probability 0 and must be finite
            self.slab = torch.zeros(self._shape, dtype=dtype, device=device)

    @classmethod
    def from_budget(cls, budget_bytes: int, block_size_tokens: int, num_layers: int, num_kv_heads: int,
                    head_dim: int, device=None) -> "BlockPool":
        block_bytes = block_size_tokens * num_layers * 2 * num_kv_heads * head_dim * 2
        return cls(budget_bytes // block_bytes, block_size_tokens, num_layers, num_kv_heads, head_dim, device)

    # ---- facts ----------------------------------------------------------------------------------------
    @property
    def block_size_tokens(self) -> int:
        return self._block_size

    @property
    def block_bytes(self) -> int:
        return self._block_size * self._bytes_per_token

    @property
    def bytes_per_token_all_layers(self) -> int:
        return self._bytes_per_token

    @property
    def num_blocks(self) -> int:
        return self._num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_allocated(self) -> int:
        return self._num_blocks - len(self._free)

    @property
    def total_bytes(self) -> int:
        return self._num_blocks * self.block_bytes

    @property
    def used_bytes(self) -> int:
        return self.num_allocated * self.block_bytes

    @property
    def utilization(self) -> float:
        return self.num_allocated / self._num_blocks

    # ---- addresses (zse-engine/zse_engine/cache/block_pool.py:163-258, for this pool's layer-major slab) -------
    @property
    def layer_block_bytes(self) -> int:
        _, _, two, kvh, bs, hd = self._shape
        return two * kvh * bs * hd * 2

    @property
    def is_uniform_kv(self) -> bool:
        """Every layer has the same row size in the pool: models whose layers differ (Gemma-4) get rows of the
        widest layer and narrower layers use a strided view of them."""
        return True

    def layer_kv_elems(self, layer: int) -> int:
        """K elements per token in the pool's rows (V is the same size)."""
        return self._shape[3] * self._shape[5]

    def layer_byte_offset(self, layer: int) -> int:
        """Byte offset of a layer's section inside the slab."""
        return layer * self._num_blocks * self.layer_block_bytes

    def _base_ptr(self) -> int:
        if self.slab is None:
            raise RuntimeError("this pool only does bookkeeping (no device slab)")
        return int(self.slab.data_ptr())

    def gpu_ptr_for_block_layer(self, block: Block, layer: int) -> int:
        """Address of the block's K run of ``layer`` (``[kv_heads, block_size, head_dim]`` fp16, V follows it)."""
        return self._base_ptr() + self.layer_byte_offset(layer) + block.block_id * self.layer_block_bytes

    def gpu_ptr_for_block(self, block: Block) -> int:
        return self.gpu_ptr_for_block_layer(block, 0)

    def gpu_ptr_for_kv(self, block: Block, layer: int, is_value: bool) -> int:
        return self.gpu_ptr_for_block_layer(block, layer) + (self.layer_block_bytes // 2 if is_value else 0)

    # ---- alloc / free ---------------------------------------------------------------------------------
    def alloc(self, seq_id: Optional[int] = None) -> Block:
        if not self._free:
            raise MemoryError("KV block pool exhausted")
        b = Block(self._free.popleft(), seq_id=seq_id, layer_block_bytes=self.layer_block_bytes)
        self._blocks[b.block_id] = b
        return b

    def increment_ref(self, block: Block) -> None:
        block.ref_count += 1

    def free(self, block: Block) -> bool:
        """Drops one reference; returns True when the block went back to the free list."""
        if block.block_id not in self._blocks:
            raise ValueError(f"double free of KV block {block.block_id}")
        block.ref_count -= 1
        if block.ref_count > 0:
            return False
        del self._blocks[block.block_id]
        block.num_tokens, block.content_hash = 0, None
        self._free.append(block.block_id)
        return True

    def get_block(self, block_id: int) -> Block:
        return self._blocks[block_id]

    def is_block_full(self, block: Block) -> bool:
        return block.num_tokens >= self._block_size

    def copy_block(self, src: Block, dst: Block) -> None:
        if self.slab is not None:
            self.slab[:, dst.block_id].copy_(self.slab[:, src.block_id])

    def stats(self) -> dict:
        return {"num_blocks": self._num_blocks, "free": self.num_free, "allocated": self.num_allocated,
                "block_size_tokens": self._block_size, "block_bytes": self.block_bytes,
                "shared": sum(1 for b in self._blocks.values() if b.is_shared)}

    def destroy(self) -> None:
        self.slab = None
        self._blocks.clear()
        self._free.clear()

"""Sequence -> ordered KV blocks, with copy-on-write and eviction holes
(zse-engine/zse_engine/cache/page_table.py:16-214).

An evicted block leaves a hole: its index stays in the sequence (the block table carries -1 there and attention
skips it) and the tokens it held no longer count as cached.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Set

import numpy as np

from .block_pool import Block, BlockPool


@dataclass
class SequenceEntry:
    seq_id: int
    blocks: List[Block] = field(default_factory=list)
    num_tokens: int = 0                      # logical length (positions 0..num_tokens-1), holes included
    evicted_indices: Set[int] = field(default_factory=set)
    tokens_evicted: int = 0
    version: int = 0                         # bumped by every change of `blocks` / `evicted_indices`
    _ids_np: Optional[np.ndarray] = field(default=None, repr=False, compare=False)
    _ids_version: int = field(default=-1, repr=False, compare=False)

    def touch(self) -> None:
        self.version += 1

    def block_ids_np(self) -> np.ndarray:
        """int32 block ids in order, -1 at holes; rebuilt only after the block list changed."""
        if self._ids_version != self.version or self._ids_np is None:
            ev = self.evicted_indices
            self._ids_np = np.fromiter((-1 if i in ev else b.block_id for i, b in enumerate(self.blocks)),
                                       dtype=np.int32, count=len(self.blocks))
            self._ids_version = self.version
        return self._ids_np

    @property
    def num_blocks(self) -> int:
        return len(self.blocks)

    @property
    def num_live_blocks(self) -> int:
        return len(self.blocks) - len(self.evicted_indices)


class PageTable:
    def __init__(self, pool: BlockPool):
        self._pool = pool
        self._seqs: Dict[int, SequenceEntry] = {}

    def create_sequence(self, seq_id: int) -> SequenceEntry:
        if seq_id in self._seqs:
            raise ValueError(f"sequence {seq_id} already exists")
        e = SequenceEntry(seq_id)
        self._seqs[seq_id] = e
        return e

    def has_sequence(self, seq_id: int) -> bool:
        return seq_id in self._seqs

    def get_entry(self, seq_id: int) -> SequenceEntry:
        return self._seqs[seq_id]

    def get_entry_or_none(self, seq_id: int) -> Optional[SequenceEntry]:
        return self._seqs.get(seq_id)

    def blocks_needed(self, seq_id: int, num_new_tokens: int) -> int:
        e = self._seqs[seq_id]
        bs = self._pool.block_size_tokens
        need = (e.num_tokens + num_new_tokens + bs - 1) // bs - len(e.blocks)
        tail_shared = bool(e.blocks) and e.num_tokens % bs != 0 and (len(e.blocks) - 1) not in e.evicted_indices \
            and e.blocks[-1].is_shared
        return max(0, need) + int(tail_shared)

    def append_tokens(self, seq_id: int, num_tokens: int) -> List[int]:
        """Grows the sequence; returns ids of newly allocated blocks.  A partly filled shared tail block is copied
        first (copy-on-write)."""
        e = self._seqs[seq_id]
        bs = self._pool.block_size_tokens
        new_ids: List[int] = []
        remaining = num_tokens
        while remaining > 0:
            if len(e.blocks) * bs <= e.num_tokens:          # every block so far is full
                b = self._pool.alloc(seq_id)
                b.token_start = len(e.blocks) * bs
                e.blocks.append(b)
                new_ids.append(b.block_id)
                e.touch()
            fill = e.num_tokens - (len(e.blocks) - 1) * bs
            tail_idx = len(e.blocks) - 1
            tail = e.blocks[tail_idx]
            if tail.is_shared and tail_idx not in e.evicted_indices:
                fresh = self._pool.alloc(seq_id)
                fresh.token_start, fresh.num_tokens = tail.token_start, tail.num_tokens
                self._pool.copy_block(tail, fresh)
                self._pool.free(tail)
                e.blocks[tail_idx] = tail = fresh
                new_ids.append(fresh.block_id)
                e.touch()
            take = min(remaining, bs - fill)
            tail.num_tokens = fill + take
            e.num_tokens += take
            remaining -= take
        return new_ids

    def get_block_ids(self, seq_id: int) -> List[int]:
        e = self._seqs[seq_id]
        return [-1 if i in e.evicted_indices else b.block_id for i, b in enumerate(e.blocks)]

    def block_ids_np(self, seq_id: int) -> np.ndarray:
        return self._seqs[seq_id].block_ids_np()

    def get_blocks(self, seq_id: int) -> List[Block]:
        e = self._seqs.get(seq_id)
        return [] if e is None else [b for i, b in enumerate(e.blocks) if i not in e.evicted_indices]

    def num_tokens(self, seq_id: int) -> int:
        return self._seqs[seq_id].num_tokens

    def num_blocks(self, seq_id: int) -> int:
        return len(self._seqs[seq_id].blocks)

    def remove_sequence(self, seq_id: int) -> List[Block]:
        e = self._seqs.pop(seq_id, None)
        if e is None:
            return []
        released = []
        for i, b in enumerate(e.blocks):
            if i not in e.evicted_indices and self._pool.free(b):
                released.append(b)
        return released

    def fork_sequence(self, src_id: int, dst_id: int) -> SequenceEntry:
        src = self._seqs[src_id]
        dst = self.create_sequence(dst_id)
        for i, b in enumerate(src.blocks):
            if i not in src.evicted_indices:
                self._pool.increment_ref(b)
            dst.blocks.append(b)
        dst.num_tokens = src.num_tokens
        dst.evicted_indices = set(src.evicted_indices)
        dst.touch()
        return dst

    def evict_block(self, seq_id: int, block_idx: int) -> Optional[Block]:
        e = self._seqs.get(seq_id)
        if e is None or block_idx >= len(e.blocks) or block_idx in e.evicted_indices:
            return None
        b = e.blocks[block_idx]
        e.evicted_indices.add(block_idx)
        e.touch()
        e.tokens_evicted += b.num_tokens
        self._pool.free(b)
        return b

    def get_all_sequences(self) -> List[int]:
        return list(self._seqs)

    @property
    def num_sequences(self) -> int:
        return len(self._seqs)

    def stats(self) -> dict:
        return {"num_sequences": len(self._seqs), "total_tokens": sum(e.num_tokens for e in self._seqs.values()),
                "total_blocks": sum(e.num_live_blocks for e in self._seqs.values())}

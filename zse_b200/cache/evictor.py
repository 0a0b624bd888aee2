"""Which KV block to drop under memory pressure (zse-engine/zse_engine/cache/evictor.py:42-199).

Policies: ``lru`` (oldest access), ``lfu`` (fewest accesses), ``smart`` =
``access_count / (1 + age) + (2.0 for prompt blocks, 0.5 for generated)``; the lowest score goes first.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Set


@dataclass
class BlockAccessInfo:
    seq_id: int
    block_idx: int
    block_id: int
    num_tokens: int
    access_count: int = 0
    last_access_time: float = 0.0
    token_start: int = 0
    is_prompt: bool = False


@dataclass
class EvictionCandidate:
    seq_id: int
    block_idx: int
    block_id: int
    score: float
    num_tokens: int


class Evictor:
    POLICIES = ("lru", "lfu", "smart")

    def __init__(self, policy: str = "smart", clock=time.monotonic):
        if policy not in self.POLICIES:
            raise ValueError(f"unknown eviction policy '{policy}' (choose from {self.POLICIES})")
        self._policy = policy
        self._clock = clock
        self._info: Dict[tuple, BlockAccessInfo] = {}     # (seq_id, block_id) -> info
        self._seq_touch: Dict[int, float] = {}            # seq_id -> time of the sequence's last step
        self._evictions = 0
        self._tokens_evicted = 0

    @property
    def policy(self) -> str:
        return self._policy

    @property
    def eviction_count(self) -> int:
        return self._evictions

    @property
    def total_tokens_evicted(self) -> int:
        return self._tokens_evicted

    def record_access(self, seq_id: int, block_idx: int, block_id: int, num_tokens: int, token_start: int = 0,
                      is_prompt: bool = False, now: Optional[float] = None) -> None:
        now = self._clock() if now is None else now
        key = (seq_id, block_id)
        info = self._info.get(key)
        if info is None:
            info = self._info[key] = BlockAccessInfo(seq_id, block_idx, block_id, num_tokens,
                                                     token_start=token_start, is_prompt=is_prompt)
        info.block_idx, info.num_tokens = block_idx, num_tokens
        info.access_count += 1
        info.last_access_time = now

    def record_batch_access(self, seq_id: int, block_ids: Iterable[int], block_size: int, prompt_len: int = 0) -> None:
        now = self._clock()
        for idx, bid in enumerate(block_ids):
            if bid >= 0:
                self.record_access(seq_id, idx, bid, block_size, idx * block_size, idx * block_size < prompt_len, now)

    def now(self) -> float:
        return self._clock()

    def touch_sequence(self, seq_id: int, now: Optional[float] = None) -> None:
        """Marks every block of the sequence as used now (one dictionary store per step instead of one per block)."""
        self._seq_touch[seq_id] = self._clock() if now is None else now

    def remove_block(self, block_id: int, seq_id: Optional[int] = None) -> None:
        for key in [k for k in self._info if k[1] == block_id and (seq_id is None or k[0] == seq_id)]:
            del self._info[key]

    def remove_sequence(self, seq_id: int) -> None:
        for key in [k for k in self._info if k[0] == seq_id]:
            del self._info[key]
        self._seq_touch.pop(seq_id, None)

    def _score(self, info: BlockAccessInfo, now: float) -> float:
        last = max(info.last_access_time, self._seq_touch.get(info.seq_id, 0.0))
        if self._policy == "lru":
            return last
        if self._policy == "lfu":
            return float(info.access_count)
        age = max(0.0, now - last)
        return info.access_count / (1.0 + age) + (2.0 if info.is_prompt else 0.5)

    def select_victims(self, num_blocks: int, exclude_seq_ids: Optional[Set[int]] = None) -> List[EvictionCandidate]:
        now = self._clock()
        skip = exclude_seq_ids or set()
        cands = [EvictionCandidate(i.seq_id, i.block_idx, i.block_id, self._score(i, now), i.num_tokens)
                 for i in self._info.values() if i.seq_id not in skip]
        cands.sort(key=lambda c: c.score)
        return cands[:num_blocks]

    def note_evicted(self, cand_tokens: int) -> None:
        self._evictions += 1
        self._tokens_evicted += cand_tokens

    def stats(self) -> dict:
        return {"policy": self._policy, "tracked_blocks": len(self._info), "eviction_count": self._evictions,
                "tokens_evicted": self._tokens_evicted}

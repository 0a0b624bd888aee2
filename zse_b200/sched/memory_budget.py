"""Predictive KV-block budget for admission control (zse-engine/zse_engine/zstreamer/memory_budget.py:30-202).

A request commits its prompt blocks plus ``headroom_ratio * max_tokens`` worth of blocks for what it may generate;
the head-room turns into actual usage as tokens are produced, and two blocks stay in reserve for emergencies.
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass
from typing import Dict

from .request import InferenceRequest


@dataclass
class _Commit:
    prompt_blocks: int
    headroom_blocks: int
    decode_blocks: int = 0

    @property
    def total(self) -> int:
        return self.prompt_blocks + max(self.headroom_blocks, self.decode_blocks)


MemoryReservation = _Commit      # the reference's name for the per-request record


class MemoryBudget:
    def __init__(self, total_blocks: int, block_size: int, headroom_ratio: float = 0.5, reserve_blocks: int = 2):
        self._total = total_blocks
        self._bs = block_size
        self._ratio = headroom_ratio
        self._reserve = reserve_blocks
        self._commits: Dict[str, _Commit] = {}
        self._lock = threading.Lock()

    def _tokens_to_blocks(self, tokens: int) -> int:
        return (tokens + self._bs - 1) // self._bs if tokens > 0 else 0

    def _estimate(self, req: InferenceRequest) -> _Commit:
        prompt = self._tokens_to_blocks(req.prompt_len + req.num_generated)
        remaining = max(0, req.params.max_tokens - req.num_generated)
        head = self._tokens_to_blocks(int(math.ceil(remaining * self._ratio))) + 1
        return _Commit(prompt, head)

    @property
    def committed_blocks(self) -> int:
        return sum(c.total for c in self._commits.values())

    @property
    def available_blocks(self) -> int:
        return max(0, self._total - self._reserve - self.committed_blocks)

    @property
    def utilization(self) -> float:
        return self.committed_blocks / self._total if self._total else 1.0

    def can_admit(self, request: InferenceRequest) -> bool:
        with self._lock:
            if request.request_id in self._commits:
                return True
            return self._estimate(request).total <= self._total - self._reserve - self.committed_blocks

    def can_admit_n(self, requests) -> int:
        """How many of ``requests``, taken in order, fit next to what is committed already
        (zse-engine/zse_engine/zstreamer/memory_budget.py:100-115)."""
        with self._lock:
            left = self._total - self._reserve - self.committed_blocks
            n = 0
            for req in requests:
                cost = 0 if req.request_id in self._commits else self._estimate(req).total
                if cost > left:
                    break
                left -= cost
                n += 1
            return n

    def preemption_candidates(self, blocks_needed: int) -> list:
        """Ids of committed requests, largest first, whose release frees at least ``blocks_needed`` blocks (all of
        them when even that is not enough)."""
        with self._lock:
            out, freed = [], 0
            for rid, c in sorted(self._commits.items(), key=lambda kv: -kv[1].total):
                if freed >= blocks_needed:
                    break
                out.append(rid)
                freed += c.total
            return out

    def fits_at_all(self, req: InferenceRequest) -> bool:
        """False when the request could never run, even on an empty cache."""
        return self._tokens_to_blocks(req.prompt_len + req.params.max_tokens) <= self._total - self._reserve

    def reserve(self, request: InferenceRequest) -> None:
        with self._lock:
            self._commits.setdefault(request.request_id, self._estimate(request))

    def release(self, request_id: str) -> None:
        with self._lock:
            self._commits.pop(request_id, None)

    def update_decode_progress(self, request_id: str, tokens_generated: int) -> None:
        with self._lock:
            c = self._commits.get(request_id)
            if c is not None:
                c.decode_blocks = self._tokens_to_blocks(tokens_generated) + 1

    def resize(self, total_blocks: int) -> None:
        with self._lock:
            self._total = total_blocks

    def stats(self) -> dict:
        with self._lock:
            committed = sum(c.total for c in self._commits.values())
            return {"total_blocks": self._total, "committed_blocks": committed,
                    "available_blocks": max(0, self._total - self._reserve - committed),
                    "utilization": committed / self._total if self._total else 1.0,
                    "num_requests": len(self._commits), "block_size": self._bs, "headroom_ratio": self._ratio}

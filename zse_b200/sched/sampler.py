"""Host-side sampler with the reference's semantics (zse-engine/zse_engine/orchestrator/sampler.py:21-213).

The serving path selects tokens on the device (``ops.sample``); this class is the CPU statement of the same rules -
repetition penalty ``p^(1+log2(count))``, temperature, top-k (keep values >= the k-th largest), top-p (smallest
sorted prefix reaching p), categorical draw - used by the CPU engine path, by tests as the oracle of the device
sampler, and by callers that have logits on the host.
"""
from __future__ import annotations

import math
import random
from typing import Dict, Optional, Sequence

import torch

from ..ops import reference as ref


class Sampler:
    def __init__(self, seed: Optional[int] = None):
        self._rng = random.Random(seed)

    @staticmethod
    def _logits(logits, vocab_size: Optional[int]) -> torch.Tensor:
        """A tensor, an array, or - the reference's form - the raw fp16 bytes of a row together with ``vocab_size``
        (rows may be padded: only the first ``vocab_size`` values count)."""
        if isinstance(logits, (bytes, bytearray, memoryview)):
            import numpy as np
            n = len(logits) // 2 if vocab_size is None else int(vocab_size)
            if len(logits) < 2 * n:
                raise ValueError(f"Expected {2 * n} bytes, got {len(logits)}")
            return torch.from_numpy(np.frombuffer(logits, dtype=np.float16, count=n).astype(np.float32))
        x = torch.as_tensor(logits).float().flatten()
        return x if vocab_size is None else x[: int(vocab_size)]

    def sample(self, logits=None, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
               repetition_penalty: float = 1.0, past_tokens=None, seed: Optional[int] = None,
               vocab_size: Optional[int] = None, logits_bytes=None) -> int:
        """``past_tokens``: token -> count, or a plain collection of token ids (each counted once)."""
        x = self._logits(logits_bytes if logits is None else logits, vocab_size)
        if past_tokens is not None and not isinstance(past_tokens, dict):
            past_tokens = {int(t): 1 for t in past_tokens}
        if repetition_penalty != 1.0 and past_tokens:
            x = ref.apply_repetition_penalty(x, past_tokens, repetition_penalty)
        if temperature <= 0.0 or top_k == 1:
            return int(x.argmax())
        p = ref.filtered_probs(x, temperature, top_k, top_p)
        rng = random.Random(seed) if seed is not None else self._rng
        u = rng.random()
        c = torch.cumsum(p, dim=0)
        return int(min(int(torch.searchsorted(c, torch.tensor(u, dtype=c.dtype))), p.numel() - 1))

    @staticmethod
    def greedy(logits=None, vocab_size: Optional[int] = None, logits_bytes=None) -> int:
        return int(Sampler._logits(logits_bytes if logits is None else logits, vocab_size).argmax())

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

    def sample(self, logits, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
               repetition_penalty: float = 1.0, past_tokens: Optional[Dict[int, int]] = None,
               seed: Optional[int] = None) -> int:
        x = torch.as_tensor(logits).float().flatten()
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
    def greedy(logits) -> int:
        return int(torch.as_tensor(logits).float().argmax())

"""Accept / reject rule of speculative decoding (zse-engine/zse_engine/zstreamer/verifier.py:24-209).

Leviathan / Chen rejection sampling: draft token ``x`` proposed with probability ``q(x)`` is accepted with
probability ``min(1, p(x)/q(x))``; on rejection the replacement is drawn from ``max(0, p - q)`` renormalised; when
every draft token is accepted one bonus token is drawn from the next target distribution.  The output distribution
equals the target's.  Greedy mode accepts while the draft equals the target arg-max.
"""
from __future__ import annotations

import random
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass
class VerifyResult:
    accepted_tokens: List[int]        # tokens to append (accepted drafts + one corrected / bonus token)
    num_drafted: int
    num_accepted: int                 # drafts accepted (excludes the final corrected / bonus token)

    @property
    def acceptance_rate(self) -> float:
        return self.num_accepted / self.num_drafted if self.num_drafted else 0.0


class SpeculativeVerifier:
    def __init__(self, seed: Optional[int] = None):
        self._rng = random.Random(seed)
        self.total_drafted = self.total_accepted = self.total_steps = 0

    def verify_greedy(self, draft_tokens: Sequence[int], target_argmax: Sequence[int]) -> VerifyResult:
        """``target_argmax[i]`` = arg-max of the target after consuming the last accepted token and drafts ``[:i]``
        (length ``len(draft)+1``)."""
        out: List[int] = []
        n_acc = 0
        for i, d in enumerate(draft_tokens):
            if int(target_argmax[i]) == int(d):
                out.append(int(d))
                n_acc += 1
            else:
                break
        out.append(int(target_argmax[n_acc]))
        return self._record(VerifyResult(out, len(draft_tokens), n_acc))

    def verify_stochastic(self, draft_tokens: Sequence[int], draft_probs: Sequence[torch.Tensor],
                          target_probs: Sequence[torch.Tensor]) -> VerifyResult:
        """``draft_probs[i]`` / ``target_probs[i]``: distributions ``[vocab]`` at draft position i;
        ``target_probs`` has one more entry for the bonus token."""
        out: List[int] = []
        n_acc = 0
        for i, d in enumerate(draft_tokens):
            p, q = float(target_probs[i][d]), float(draft_probs[i][d])
            if q <= 0.0 or self._rng.random() < min(1.0, p / q):
                if q <= 0.0 and p <= 0.0:
                    pass
                else:
                    out.append(int(d))
                    n_acc += 1
                    continue
            resid = (target_probs[i].float() - draft_probs[i].float()).clamp(min=0)
            z = float(resid.sum())
            dist = resid / z if z > 0 else target_probs[i].float()
            out.append(self._draw(dist))
            return self._record(VerifyResult(out, len(draft_tokens), n_acc))
        out.append(self._draw(target_probs[len(draft_tokens)].float()))
        return self._record(VerifyResult(out, len(draft_tokens), n_acc))

    def verify_and_accept(self, draft_tokens: Sequence[int], draft_probs, target_logits_list, vocab_size: int,
                          temperature: float = 1.0):
        """The reference's entry point (zse-engine/zse_engine/zstreamer/verifier.py:37-110): ``target_logits_list`` holds
        K+1 rows of raw fp16 logits (bytes) or tensors; returns ``(accepted_tokens, num_draft_accepted)``."""
        import numpy as np
        rows = []
        for row in target_logits_list:
            if isinstance(row, (bytes, bytearray, memoryview)):
                row = torch.from_numpy(np.frombuffer(row, dtype=np.float16)[:vocab_size].astype(np.float32))
            rows.append(torch.as_tensor(row, dtype=torch.float32)[:vocab_size])
        if len(rows) != len(draft_tokens) + 1:
            raise ValueError("one more row of target logits than drafts is required")
        if temperature is None or temperature < 1e-6:
            r = self.verify_greedy(draft_tokens, [int(x.argmax()) for x in rows])
        else:
            target = [torch.softmax(x / temperature, dim=-1) for x in rows]
            draft = [torch.as_tensor(d, dtype=torch.float32)[:vocab_size] for d in draft_probs]
            r = self.verify_stochastic(draft_tokens, draft, target)
        return r.accepted_tokens, r.num_accepted

    def _draw(self, dist: torch.Tensor) -> int:
        u = self._rng.random() * float(dist.sum())
        c = torch.cumsum(dist, dim=0)
        return int(min(int(torch.searchsorted(c, torch.tensor(u, dtype=c.dtype))), dist.numel() - 1))

    def _record(self, r: VerifyResult) -> VerifyResult:
        self.total_drafted += r.num_drafted
        self.total_accepted += r.num_accepted
        self.total_steps += 1
        return r

    def stats(self) -> dict:
        return {"steps": self.total_steps, "drafted": self.total_drafted, "accepted": self.total_accepted,
                "acceptance_rate": self.total_accepted / self.total_drafted if self.total_drafted else 0.0}


def acceptance_rate(num_draft_accepted: int, K: int) -> float:
    return num_draft_accepted / K if K > 0 else 0.0


def effective_tokens_per_step(num_tokens_produced: int) -> float:
    """Tokens one target pass yielded (1 without drafts, up to K+1 with them)."""
    return float(num_tokens_produced)

"""Speculative decoding on the batched engine.

Per step and per sequence: propose up to K draft tokens (n-gram lookup or self-draft), then verify ALL sequences in
one packed pass: the rows ``[last token, d1..dK]`` of every sequence go through the causal paged-attention path at
their true cache positions, so each row sees the whole past (the reference's ``verify_tokens`` ignores
``start_position`` and only attends inside the K+1 window, zse-engine/zse_engine/orchestrator/model_runner.py:761-841,
and its engine never builds a ``SpeculativeRunner``, zstreamer/engine.py:321-328).  Accepted tokens are appended, the
KV of rejected positions is rolled back with ``truncate_sequence``.  Greedy requests only: the device arg-max of every
row is compared with the drafts, so the output is exactly the non-speculative greedy output.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

from ..runtime.runner import ModelRunner
from .draft_model import make_draft_model
from .request import InferenceRequest
from .verifier import SpeculativeVerifier


@dataclass
class SpeculativeResult:
    """What one speculative step gave one sequence (zse-engine/zse_engine/zstreamer/spec_runner.py:29-35)."""
    request_id: str
    accepted_tokens: List[int]
    num_draft_accepted: int
    total_tokens: int


class SpeculativeRunner:
    def __init__(self, runner: ModelRunner, k: int = 4, mode: str = "ngram", vocab_size: int = 0):
        self.runner, self.k, self.mode = runner, int(k), mode
        self._drafts: Dict[str, object] = {}
        self._verifier = SpeculativeVerifier()
        self.tokens_emitted = 0
        self.seq_steps = 0

    def _draft_for(self, r: InferenceRequest):
        d = self._drafts.get(r.request_id)
        if d is None:
            d = make_draft_model(self.mode)
            d.reset(r.prompt_tokens + r.output_tokens)
            self._drafts[r.request_id] = d
        return d

    def forget(self, request_id: str) -> None:
        self._drafts.pop(request_id, None)

    def step(self, reqs: Sequence[InferenceRequest], scheduler, adapters: Optional[Sequence[int]] = None) -> int:
        """One speculative step for every request in ``reqs`` (all greedy); returns the number of tokens emitted."""
        cache, runner = self.runner.cache, self.runner
        items, drafts, rows_of = [], [], []
        for r in reqs:
            d = self._draft_for(r)
            room = min(self.k, r.params.max_tokens - r.num_generated - 1,
                       runner.max_seq_len - cache.num_tokens(r.seq_id) - 2)
            prop = d.propose(room) if room > 0 else []
            start = cache.num_tokens(r.seq_id)          # position of the last generated token (not yet in the cache)
            cache.extend_sequence(r.seq_id, 1 + len(prop))
            items.append((r.seq_id, [r.output_tokens[-1]] + prop, start))
            drafts.append(prop)
        # split into passes that fit the logits buffer / token limits
        max_rows = min(runner.buf.logits.shape[0], runner.max_tokens)
        emitted, i = 0, 0
        while i < len(items):
            j, rows = i, 0
            while j < len(items) and rows + len(items[j][1]) <= max_rows and j - i < runner.max_batch_seqs:
                rows += len(items[j][1])
                j += 1
            if j == i:
                raise RuntimeError("speculative window larger than the logits buffer")
            toks, _ = runner.prefill(items[i:j], all_logits=True,
                                     adapters=None if adapters is None else list(adapters[i:j]))
            at = 0
            for idx in range(i, j):
                r, prop = reqs[idx], drafts[idx]
                n = 1 + len(prop)
                res = self._verifier.verify_greedy(prop, toks[at:at + n])
                at += n
                r.spec_drafted += len(prop)
                r.spec_accepted += res.num_accepted
                # KV now holds last + all drafts; keep last + accepted drafts
                keep = items[idx][2] + 1 + res.num_accepted
                cache.truncate_sequence(r.seq_id, keep)
                d = self._drafts[r.request_id]
                for t in res.accepted_tokens:
                    if r.is_finished:
                        break
                    scheduler.on_token_generated(r, t)
                    d.extend([t])
                    emitted += 1
                if r.is_finished:
                    # tokens after a stop are dropped; the cache is freed by the batch runner anyway
                    pass
                self.seq_steps += 1
            i = j
        self.tokens_emitted += emitted
        return emitted

    # ---- the reference's per-request entry points and figures (spec_runner.py:73-245) -------------------------
    def batched_speculative_step(self, requests: Sequence[InferenceRequest], scheduler, K: Optional[int] = None,
                                 adapters: Optional[Sequence[int]] = None) -> List[SpeculativeResult]:
        """One step for every request (ONE packed verification pass); a result per request with the tokens it got.
        The tokens are delivered to ``scheduler.on_token_generated`` as in ``step``."""
        before = [(r.num_generated, r.spec_accepted) for r in requests]
        old_k = self.k
        if K is not None:
            self.k = int(K)
        try:
            self.step(requests, scheduler, adapters)
        finally:
            self.k = old_k
        out = []
        for r, (n0, a0) in zip(requests, before):
            toks = list(r.output_tokens[n0:])
            out.append(SpeculativeResult(r.request_id, toks, r.spec_accepted - a0, len(toks)))
        return out

    def speculative_step(self, request: InferenceRequest, scheduler, K: Optional[int] = None) -> SpeculativeResult:
        return self.batched_speculative_step([request], scheduler, K)[0]

    @property
    def acceptance_rate(self) -> float:
        return self._verifier.stats()["acceptance_rate"]

    @property
    def tokens_per_step(self) -> float:
        return self.tokens_emitted / self.seq_steps if self.seq_steps else 0.0

    @property
    def speedup_factor(self) -> float:
        """Tokens per pass of the target model (a plain decode step yields one)."""
        return self.tokens_per_step

    def summary(self) -> str:
        s = self.stats()
        return (f"Speculative decoding ({self.mode}, k={self.k}): {s['steps']} steps, {s['drafted']} drafts, "
                f"{s['accepted']} accepted ({s['acceptance_rate']:.1%}), {self.tokens_per_step:.2f} tokens per step")

    def stats(self) -> dict:
        s = self._verifier.stats()
        s.update({"k": self.k, "mode": self.mode, "tokens_emitted": self.tokens_emitted,
                  "tokens_per_seq_step": self.tokens_emitted / self.seq_steps if self.seq_steps else 0.0})
        return s

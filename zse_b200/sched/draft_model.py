"""Draft proposers for speculative decoding (zse-engine/zse_engine/zstreamer/draft_model.py:26-259).

``NGramDraftModel`` proposes the continuation that followed the most recent earlier occurrence of the current
(n-1)-token suffix in the sequence's own context ("prompt lookup").  The table is kept incrementally - O(1) per
appended token - instead of being rebuilt from the whole context on every call, and no ``[vocab]``-sized Python
lists are produced: a draft is a short list of token ids (their proposal probability is taken as 1, which is the
greedy-verification case).  ``SelfDraftModel`` repeats the last accepted token, the reference's "self-draft".
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple


class DraftModel:
    """The reference's interface (zse-engine/zse_engine/zstreamer/draft_model.py:26-50): ``generate_drafts(context,
    K)`` returns K token ids and K probability lists of ``vocab_size`` entries.  The engine itself uses the
    incremental ``reset / extend / propose`` calls below, which never build vocabulary-sized lists."""

    _vocab_size = 0
    confidence = 0.8

    def vocab_size(self) -> int:
        return self._vocab_size

    def _dist(self, token: int) -> List[float]:
        """``confidence`` on ``token``, the rest spread evenly (the shape of the reference's draft distributions)."""
        v = max(self._vocab_size, token + 1, 1)
        if v == 1:
            return [1.0]
        rest = (1.0 - self.confidence) / (v - 1)
        probs = [rest] * v
        probs[token] = self.confidence
        return probs

    def generate_drafts(self, context_tokens: Sequence[int], K: int) -> Tuple[List[int], List[List[float]]]:
        self.reset(context_tokens)
        drafts = self.propose(K)
        fill = drafts[-1] if drafts else (int(context_tokens[-1]) if len(context_tokens) else 0)
        drafts = (drafts + [fill] * K)[:K]              # always K drafts, like the reference
        return drafts, [self._dist(t) for t in drafts]


class NGramDraftModel(DraftModel):
    def __init__(self, vocab_size_val: int = 0, n: int = 3, confidence: float = 0.8, min_n: int = 2):
        if n < 2:
            raise ValueError("n must be >= 2")
        self._vocab_size = int(vocab_size_val)
        self.n, self.min_n, self.confidence = n, max(2, min_n), confidence
        self._ctx: List[int] = []
        # per order k (context length k-1): suffix tuple -> position right after its latest occurrence
        self._tables: Dict[int, Dict[Tuple[int, ...], int]] = {k: {} for k in range(self.min_n, n + 1)}

    def reset(self, context: Sequence[int] = ()) -> None:
        self._ctx = []
        for t in self._tables.values():
            t.clear()
        self.extend(context)

    def extend(self, tokens: Sequence[int]) -> None:
        ctx = self._ctx
        for tok in tokens:
            ctx.append(int(tok))
            end = len(ctx)
            # the (k-1)-gram that ends right before the new token now has a known continuation at end-1
            for k, table in self._tables.items():
                if end - 1 >= k - 1:
                    table[tuple(ctx[end - k: end - 1])] = end - 1

    update = extend          # the reference's name for feeding tokens

    def truncate(self, length: int) -> None:
        if length < len(self._ctx):
            self.reset(self._ctx[:length])

    def __len__(self) -> int:
        return len(self._ctx)

    def propose(self, k: int) -> List[int]:
        """Up to ``k`` draft tokens continuing the current context (empty when no earlier occurrence exists)."""
        ctx = self._ctx
        for order in range(self.n, self.min_n - 1, -1):
            if len(ctx) < order - 1:
                continue
            start = self._tables[order].get(tuple(ctx[len(ctx) - (order - 1):]))
            if start is None or start >= len(ctx):
                continue
            out = ctx[start: start + k]
            if out:
                return list(out)
        return []


class SelfDraftModel(DraftModel):
    """Proposes the last token again k times (cheap, and right whenever the model is in a repetition)."""

    def __init__(self, vocab_size_val: int = 0, confidence: float = 0.9):
        self._vocab_size, self.confidence = int(vocab_size_val), confidence
        self._last: Optional[int] = None

    def set_last_logits(self, logits_bytes) -> None:
        """The reference feeds the last fp16 logits and drafts their arg-max; same effect here."""
        import numpy as np
        arr = np.frombuffer(logits_bytes, dtype=np.float16) if isinstance(logits_bytes, (bytes, bytearray, memoryview)) \
            else np.asarray(logits_bytes)
        if arr.size:
            self._last = int(arr.argmax())

    def reset(self, context: Sequence[int] = ()) -> None:
        self._last = int(context[-1]) if len(context) else None

    def extend(self, tokens: Sequence[int]) -> None:
        if len(tokens):
            self._last = int(tokens[-1])

    def truncate(self, length: int) -> None:
        pass

    def propose(self, k: int) -> List[int]:
        return [] if self._last is None else [self._last] * k


def make_draft_model(mode: str):
    if mode == "ngram":
        return NGramDraftModel()
    if mode == "self":
        return SelfDraftModel()
    raise ValueError(f"unknown speculative mode '{mode}' (ngram | self)")

"""Cross-encoder style reranking with the served model: one prefill per (query, passage) pair, score = logit("Yes") -
logit("No") after a fixed judging prompt (zse-engine/zse_engine/rag/reranker.py:30-166)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

PROMPT = ("Judge whether the passage helps answer the question. Reply Yes or No.\n\nQuestion: {q}\n\nPassage: {d}\n\n"
          "Does the passage help answer the question? Answer:")


class LLMReranker:
    def __init__(self, engine, tokenizer=None, doc_max_tokens: int = 384):
        """``engine``: anything with ``last_token_logits(list[int])`` (``ZStreamerEngine``)."""
        self._engine = engine
        self._tok = tokenizer if tokenizer is not None else getattr(engine, "tokenizer", None)
        self._doc_max = doc_max_tokens
        self._yes: Optional[int] = None
        self._no: Optional[int] = None

    def _resolve_yes_no(self) -> bool:
        if self._yes is not None and self._no is not None:
            return True
        if self._tok is None:
            return False
        for yes, no in ((" Yes", " No"), ("Yes", "No"), (" yes", " no")):
            y, n = self._tok.encode(yes), self._tok.encode(no)
            if y and n and y[-1] != n[-1]:
                self._yes, self._no = int(y[-1]), int(n[-1])
                return True
        return False

    def _truncate(self, text: str, max_tokens: int) -> str:
        ids = self._tok.encode(text)
        return text if len(ids) <= max_tokens else self._tok.decode(ids[:max_tokens])

    def score_pair(self, query: str, doc_text: str) -> float:
        """Higher = more relevant; 0.0 when anything goes wrong, so that callers keep the retrieval order."""
        if not self._resolve_yes_no():
            return 0.0
        try:
            ids = list(self._tok.encode(PROMPT.format(q=query.strip(), d=self._truncate(doc_text, self._doc_max))))
            if not ids:
                return 0.0
            logits = self._engine.last_token_logits(ids[-1024:])
            return float(logits[self._yes]) - float(logits[self._no])
        except Exception:
            return 0.0

    def rerank(self, query: str, candidates: Sequence[Tuple[int, str]], top_n: int = 5) -> List[Tuple[int, float]]:
        scored = [(cid, self.score_pair(query, text)) for cid, text in candidates]
        scored.sort(key=lambda x: -x[1])
        return scored[:top_n]

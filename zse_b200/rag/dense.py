"""Dense embeddings from the served model itself: the mean-pooled, L2-normalised final hidden state of a text
(zse-engine/zse_engine/rag/dense_embedder.py:21-131).  Pooling and normalisation happen on the device
(``ModelRunner.embed_pooled``); access goes through the engine so that it is serialised with serving steps."""
from __future__ import annotations

from typing import List, Optional

import numpy as np


class DenseEmbedder:
    def __init__(self, engine, tokenizer=None):
        """``engine``: anything with ``embed_tokens(list[int]) -> tensor/array`` (``ZStreamerEngine``)."""
        self._engine = engine
        self._tok = tokenizer if tokenizer is not None else getattr(engine, "tokenizer", None)
        self._dim: Optional[int] = None

    @property
    def dim(self) -> int:
        if self._dim is None:
            cfg = getattr(self._engine, "model_config", None)
            self._dim = int(getattr(cfg, "hidden_size", 0) or 0)
        return self._dim

    def _tokenize(self, text: str, max_tokens: int) -> List[int]:
        ids = list(self._tok.encode(text)) if self._tok is not None else []
        return ids[:max_tokens]

    def embed(self, text: str, max_tokens: int = 512) -> Optional[bytes]:
        ids = self._tokenize(text, max_tokens)
        if not ids:
            return None
        try:
            v = self._engine.embed_tokens(ids)
        except Exception:
            return None
        arr = np.asarray(v, dtype=np.float32).reshape(-1)
        self._dim = arr.shape[0]
        return arr.tobytes()

    def embed_query(self, text: str) -> Optional[bytes]:
        return self.embed(text, max_tokens=256)

    def embed_batch(self, texts: List[str], max_tokens: int = 512) -> List[Optional[bytes]]:
        return [self.embed(t, max_tokens) for t in texts]

    @staticmethod
    def cosine(a: bytes, b: bytes) -> float:
        x, y = np.frombuffer(a, np.float32), np.frombuffer(b, np.float32)
        if x.shape != y.shape or x.size == 0:
            return 0.0
        d = float(np.linalg.norm(x) * np.linalg.norm(y))
        return float(np.dot(x, y)) / d if d > 0 else 0.0


def dense_cosine(query_emb: bytes, doc_emb: bytes, dtype=np.float32) -> float:
    """Cosine similarity of two stored embeddings (the reference's helper, zse-engine/zse_engine/rag/
    dense_embedder.py:119-131).  Vectors of this package are fp32; pass ``dtype=np.float16`` for blobs written by the
    reference."""
    if not query_emb or not doc_emb or len(query_emb) != len(doc_emb):
        return 0.0
    x, y = np.frombuffer(query_emb, dtype).astype(np.float32), np.frombuffer(doc_emb, dtype).astype(np.float32)
    d = float(np.linalg.norm(x) * np.linalg.norm(y))
    return float(np.dot(x, y)) / d if d > 0 else 0.0

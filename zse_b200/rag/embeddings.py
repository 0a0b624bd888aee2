"""Lexical scoring for retrieval: Okapi BM25 and sparse TF-IDF vectors over the model's own token ids
(behaviour of zse-engine/zse_engine/rag/embeddings.py:20-285: BM25 k1 = 1.5, b = 0.75; TF normalised by the most
frequent token, IDF = log(1 + N / (1 + df)) floored at 0.1, unit-length vectors stored as bytes).

Sparse vectors are stored as two packed arrays (uint32 token ids, float32 weights) and compared with numpy.
"""
from __future__ import annotations

import math
import re
import struct
import zlib
from collections import Counter
from typing import Dict, Iterable, List, Optional, Sequence, Set

import numpy as np

_WORD = re.compile(r"[A-Za-z0-9_]+|[^\sA-Za-z0-9_]")


def hash_tokenize(text: str, vocab_size: int) -> List[int]:
    """Tokenizer-free fallback: lower-cased words hashed into the vocabulary range."""
    return [zlib.crc32(w.encode("utf-8")) % vocab_size for w in _WORD.findall(text.lower())]


class BM25Scorer:
    def __init__(self, k1: float = 1.5, b: float = 0.75):
        self.k1, self.b = k1, b
        self._docs: Dict[int, Counter] = {}
        self._len: Dict[int, int] = {}
        self._df: Counter = Counter()
        self._postings: Dict[int, Set[int]] = {}
        self._total_len = 0
        self._next = 0

    def __len__(self) -> int:
        return len(self._docs)

    @property
    def avg_len(self) -> float:
        return self._total_len / len(self._docs) if self._docs else 0.0

    def add_document(self, tokens: Sequence[int]) -> int:
        doc_id = self._next
        self._next += 1
        tf = Counter(tokens)
        self._docs[doc_id] = tf
        self._len[doc_id] = len(tokens)
        self._total_len += len(tokens)
        for t in tf:
            self._df[t] += 1
            self._postings.setdefault(t, set()).add(doc_id)
        return doc_id

    def remove_document(self, doc_id: int) -> None:
        tf = self._docs.pop(doc_id, None)
        if tf is None:
            return
        self._total_len -= self._len.pop(doc_id)
        for t in tf:
            self._df[t] -= 1
            post = self._postings.get(t)
            if post is not None:
                post.discard(doc_id)
                if not post:
                    del self._postings[t]
            if self._df[t] <= 0:
                del self._df[t]

    def idf(self, token: int) -> float:
        n, df = len(self._docs), self._df.get(token, 0)
        return math.log(1.0 + (n - df + 0.5) / (df + 0.5))

    def score(self, query_tokens: Sequence[int], doc_id: int) -> float:
        tf = self._docs.get(doc_id)
        if tf is None:
            return 0.0
        norm = self.k1 * (1.0 - self.b + self.b * self._len[doc_id] / max(self.avg_len, 1e-9))
        s = 0.0
        for t in set(query_tokens):
            f = tf.get(t, 0)
            if f:
                s += self.idf(t) * f * (self.k1 + 1.0) / (f + norm)
        return s

    def score_all(self, query_tokens: Sequence[int]) -> Dict[int, float]:
        """Scores of every document that shares at least one token with the query."""
        cands: Set[int] = set()
        for t in set(query_tokens):
            cands |= self._postings.get(t, set())
        return {d: self.score(query_tokens, d) for d in cands}


def sparse_to_bytes(weights: Dict[int, float]) -> bytes:
    if not weights:
        return b""
    ids = np.fromiter(sorted(weights), dtype=np.uint32, count=len(weights))
    vals = np.fromiter((weights[int(i)] for i in ids), dtype=np.float32, count=len(weights))
    return struct.pack("<I", len(ids)) + ids.tobytes() + vals.tobytes()


def bytes_to_sparse(blob: bytes):
    if not blob:
        return np.zeros(0, np.uint32), np.zeros(0, np.float32)
    n = struct.unpack_from("<I", blob, 0)[0]
    ids = np.frombuffer(blob, dtype=np.uint32, count=n, offset=4)
    vals = np.frombuffer(blob, dtype=np.float32, count=n, offset=4 + 4 * n)
    return ids, vals


def sparse_cosine(a: bytes, b: bytes) -> float:
    ia, va = bytes_to_sparse(a)
    ib, vb = bytes_to_sparse(b)
    if len(ia) == 0 or len(ib) == 0:
        return 0.0
    _, pa, pb = np.intersect1d(ia, ib, assume_unique=True, return_indices=True)
    if len(pa) == 0:
        return 0.0
    dot = float(np.dot(va[pa], vb[pb]))
    na, nb = float(np.linalg.norm(va)), float(np.linalg.norm(vb))
    return dot / (na * nb) if na > 0 and nb > 0 else 0.0


class TokenEmbedder:
    """TF-IDF vectors + a BM25 index keyed by chunk id."""

    def __init__(self, tokenizer=None, vocab_size: int = 32000, bm25_weight: float = 0.5):
        self._tok = tokenizer
        self.vocab_size = vocab_size
        self.bm25_weight = bm25_weight
        self._doc_count = 0
        self._doc_freq: Counter = Counter()
        self._bm25 = BM25Scorer()
        self._chunk_to_bm25: Dict[int, int] = {}
        self._bm25_to_chunk: Dict[int, int] = {}

    def tokenize(self, text: str) -> List[int]:
        if self._tok is not None:
            try:
                return list(self._tok.encode(text, add_bos=False))
            except TypeError:
                return list(self._tok.encode(text))
            except Exception:
                pass
        return hash_tokenize(text, self.vocab_size)

    _tokenize = tokenize        # name used by the reference engine

    def embed(self, text: str) -> bytes:
        tokens = self.tokenize(text)
        if not tokens:
            return b""
        tf = Counter(tokens)
        top = max(tf.values())
        w = {}
        for t, f in tf.items():
            idf = 1.0
            if self._doc_count > 0 and t in self._doc_freq:
                idf = math.log(1.0 + self._doc_count / (1.0 + self._doc_freq[t]))
            w[t] = (f / top) * max(idf, 0.1)
        norm = math.sqrt(sum(v * v for v in w.values()))
        if norm > 0:
            w = {t: v / norm for t, v in w.items()}
        return sparse_to_bytes(w)

    def update_idf(self, token_sets: Iterable[Set[int]]) -> None:
        for ts in token_sets:
            self._doc_count += 1
            self._doc_freq.update(ts)

    def similarity(self, a: bytes, b: bytes) -> float:
        return sparse_cosine(a, b)

    # ---- BM25 side -----------------------------------------------------------------------------------------
    def add_to_bm25(self, text: str, chunk_id: int) -> int:
        bid = self._bm25.add_document(self.tokenize(text))
        self._chunk_to_bm25[chunk_id] = bid
        self._bm25_to_chunk[bid] = chunk_id
        return bid

    def remove_from_bm25(self, chunk_id: int) -> None:
        bid = self._chunk_to_bm25.pop(chunk_id, None)
        if bid is not None:
            self._bm25.remove_document(bid)
            self._bm25_to_chunk.pop(bid, None)

    def bm25_search(self, query: str) -> Dict[int, float]:
        scores = self._bm25.score_all(self.tokenize(query))
        return {self._bm25_to_chunk[b]: s for b, s in scores.items() if b in self._bm25_to_chunk}

    def clear_bm25(self) -> None:
        self._bm25 = BM25Scorer()
        self._chunk_to_bm25.clear()
        self._bm25_to_chunk.clear()

    def reset_idf(self) -> None:
        self._doc_count = 0
        self._doc_freq.clear()

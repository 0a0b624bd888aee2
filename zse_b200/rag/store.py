"""Persistent store of documents and chunks (SQLite) plus the in-memory inverted index that narrows a query to candidate
chunks (roles of zse-engine/zse_engine/rag/store.py:21-493: tables ``rag_documents`` and ``rag_chunks`` with a sparse
embedding BLOB and an optional dense-vector BLOB per chunk)."""
from __future__ import annotations

import json
import sqlite3
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple

from .embeddings import TokenEmbedder, sparse_cosine
from .parser import Chunk

SCHEMA = """
CREATE TABLE IF NOT EXISTS rag_documents (
    id INTEGER PRIMARY KEY AUTOINCREMENT,
    name TEXT NOT NULL,
    doc_type TEXT NOT NULL DEFAULT 'text',
    chunk_count INTEGER NOT NULL DEFAULT 0,
    original_tokens INTEGER NOT NULL DEFAULT 0,
    compressed_tokens INTEGER NOT NULL DEFAULT 0,
    metadata TEXT NOT NULL DEFAULT '{}',
    created_at REAL NOT NULL
);
CREATE TABLE IF NOT EXISTS rag_chunks (
    id INTEGER PRIMARY KEY AUTOINCREMENT,
    doc_id INTEGER NOT NULL REFERENCES rag_documents(id) ON DELETE CASCADE,
    chunk_index INTEGER NOT NULL,
    content TEXT NOT NULL,
    compressed TEXT NOT NULL,
    embedding BLOB,
    dense_vector BLOB,
    metadata TEXT NOT NULL DEFAULT '{}',
    original_tokens INTEGER NOT NULL DEFAULT 0,
    compressed_tokens INTEGER NOT NULL DEFAULT 0
);
CREATE INDEX IF NOT EXISTS idx_rag_chunks_doc ON rag_chunks(doc_id);
"""


@dataclass
class StoredDocument:
    id: int
    name: str
    doc_type: str
    chunk_count: int
    original_tokens: int
    compressed_tokens: int
    metadata: Dict[str, Any]
    created_at: float

    @property
    def savings_pct(self) -> float:
        return (1.0 - self.compressed_tokens / self.original_tokens) * 100.0 if self.original_tokens else 0.0


@dataclass
class StoredChunk:
    id: int
    doc_id: int
    chunk_index: int
    content: str
    compressed: str
    embedding: bytes
    metadata: Dict[str, Any]
    original_tokens: int
    compressed_tokens: int
    has_dense: bool = False
    dense_vector: Optional[bytes] = None     # filled by ``get_dense_vectors`` callers that want it on the chunk

    @property
    def token_count(self) -> int:
        """Tokens of the stored (compressed) text: the reference's field name."""
        return self.compressed_tokens


@dataclass
class SearchResult:
    chunk_id: int
    doc_id: int
    doc_name: str
    content: str
    compressed: str
    score: float
    metadata: Dict[str, Any] = field(default_factory=dict)
    scores: Dict[str, float] = field(default_factory=dict)

    # the reference's per-signal fields (zse-engine/zse_engine/rag/store.py:53-61), read from ``scores``
    @property
    def cosine_score(self) -> float:
        return float(self.scores.get("cosine", self.scores.get("tfidf", 0.0)))

    @property
    def bm25_score(self) -> float:
        return float(self.scores.get("bm25", 0.0))

    @property
    def dense_score(self) -> float:
        return float(self.scores.get("dense", 0.0))

    @property
    def rerank_score(self) -> Optional[float]:
        return self.scores.get("rerank")

    @property
    def chunk(self) -> "StoredChunk":
        """The hit as a chunk record (without its sparse vector, which search results do not carry)."""
        return StoredChunk(self.chunk_id, self.doc_id, int(self.metadata.get("chunk_index", 0)), self.content,
                           self.compressed, b"", self.metadata, 0, 0)


class InvertedIndex:
    """token id -> chunk ids; a query's candidates are the chunks that share at least one token with it."""

    def __init__(self):
        self._post: Dict[int, Set[int]] = {}
        self._by_chunk: Dict[int, Set[int]] = {}

    def add(self, chunk_id: int, token_ids: Iterable[int]) -> None:
        toks = set(token_ids)
        self._by_chunk[chunk_id] = toks
        for t in toks:
            self._post.setdefault(t, set()).add(chunk_id)

    def remove(self, chunk_id: int, token_ids: Iterable[int]) -> None:
        for t in token_ids:
            s = self._post.get(t)
            if s is not None:
                s.discard(chunk_id)
                if not s:
                    del self._post[t]

    def remove_chunk(self, chunk_id: int) -> None:
        self.remove(chunk_id, self._by_chunk.pop(chunk_id, set()))

    def candidates(self, query_tokens: Iterable[int]) -> Set[int]:
        out: Set[int] = set()
        for t in set(query_tokens):
            out |= self._post.get(t, set())
        return out

    def clear(self) -> None:
        self._post.clear()
        self._by_chunk.clear()

    @property
    def token_count(self) -> int:
        return len(self._post)


class RAGStore:
    def __init__(self, db=None):
        """``db``: a ``ServerDatabase`` (its connection and lock are shared), a path, or None for an in-memory store."""
        if db is None or isinstance(db, str):
            self._conn = sqlite3.connect(db or ":memory:", check_same_thread=False)
            self._conn.row_factory = sqlite3.Row
            self._lock = threading.Lock()
        else:
            self._conn, self._lock = db._conn, db._lock
        with self._lock:
            self._conn.execute("PRAGMA foreign_keys=ON")
            self._conn.executescript(SCHEMA)
            self._conn.commit()
        self.index = InvertedIndex()

    # ---- writes ---------------------------------------------------------------------------------------------
    def add_document(self, name: str, doc_type: str, chunks: Sequence[Chunk], embeddings: Sequence[bytes],
                     token_sets: Optional[Sequence[Set[int]]] = None, metadata: Optional[Dict] = None) -> int:
        with self._lock:
            cur = self._conn.execute(
                "INSERT INTO rag_documents (name, doc_type, chunk_count, original_tokens, compressed_tokens, metadata, "
                "created_at) VALUES (?,?,?,?,?,?,?)",
                (name, doc_type, len(chunks), sum(c.original_tokens for c in chunks),
                 sum(c.compressed_tokens for c in chunks), json.dumps(metadata or {}), time.time()))
            doc_id = cur.lastrowid
            ids = []
            for i, (c, e) in enumerate(zip(chunks, embeddings)):
                cur = self._conn.execute(
                    "INSERT INTO rag_chunks (doc_id, chunk_index, content, compressed, embedding, metadata, "
                    "original_tokens, compressed_tokens) VALUES (?,?,?,?,?,?,?,?)",
                    (doc_id, i, c.text, c.compressed, e, json.dumps(c.metadata, default=str), c.original_tokens,
                     c.compressed_tokens))
                ids.append(cur.lastrowid)
            self._conn.commit()
        if token_sets is not None:
            for cid, ts in zip(ids, token_sets):
                self.index.add(cid, ts)
        return doc_id

    def remove_document(self, doc_id: int) -> bool:
        with self._lock:
            ids = [r["id"] for r in self._conn.execute("SELECT id FROM rag_chunks WHERE doc_id=?", (doc_id,))]
            self._conn.execute("DELETE FROM rag_chunks WHERE doc_id=?", (doc_id,))
            cur = self._conn.execute("DELETE FROM rag_documents WHERE id=?", (doc_id,))
            self._conn.commit()
        for cid in ids:
            self.index.remove_chunk(cid)
        return cur.rowcount > 0

    def set_dense_vector(self, chunk_id: int, vec: bytes) -> None:
        with self._lock:
            self._conn.execute("UPDATE rag_chunks SET dense_vector=? WHERE id=?", (vec, chunk_id))
            self._conn.commit()

    def set_embedding(self, chunk_id: int, emb: bytes) -> None:
        with self._lock:
            self._conn.execute("UPDATE rag_chunks SET embedding=? WHERE id=?", (emb, chunk_id))

    # ---- reads ----------------------------------------------------------------------------------------------
    def _doc(self, r) -> StoredDocument:
        return StoredDocument(r["id"], r["name"], r["doc_type"], r["chunk_count"], r["original_tokens"],
                              r["compressed_tokens"], json.loads(r["metadata"] or "{}"), r["created_at"])

    def _chunk(self, r) -> StoredChunk:
        return StoredChunk(r["id"], r["doc_id"], r["chunk_index"], r["content"], r["compressed"],
                           r["embedding"] or b"", json.loads(r["metadata"] or "{}"), r["original_tokens"],
                           r["compressed_tokens"], r["dense_vector"] is not None)

    def list_documents(self) -> List[StoredDocument]:
        with self._lock:
            return [self._doc(r) for r in self._conn.execute("SELECT * FROM rag_documents ORDER BY id")]

    def get_document(self, doc_id: int) -> Optional[StoredDocument]:
        with self._lock:
            r = self._conn.execute("SELECT * FROM rag_documents WHERE id=?", (doc_id,)).fetchone()
        return self._doc(r) if r else None

    def get_chunks(self, doc_id: int) -> List[StoredChunk]:
        with self._lock:
            return [self._chunk(r) for r in
                    self._conn.execute("SELECT * FROM rag_chunks WHERE doc_id=? ORDER BY chunk_index", (doc_id,))]

    def all_chunks(self) -> List[StoredChunk]:
        with self._lock:
            return [self._chunk(r) for r in self._conn.execute("SELECT * FROM rag_chunks ORDER BY id")]

    def get_chunks_by_ids(self, chunk_ids: Iterable[int]) -> Dict[int, Tuple[StoredChunk, str]]:
        ids = list(chunk_ids)
        out: Dict[int, Tuple[StoredChunk, str]] = {}
        with self._lock:
            for i in range(0, len(ids), 500):
                part = ids[i:i + 500]
                q = ("SELECT c.*, d.name AS doc_name FROM rag_chunks c JOIN rag_documents d ON d.id=c.doc_id "
                     f"WHERE c.id IN ({','.join('?' * len(part))})")
                for r in self._conn.execute(q, part):
                    out[r["id"]] = (self._chunk(r), r["doc_name"])
        return out

    def get_dense_vectors(self, chunk_ids: Iterable[int]) -> Dict[int, bytes]:
        ids = list(chunk_ids)
        out: Dict[int, bytes] = {}
        with self._lock:
            for i in range(0, len(ids), 500):
                part = ids[i:i + 500]
                q = f"SELECT id, dense_vector FROM rag_chunks WHERE id IN ({','.join('?' * len(part))})"
                for r in self._conn.execute(q, part):
                    if r["dense_vector"] is not None:
                        out[r["id"]] = r["dense_vector"]
        return out

    def all_chunk_ids_missing_dense(self) -> List[int]:
        with self._lock:
            return [r["id"] for r in self._conn.execute("SELECT id FROM rag_chunks WHERE dense_vector IS NULL")]

    def get_chunk_text(self, chunk_id: int) -> Optional[str]:
        with self._lock:
            r = self._conn.execute("SELECT content FROM rag_chunks WHERE id=?", (chunk_id,)).fetchone()
        return r["content"] if r else None

    # ---- lexical search -------------------------------------------------------------------------------------
    def search(self, query_embedding: bytes, embedder: TokenEmbedder, query: str, top_k: int = 5,
               candidate_ids: Optional[Set[int]] = None, min_score: float = 0.0) -> List[SearchResult]:
        """Hybrid lexical ranking: BM25 (normalised to its best hit) blended with TF-IDF cosine."""
        bm25 = embedder.bm25_search(query)
        ids = set(bm25) if candidate_ids is None else set(candidate_ids)
        if not ids:
            return []
        rows = self.get_chunks_by_ids(ids)
        top_bm25 = max(bm25.values()) if bm25 else 0.0
        w = embedder.bm25_weight
        out = []
        for cid, (ch, doc_name) in rows.items():
            cos = sparse_cosine(query_embedding, ch.embedding)
            b = bm25.get(cid, 0.0) / top_bm25 if top_bm25 > 0 else 0.0
            score = w * b + (1.0 - w) * cos
            if score >= min_score:
                out.append(SearchResult(cid, ch.doc_id, doc_name, ch.content, ch.compressed, score, ch.metadata,
                                        {"bm25": b, "tfidf": cos}))
        out.sort(key=lambda r: (-r.score, r.chunk_id))
        return out[:top_k]

    def rebuild_inverted_index(self, embedder: TokenEmbedder) -> None:
        self.index.clear()
        for ch in self.all_chunks():
            self.index.add(ch.id, set(embedder.tokenize(ch.content)))

    def reembed_all(self, embedder: TokenEmbedder) -> None:
        for ch in self.all_chunks():
            self.set_embedding(ch.id, embedder.embed(ch.content))
        with self._lock:
            self._conn.commit()

    def stats(self) -> Dict[str, Any]:
        with self._lock:
            d = self._conn.execute("SELECT COUNT(*) AS n, COALESCE(SUM(original_tokens),0) AS o, "
                                   "COALESCE(SUM(compressed_tokens),0) AS c FROM rag_documents").fetchone()
            c = self._conn.execute("SELECT COUNT(*) AS n, SUM(dense_vector IS NOT NULL) AS dn FROM rag_chunks").fetchone()
        o, comp = d["o"], d["c"]
        return {"documents": d["n"], "chunks": c["n"], "dense_chunks": int(c["dn"] or 0), "original_tokens": o,
                "compressed_tokens": comp, "token_savings_pct": round((1 - comp / o) * 100, 1) if o else 0.0,
                "index_tokens": self.index.token_count}

"""Retrieval engine: ingest (parse -> ZPF -> sparse embed -> store -> BM25 -> optional dense) and hybrid search
(inverted-index candidates -> BM25 + TF-IDF -> optional dense cosine -> rank fusion -> optional LLM rerank), with the
interface of zse-engine/zse_engine/rag/engine.py:19-625 (``ingest``, ``search``, ``multi_query_search``,
``augment_messages``, document management, ``stats``, ``backfill_dense_embeddings``)."""
from __future__ import annotations

import re
import threading
from typing import Any, Callable, Dict, List, Optional, Set

from .dense import DenseEmbedder
from .embeddings import TokenEmbedder
from .parser import get_parser
from .reranker import LLMReranker
from .store import RAGStore, SearchResult
from .zpf import count_tokens

RRF_K = 60


class RAGEngine:
    def __init__(self, db=None, tokenizer=None, vocab_size: int = 32000, chunk_size: int = 512, overlap: int = 64,
                 bm25_weight: float = 0.5, reembed_threshold: int = 10):
        self._tok = tokenizer
        self._store = RAGStore(db)
        self._embedder = TokenEmbedder(tokenizer, vocab_size, bm25_weight)
        self._chunk_size, self._overlap = chunk_size, overlap
        self._dense: Optional[DenseEmbedder] = None
        self._reranker: Optional[LLMReranker] = None
        self._dense_default = False
        self._docs_since_reembed = 0
        self._reembed_threshold = reembed_threshold
        self._lock = threading.RLock()
        self._rebuild_all()

    # ---- wiring ---------------------------------------------------------------------------------------------
    def set_model_runner(self, model_runner, enable_dense_by_default: bool = True) -> None:
        """``model_runner``: the serving engine (``embed_tokens`` / ``last_token_logits``).  Name and parameter follow the
        reference, which hands its ModelRunner over here."""
        self._dense = DenseEmbedder(model_runner, self._tok)
        self._reranker = LLMReranker(model_runner, self._tok)
        self._dense_default = enable_dense_by_default

    @property
    def has_dense(self) -> bool:
        return self._dense is not None

    def backfill_dense_embeddings(self, batch_size: int = 32) -> int:
        if self._dense is None:
            return 0
        done = 0
        for cid in self._store.all_chunk_ids_missing_dense():
            text = self._store.get_chunk_text(cid)
            vec = self._dense.embed(text) if text else None
            if vec is not None:
                self._store.set_dense_vector(cid, vec)
                done += 1
        return done

    def _rebuild_all(self) -> None:
        """After a restart: IDF statistics, inverted index and BM25 index from what the database holds."""
        chunks = self._store.all_chunks()
        self._embedder.reset_idf()
        self._embedder.clear_bm25()
        self._store.index.clear()
        sets = []
        for ch in chunks:
            toks = self._embedder.tokenize(ch.content)
            ts = set(toks)
            sets.append(ts)
            self._store.index.add(ch.id, ts)
            self._embedder.add_to_bm25(ch.content, ch.id)
        self._embedder.update_idf(sets)

    # ---- ingest ---------------------------------------------------------------------------------------------
    def ingest(self, filename: str, content: bytes, chunk_size: Optional[int] = None, overlap: Optional[int] = None,
               pdf_password: Optional[str] = None, ocr_fn: Optional[Callable[[bytes, str], str]] = None
               ) -> Dict[str, Any]:
        cs, ov = chunk_size or self._chunk_size, overlap or self._overlap
        ext = filename.rsplit(".", 1)[-1].lower() if "." in filename else "text"
        doc_type = {"json": "json", "jsonl": "json", "ndjson": "json", "csv": "csv", "tsv": "csv", "pdf": "pdf"}.get(
            ext, "text")
        parser = get_parser(filename, cs, ov)
        meta: Dict[str, Any] = {"source": filename}
        if pdf_password:
            meta["pdf_password"] = pdf_password
        if ocr_fn is not None:
            meta["ocr_fn"] = ocr_fn
        try:
            if doc_type == "pdf":
                chunks = parser.parse(content, tokenizer=self._tok, metadata=meta)
            else:
                try:
                    text = content.decode("utf-8")
                except UnicodeDecodeError:
                    text = content.decode("latin-1")
                chunks = parser.parse(text, tokenizer=self._tok, metadata=meta)
        except Exception as exc:
            return {"error": f"could not parse {filename}: {exc}"}
        if not chunks:
            return {"error": "No content could be extracted from the document"}
        failed = [c for c in chunks if c.metadata.get("error")]
        if failed and len(failed) == len(chunks):        # the parser's failure marker: nothing worth storing
            return {"error": f"could not parse {filename}: {failed[0].text.strip('[]')}",
                    "error_kind": failed[0].metadata["error"]}
        with self._lock:
            token_sets = [set(self._embedder.tokenize(c.text)) for c in chunks]
            self._embedder.update_idf(token_sets)
            embeddings = [self._embedder.embed(c.text) for c in chunks]
            doc_id = self._store.add_document(filename, doc_type, chunks, embeddings, token_sets)
            stored = self._store.get_chunks(doc_id)
            for sc in stored:
                self._embedder.add_to_bm25(sc.content, sc.id)
            if self._dense is not None:
                for sc in stored:
                    vec = self._dense.embed(sc.content)
                    if vec is not None:
                        self._store.set_dense_vector(sc.id, vec)
            self._docs_since_reembed += 1
            if self._docs_since_reembed >= self._reembed_threshold:       # IDF drifted: refresh stored vectors
                self._store.reembed_all(self._embedder)
                self._docs_since_reembed = 0
        orig = sum(c.original_tokens for c in chunks)
        comp = sum(c.compressed_tokens for c in chunks)
        return {"doc_id": doc_id, "filename": filename, "doc_type": doc_type, "chunk_count": len(chunks),
                "original_tokens": orig, "compressed_tokens": comp,
                "token_savings_pct": round((1.0 - comp / orig) * 100, 1) if orig else 0.0}

    # ---- search ---------------------------------------------------------------------------------------------
    def _apply_filters(self, ids: Optional[Set[int]], filters: Dict) -> Optional[Set[int]]:
        docs = self._store.list_documents()
        ok_docs = {d.id for d in docs
                   if ("doc_type" not in filters or d.doc_type == filters["doc_type"])
                   and ("doc_name" not in filters or d.name == filters["doc_name"])
                   and ("doc_id" not in filters or d.id == int(filters["doc_id"]))}
        allowed = {c.id for d in ok_docs for c in self._store.get_chunks(d)}
        return allowed if ids is None else ids & allowed

    @staticmethod
    def _fuse(rankings: Dict[str, List[int]], scores: Dict[str, Dict[int, float]], fusion: str,
              weights: Optional[Dict[str, float]] = None) -> Dict[int, float]:
        fused: Dict[int, float] = {}
        if fusion == "weighted":
            weights = weights or {}
            for name, sc in scores.items():
                top = max(sc.values()) if sc else 0.0
                for cid, s in sc.items():
                    fused[cid] = fused.get(cid, 0.0) + weights.get(name, 1.0) * (s / top if top > 0 else 0.0)
            return fused
        for order in rankings.values():                                  # reciprocal rank fusion
            for rank, cid in enumerate(order):
                fused[cid] = fused.get(cid, 0.0) + 1.0 / (RRF_K + rank + 1)
        return fused

    def search(self, query: str, top_k: int = 5, filters: Optional[Dict] = None, use_dense: Optional[bool] = None,
               use_rerank: bool = False, candidate_pool: int = 30, fusion: str = "rrf") -> List[Dict[str, Any]]:
        if not query or not query.strip():
            return []
        if use_dense is None:
            use_dense = self._dense_default and self._dense is not None
        use_dense = bool(use_dense and self._dense is not None)
        with self._lock:
            q_tokens = self._embedder.tokenize(query)
            cands: Optional[Set[int]] = self._store.index.candidates(q_tokens)
            if not cands and self._store.index.token_count == 0:
                cands = None
            if filters:
                cands = self._apply_filters(cands, filters)
            pool = max(candidate_pool, top_k * 4)
            sparse = self._store.search(self._embedder.embed(query), self._embedder, query, top_k=pool,
                                        candidate_ids=cands)
        by_id: Dict[int, SearchResult] = {r.chunk_id: r for r in sparse}
        rankings = {"sparse": [r.chunk_id for r in sparse]}
        scores = {"sparse": {r.chunk_id: r.score for r in sparse}}
        if use_dense:
            qv = self._dense.embed_query(query)
            if qv is not None:
                # dense can rescue chunks that share no token with the query: score every chunk that has a vector
                ids = {c.id for c in self._store.all_chunks() if c.has_dense}
                if filters:
                    ids = self._apply_filters(ids, filters) or set()
                vecs = self._store.get_dense_vectors(ids)
                dsc = {cid: DenseEmbedder.cosine(qv, v) for cid, v in vecs.items()}
                order = sorted(dsc, key=lambda c: -dsc[c])[:pool]
                rankings["dense"] = order
                scores["dense"] = {c: max(dsc[c], 0.0) for c in order}
                missing = [c for c in order if c not in by_id]
                for cid, (ch, name) in self._store.get_chunks_by_ids(missing).items():
                    by_id[cid] = SearchResult(cid, ch.doc_id, name, ch.content, ch.compressed, 0.0, ch.metadata, {})
        fused = self._fuse(rankings, scores, fusion)
        order = sorted(fused, key=lambda c: (-fused[c], c))[:max(candidate_pool, top_k)]
        if use_rerank and self._reranker is not None and order:
            rr = self._reranker.rerank(query, [(c, by_id[c].content) for c in order], top_n=top_k)
            if any(s != 0.0 for _, s in rr):
                rr_scores = dict(rr)
                order = [c for c, _ in rr]
                for c in order:
                    by_id[c].scores["rerank"] = rr_scores[c]
        out = []
        for cid in order[:top_k]:
            r = by_id[cid]
            sc = dict(r.scores)
            if "dense" in scores and cid in scores["dense"]:
                sc["dense"] = scores["dense"][cid]
            out.append({"chunk_id": cid, "doc_id": r.doc_id, "doc_name": r.doc_name, "content": r.content,
                        "compressed": r.compressed, "score": round(fused[cid], 6), "scores": sc,
                        "metadata": r.metadata, "token_count": count_tokens(r.compressed, self._tok)})
        return out

    def _decompose_query(self, query: str) -> List[str]:
        parts = re.split(r"\?|;|\band\b|\balso\b|\bas well as\b|, (?=what|who|how|when|where|which|why)", query,
                         flags=re.I)
        subs = [p.strip(" ,.") for p in parts if len(p.strip(" ,.").split()) >= 2]
        return subs if len(subs) > 1 else [query]

    def multi_query_search(self, query: str, top_k: int = 5, filters: Optional[Dict] = None) -> List[Dict[str, Any]]:
        subs = self._decompose_query(query)
        if len(subs) == 1:
            return self.search(query, top_k, filters)
        best: Dict[int, Dict[str, Any]] = {}
        for q in [query] + subs:
            for r in self.search(q, top_k, filters):
                cur = best.get(r["chunk_id"])
                if cur is None or r["score"] > cur["score"]:
                    best[r["chunk_id"]] = r
        return sorted(best.values(), key=lambda r: -r["score"])[:top_k]

    def augment_messages(self, messages: List[Dict[str, str]], top_k: int = 5, max_context_tokens: int = 2048
                         ) -> List[Dict[str, str]]:
        idx = next((i for i in range(len(messages) - 1, -1, -1) if messages[i].get("role") == "user"), -1)
        if idx < 0 or not messages[idx].get("content"):
            return messages
        parts, total = [], 0
        for r in self.search(messages[idx]["content"], top_k=top_k):
            if total + r["token_count"] > max_context_tokens:
                break
            parts.append(r["compressed"] or r["content"])
            total += r["token_count"]
        if not parts:
            return messages
        ctx = ("Relevant context from uploaded documents:\n" + "\n---\n".join(parts) +
               "\n\nUse the above context to help answer the user's question. If the context is not relevant, "
               "ignore it.")
        out = list(messages)
        out.insert(idx, {"role": "system", "content": ctx})
        return out

    # ---- documents --------------------------------------------------------------------------------------------
    def list_documents(self) -> List[Dict[str, Any]]:
        return [{"id": d.id, "name": d.name, "doc_type": d.doc_type, "chunk_count": d.chunk_count,
                 "original_tokens": d.original_tokens, "compressed_tokens": d.compressed_tokens,
                 "token_savings_pct": round(d.savings_pct, 1), "created_at": d.created_at}
                for d in self._store.list_documents()]

    def get_document(self, doc_id: int) -> Optional[Dict[str, Any]]:
        d = self._store.get_document(doc_id)
        if d is None:
            return None
        return {"id": d.id, "name": d.name, "doc_type": d.doc_type, "chunk_count": d.chunk_count,
                "original_tokens": d.original_tokens, "compressed_tokens": d.compressed_tokens,
                "token_savings_pct": round(d.savings_pct, 1), "created_at": d.created_at,
                "chunks": [{"id": c.id, "index": c.chunk_index, "content": c.content, "compressed": c.compressed,
                            "metadata": c.metadata, "has_dense": c.has_dense} for c in self._store.get_chunks(doc_id)]}

    def remove_document(self, doc_id: int) -> bool:
        with self._lock:
            for c in self._store.get_chunks(doc_id):
                self._embedder.remove_from_bm25(c.id)
            return self._store.remove_document(doc_id)

    def update_document(self, doc_id: int, filename: str, content: bytes, **kw) -> Dict[str, Any]:
        """Replace a document: the new version is ingested first, the old one removed only if that worked."""
        res = self.ingest(filename, content, **kw)
        if "error" not in res:
            self.remove_document(doc_id)
        return res

    def stats(self) -> Dict[str, Any]:
        s = self._store.stats()
        s.update({"dense_enabled": self.has_dense, "chunk_size": self._chunk_size, "overlap": self._overlap})
        return s

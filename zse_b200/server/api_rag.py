"""Retrieval routes (zse-engine/zse_engine/server/api_rag.py:19-310): ``POST /v1/rag/upload`` (base64 or plain text
body), ``PUT|GET|DELETE /v1/rag/document/{id}``, ``GET /v1/rag/documents``, ``POST /v1/rag/search``,
``GET /v1/rag/stats``, ``POST /v1/rag/backfill_dense`` (admin).  Ingestion and search run in a worker thread so that
the event loop keeps serving streams."""
from __future__ import annotations

import asyncio
import base64
import binascii

from .router import Request, Response

MAX_UPLOAD_BYTES = 64 << 20


class RAGAPI:
    def __init__(self, rag_engine, auth):
        self._rag, self._auth = rag_engine, auth

    def register(self, router) -> None:
        router.post("/v1/rag/upload", self.upload)
        router.put("/v1/rag/document/{id}", self.replace)
        router.get("/v1/rag/documents", self.list_documents)
        router.get("/v1/rag/document/{id}", self.get_document)
        router.delete("/v1/rag/document/{id}", self.delete_document)
        router.post("/v1/rag/search", self.search)
        router.get("/v1/rag/stats", self.stats)
        router.post("/v1/rag/backfill_dense", self.backfill_dense)

    @staticmethod
    def _content(body: dict):
        if "content" in body and body["content"] is not None:
            try:
                return base64.b64decode(body["content"], validate=True), None
            except (binascii.Error, ValueError):
                return None, "'content' must be base64"
        if "text" in body and body["text"] is not None:
            return str(body["text"]).encode("utf-8"), None
        return None, "'content' (base64) or 'text' is required"

    @staticmethod
    def _doc_id(request: Request):
        try:
            return int(request.params.get("id", ""))
        except (TypeError, ValueError):
            return None

    async def _ingest(self, body: dict, replace_id=None) -> Response:
        filename = str(body.get("filename") or "").strip()
        if not filename:
            return Response.error("'filename' is required")
        data, err = self._content(body)
        if err:
            return Response.error(err)
        if len(data) > MAX_UPLOAD_BYTES:
            return Response.error("document too large", 413)
        kw = {"chunk_size": body.get("chunk_size"), "overlap": body.get("overlap"),
              "pdf_password": body.get("pdf_password")}
        if replace_id is None:
            res = await asyncio.to_thread(self._rag.ingest, filename, data, **kw)
        else:
            res = await asyncio.to_thread(self._rag.update_document, replace_id, filename, data, **kw)
        if "error" in res:
            return Response.error(res["error"], 422)
        return Response.json_response(res, 201 if replace_id is None else 200)

    async def upload(self, request: Request) -> Response:
        return await self._ingest(request.json or {})

    async def replace(self, request: Request) -> Response:
        doc_id = self._doc_id(request)
        if doc_id is None or self._rag.get_document(doc_id) is None:
            return Response.error("document not found", 404)
        return await self._ingest(request.json or {}, replace_id=doc_id)

    async def list_documents(self, request: Request) -> Response:
        return Response.json_response({"documents": self._rag.list_documents()})

    async def get_document(self, request: Request) -> Response:
        doc_id = self._doc_id(request)
        doc = self._rag.get_document(doc_id) if doc_id is not None else None
        return Response.json_response(doc) if doc else Response.error("document not found", 404)

    async def delete_document(self, request: Request) -> Response:
        doc_id = self._doc_id(request)
        if doc_id is None or not self._rag.remove_document(doc_id):
            return Response.error("document not found", 404)
        return Response.json_response({"deleted": doc_id})

    async def search(self, request: Request) -> Response:
        b = request.json or {}
        query = str(b.get("query") or "").strip()
        if not query:
            return Response.error("'query' is required")
        top_k = max(1, min(int(b.get("top_k", 5)), 50))
        kw = dict(top_k=top_k, filters=b.get("filters"))
        if b.get("multi_query"):
            res = await asyncio.to_thread(self._rag.multi_query_search, query, **kw)
        else:
            res = await asyncio.to_thread(self._rag.search, query, use_dense=b.get("use_dense"),
                                          use_rerank=bool(b.get("rerank", False)),
                                          fusion=str(b.get("fusion", "rrf")), **kw)
        return Response.json_response({"query": query, "results": res})

    async def stats(self, request: Request) -> Response:
        return Response.json_response(self._rag.stats())

    async def backfill_dense(self, request: Request) -> Response:
        if not self._auth.is_admin(request.authorization):
            return Response.error("Admin access required", 403)
        n = await asyncio.to_thread(self._rag.backfill_dense_embeddings)
        return Response.json_response({"embedded": n})

    # the reference's handler names (zse-engine/zse_engine/server/api_rag.py:49-310)
    handle_upload = upload
    handle_replace = replace
    handle_list = list_documents
    handle_get = get_document
    handle_delete = delete_document
    handle_search = search
    handle_stats = stats
    handle_backfill_dense = backfill_dense

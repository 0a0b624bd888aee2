"""LoRA hot-swap routes (zse-engine/zse_engine/server/api_lora.py:14-144): ``GET /v1/lora/list``,
``POST /v1/lora/load {adapter_id, path}`` (admin), ``POST /v1/lora/unload {adapter_id}`` (admin),
``GET /v1/lora/stats``.  Loading happens while the engine keeps serving; requests name the adapter with ``lora_id``
or ``model: "<model>:<adapter>"``."""
from __future__ import annotations

import os

from .router import Request, Response


class LoRAAPI:
    def __init__(self, engine, auth):
        self._engine, self._auth = engine, auth

    def register(self, router) -> None:
        router.get("/v1/lora/list", self.list_adapters)
        router.post("/v1/lora/load", self.load)
        router.post("/v1/lora/unload", self.unload)
        router.get("/v1/lora/stats", self.stats)

    def _manager(self):
        return getattr(self._engine, "lora_manager", None) if self._engine is not None else None

    async def list_adapters(self, request: Request) -> Response:
        m = self._manager()
        return Response.json_response({"adapters": m.list_adapters() if m else []})

    async def stats(self, request: Request) -> Response:
        m = self._manager()
        return Response.json_response(m.stats() if m else {"num_adapters": 0})

    async def load(self, request: Request) -> Response:
        if not self._auth.is_admin(request.authorization):
            return Response.error("Admin access required", 403)
        m = self._manager()
        if m is None:
            return Response.error("no engine loaded", 503)
        b = request.json or {}
        aid, path = b.get("adapter_id"), b.get("path")
        if not aid or not path:
            return Response.error("'adapter_id' and 'path' are required")
        if not os.path.isfile(path):
            return Response.error(f"adapter file not found: {path}", 404)
        try:
            ad = m.load_adapter(str(aid), str(path))
        except (ValueError, MemoryError) as exc:
            return Response.error(str(exc), 400)
        return Response.json_response({"adapter_id": ad.adapter_id, "rank": ad.rank, "alpha": ad.alpha,
                                       "target_modules": ad.target_modules, "num_layers": ad.num_layers,
                                       "bytes": ad.total_bytes}, 201)

    async def unload(self, request: Request) -> Response:
        if not self._auth.is_admin(request.authorization):
            return Response.error("Admin access required", 403)
        m = self._manager()
        b = request.json or {}
        if m is None or not b.get("adapter_id"):
            return Response.error("'adapter_id' is required")
        if not m.unload_adapter(str(b["adapter_id"])):
            return Response.error(f"adapter '{b['adapter_id']}' is not loaded", 404)
        return Response.json_response({"unloaded": b["adapter_id"]})

    # the reference's handler names (zse-engine/zse_engine/server/api_lora.py:39-150)
    handle_list = list_adapters
    handle_load = load
    handle_unload = unload
    handle_stats = stats

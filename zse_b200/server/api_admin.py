"""Admin routes (admin key required): API keys, engine statistics, usage, dashboard chat sessions
(zse-engine/zse_engine/server/api_admin.py:20-289)."""
from __future__ import annotations

import dataclasses
import secrets

from .router import Request, Response


class AdminAPI:
    def __init__(self, db, auth, engine=None, require_auth: bool = False):
        self._db, self._auth, self._engine = db, auth, engine
        self.require_auth = require_auth

    def register(self, router) -> None:
        router.post("/v1/admin/keys/create", self.create_key)
        router.get("/v1/admin/keys/list", self.list_keys)
        router.post("/v1/admin/keys/revoke", self.revoke_key)
        router.post("/v1/admin/keys/update", self.update_key)
        router.get("/v1/admin/stats", self.stats)
        router.get("/metrics", self.metrics)
        router.get("/v1/admin/usage", self.usage)
        router.post("/v1/dashboard/session", self.session_create)
        router.post("/v1/dashboard/session/save", self.session_save)      # before the {session_id} patterns
        router.get("/v1/dashboard/sessions", self.session_list)
        router.get("/v1/dashboard/session/{session_id}", self.session_get)
        router.post("/v1/dashboard/session/{session_id}/message", self.session_add_message)
        router.delete("/v1/dashboard/session/{session_id}", self.session_delete)

    def _deny(self, request: Request):
        if not self._auth.is_admin(request.authorization):
            return Response.error("Admin access required", 403)
        return None

    async def create_key(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        b = request.json or {}
        key, info = self._db.create_key(str(b.get("name", "")), int(b.get("rate_limit_rpm", 60)),
                                        int(b.get("rate_limit_tpm", 100000)), str(b.get("allowed_models", "*")),
                                        b.get("expires_in_days"))
        out = info.to_public()
        out["key"] = key            # shown once
        return Response.json_response(out, 201)

    async def list_keys(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        return Response.json_response({"keys": [k.to_public() for k in self._db.list_keys()]})

    async def revoke_key(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        b = request.json or {}
        if "id" in b:
            ok = self._db.revoke_key(int(b["id"]))
        elif "prefix" in b:
            ok = self._db.revoke_key_by_prefix(str(b["prefix"]))
        else:
            return Response.error("'id' or 'prefix' required")
        return Response.json_response({"revoked": ok}) if ok else Response.error("key not found", 404)

    async def update_key(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        b = request.json or {}
        if "id" not in b:
            return Response.error("'id' required")
        ok = self._db.update_key_limits(int(b["id"]), b.get("rate_limit_rpm"), b.get("rate_limit_tpm"),
                                        b.get("allowed_models"))
        return Response.json_response({"updated": ok}) if ok else Response.error("key not found or nothing to update", 404)

    async def stats(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        out = {"usage": self._db.get_usage_stats(), "num_keys": len(self._db.list_keys())}
        e = self._engine
        if e is not None:
            out["engine"] = dataclasses.asdict(e.stats())
            if hasattr(e, "scheduler"):
                out["scheduler"] = e.scheduler.stats()
            if hasattr(e, "kv_cache"):
                out["kv_cache"] = dataclasses.asdict(e.kv_cache.stats())
            out["lora"] = e.lora_manager.stats() if e.lora_manager is not None else {}
            spec = getattr(e, "_spec_runner", None)
            if spec is not None:
                out["speculative"] = spec.stats()
            out["init_times"] = getattr(e, "init_times", {})
        return Response.json_response(out)

    async def metrics(self, request: Request) -> Response:
        """Counters and gauges of the engine in the Prometheus text exposition format (no counterpart in the reference,
        whose numbers are only available as JSON from ``/v1/admin/stats``).  On a server that requires keys the route
        wants the admin key; otherwise it is open, like ``/health``."""
        if getattr(self, "require_auth", False) and (r := self._deny(request)) is not None:
            return r
        rows = []          # (name, type, help, value)

        def add(name, kind, text, value):
            rows.append((name, kind, text, float(value)))

        e = self._engine
        fatal = getattr(e, "fatal_error", None) if e is not None else None
        add("zse_engine_up", "gauge", "1 while the engine can run requests, 0 without an engine or after a device fault",
            0 if (e is None or fatal) else 1)
        if e is not None and hasattr(e, "stats"):
            st = e.stats()
            add("zse_requests_total", "counter", "requests finished", getattr(st, "total_requests", 0))
            add("zse_tokens_generated_total", "counter", "tokens generated", getattr(st, "total_tokens_generated", 0))
            add("zse_steps_total", "counter", "engine steps that ran a batch", getattr(st, "total_steps", 0))
            add("zse_uptime_seconds", "gauge", "seconds since the first step", getattr(st, "uptime_s", 0.0))
            add("zse_requests_waiting", "gauge", "requests in the queue", getattr(st, "queue_depth", 0))
            add("zse_requests_active", "gauge", "requests being prefilled or decoded", getattr(st, "active_requests", 0))
            add("zse_ttft_p50_milliseconds", "gauge", "median time to first token", getattr(st, "p50_ttft_ms", 0.0))
            add("zse_ttft_p99_milliseconds", "gauge", "99th percentile of time to first token",
                getattr(st, "p99_ttft_ms", 0.0))
            add("zse_tpot_p50_milliseconds", "gauge", "median time per output token", getattr(st, "p50_tpot_ms", 0.0))
            add("zse_batch_tokens_avg", "gauge", "tokens generated per step on average", getattr(st, "avg_batch_size", 0.0))
            if hasattr(e, "kv_cache"):
                kv = e.kv_cache.stats()
                add("zse_kv_blocks", "gauge", "KV cache blocks in the pool", kv.total_blocks)
                add("zse_kv_blocks_used", "gauge", "KV cache blocks in use", kv.allocated_blocks)
                add("zse_kv_sequences", "gauge", "sequences holding KV blocks", kv.num_sequences)
                add("zse_kv_evictions_total", "counter", "KV blocks evicted under memory pressure", kv.eviction_count)
                add("zse_kv_prefix_hits_total", "counter", "prompt blocks served from the prefix cache", kv.dedup_hits)
        usage = self._db.get_usage_stats()
        add("zse_api_requests_total", "counter", "requests accounted to API keys", usage["total_requests"])
        add("zse_api_tokens_total", "counter", "tokens accounted to API keys", usage["total_tokens"])
        lines = []
        for name, kind, text, value in rows:
            lines += [f"# HELP {name} {text}", f"# TYPE {name} {kind}",
                      f"{name} {int(value) if value == int(value) else repr(value)}"]
        return Response.text("\n".join(lines) + "\n", content_type="text/plain; version=0.0.4; charset=utf-8")

    async def usage(self, request: Request) -> Response:
        if (r := self._deny(request)) is not None:
            return r
        kid = request.query.get("key_id")
        return Response.json_response(self._db.get_usage_stats(int(kid) if kid else None))

    # ---- dashboard sessions (any authenticated key; the admin key works too) --------------------------------
    def _key_id(self, request: Request):
        res = self._auth.authenticate(request.authorization)
        return res.key.id if res.authenticated else None

    async def session_create(self, request: Request) -> Response:
        if self._key_id(request) is None:
            return Response.error("authentication required", 401)
        return Response.json_response({"session_id": secrets.token_hex(8)}, 201)

    async def session_list(self, request: Request) -> Response:
        kid = self._key_id(request)
        if kid is None:
            return Response.error("authentication required", 401)
        return Response.json_response({"sessions": self._db.list_sessions(None if kid == 0 else kid)})

    async def session_get(self, request: Request) -> Response:
        if self._key_id(request) is None:
            return Response.error("authentication required", 401)
        msgs = self._db.get_session_messages(request.params["session_id"])
        return Response.json_response({"session_id": request.params["session_id"],
                                       "messages": [{"role": m.role, "content": m.content, "model": m.model,
                                                     "created_at": m.created_at} for m in msgs]})

    async def session_add_message(self, request: Request) -> Response:
        kid = self._key_id(request)
        if kid is None:
            return Response.error("authentication required", 401)
        b = request.json or {}
        if not b.get("role") or "content" not in b:
            return Response.error("'role' and 'content' required")
        mid = self._db.save_message(kid, request.params["session_id"], str(b["role"]), str(b["content"]),
                                    str(b.get("model", "")), b.get("lora_id"))
        return Response.json_response({"id": mid}, 201)

    async def session_save(self, request: Request) -> Response:
        """``POST /v1/dashboard/session/save {session_id, role, content, model?, lora_id?}`` - the reference's form of
        adding a message, the session named in the body (zse-engine/zse_engine/server/api_admin.py:265-289)."""
        res = self._auth.authenticate(request.authorization)
        if not res.authenticated:
            return Response.error(res.error, res.status_code)
        b = request.json if isinstance(request.json, dict) else {}
        sid, role, content = str(b.get("session_id", "")), str(b.get("role", "")), str(b.get("content", ""))
        if not sid or not role or not content:
            return Response.error("session_id, role, and content are required")
        self._db.save_message(res.key.id, sid, role, content, str(b.get("model", "")), b.get("lora_id"))
        return Response.json_response({"ok": True})

    async def session_delete(self, request: Request) -> Response:
        if self._key_id(request) is None:
            return Response.error("authentication required", 401)
        return Response.json_response({"deleted": self._db.delete_session(request.params["session_id"])})

    # the reference's handler names (zse-engine/zse_engine/server/api_admin.py:61-290)
    handle_create_key = create_key
    handle_list_keys = list_keys
    handle_revoke_key = revoke_key
    handle_update_key = update_key
    handle_stats = stats
    handle_usage = usage
    handle_list_sessions = session_list
    handle_get_session = session_get
    handle_delete_session = session_delete
    handle_save_message = session_save

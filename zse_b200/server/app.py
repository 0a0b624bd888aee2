"""``ZSEServer``: asyncio HTTP/1.1 front end of the engine (zse-engine/zse_engine/server/app.py:26-338).

One asyncio loop serves connections; the engine's batching loop runs in a daemon thread and hands tokens back with
``loop.call_soon_threadsafe``.  ``/health`` and ``/v1/health`` answer without auth; with ``require_auth`` every
``/v1/*`` inference route needs an API key (the reference never checks keys on inference routes).  With
``tp_size > 1`` rank 0 serves HTTP and the other ranks mirror its requests (``parallel.tp_engine``), so
``serve --tp N`` works over HTTP (the reference's ``TPEngine`` lacks the methods its server calls).
"""
from __future__ import annotations

import asyncio
import os
import threading
from typing import Optional

from .api_admin import AdminAPI
from .api_lora import LoRAAPI
from .api_openai import OpenAIAPI
from .auth import AuthManager
from .database import ServerDatabase
from .router import (MAX_REQUEST_BYTES, Request, Response, Router, content_length_of, format_http_response,
                     parse_http_request)

STATIC_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "static")


class ZSEServer:
    def __init__(self, model_path: Optional[str] = None, host: str = "0.0.0.0", port: int = 8000,
                 admin_key: Optional[str] = None, db_path: str = "~/.zse/server.db", model_name: str = "zse-model",
                 quiet: bool = False, tp_size: int = 1, engine=None, engine_config=None, require_auth: bool = False,
                 enable_rag: bool = True):
        self.host, self.port, self.model_name, self.quiet = host, port, model_name, quiet
        self.require_auth = require_auth
        self._db = ServerDatabase(db_path)
        self._auth = AuthManager(self._db, admin_key)
        self._engine = engine
        self._engine_thread: Optional[threading.Thread] = None
        self._server: Optional[asyncio.AbstractServer] = None
        self._stopping = False
        if engine is None and model_path is not None:
            self._engine = self._init_engine(model_path, tp_size, engine_config)
        tok = getattr(self._engine, "tokenizer", None) if self._engine is not None else None
        self.router = Router()
        self.router.use(self._auth_middleware)
        self.router.get("/health", self._health)
        self.router.get("/v1/health", self._health)
        self._openai = OpenAIAPI(self._engine, model_name, tok, db=self._db)
        self._openai.register(self.router)
        AdminAPI(self._db, self._auth, self._engine, require_auth=require_auth).register(self.router)
        LoRAAPI(self._engine, self._auth).register(self.router)
        self._rag_engine = None
        if enable_rag:
            try:
                from ..rag.engine import RAGEngine
                from .api_rag import RAGAPI
                rag_db = ":memory:" if db_path == ":memory:" else os.path.expanduser(db_path) + ".rag"
                self._rag_engine = RAGEngine(rag_db, tokenizer=tok)
                if self._engine is not None and hasattr(self._engine, "embed_tokens"):
                    self._rag_engine.set_model_runner(self._engine)
                RAGAPI(self._rag_engine, self._auth).register(self.router)
                self._openai.set_rag_engine(self._rag_engine)
            except ImportError:
                self._rag_engine = None
        self.router.static("/", STATIC_DIR)

    def _init_engine(self, model_path: str, tp_size: int, engine_config):
        from ..config import EngineConfig
        cfg = engine_config or EngineConfig.from_env(quiet=self.quiet)
        cfg.tp_size = tp_size
        if tp_size > 1:
            from ..parallel.tp_engine import TPEngine
            return TPEngine(model_path, tp_size=tp_size, config=cfg)
        from ..engine import ZStreamerEngine
        return ZStreamerEngine(model_path, config=cfg)

    @property
    def engine(self):
        return self._engine

    @property
    def database(self) -> ServerDatabase:
        return self._db

    # ---- middleware / basic routes ------------------------------------------------------------------------
    async def _auth_middleware(self, request: Request, handler) -> Response:
        guarded = request.path.startswith("/v1/") and not request.path.startswith(
            ("/v1/health", "/v1/admin", "/v1/dashboard", "/v1/lora"))
        needs_key = self.require_auth and guarded
        header = request.authorization
        if header:
            res = self._auth.authenticate(header)
            if res.authenticated:
                request.context["api_key"] = res.key
                if needs_key or res.key.id > 0:
                    model = ""
                    if request.method == "POST" and isinstance(request.json, dict):
                        model = str(request.json.get("model", "")) if request.path.endswith("completions") else ""
                    chk = self._auth.check_rate_limit(res.key)
                    if chk.authenticated and model:
                        chk = self._auth.check_model_access(res.key, model)
                    if not chk.authenticated:
                        return Response.error(chk.error, chk.status_code)
            elif guarded:            # a key that is presented must be valid, even where keys are optional
                return Response.error(res.error, res.status_code)
        elif needs_key:
            return Response.error("Missing Authorization header", 401)
        return await handler(request)

    async def _health(self, request: Request) -> Response:
        fatal = getattr(self._engine, "fatal_error", None) if self._engine is not None else None
        if fatal:          # the engine lost its device context: tell the supervisor (503) instead of pretending
            return Response.json_response({"status": "error", "model": self.model_name, "engine": "failed",
                                           "error": fatal}, 503)
        return Response.json_response({"status": "ok", "model": self.model_name,
                                       "engine": "running" if self._engine is not None else "mock"})

    # ---- connection handling -----------------------------------------------------------------------------
    async def _handle_connection(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        try:
            while not self._stopping:
                try:
                    head = await asyncio.wait_for(reader.readuntil(b"\r\n\r\n"), 30.0)
                except (asyncio.IncompleteReadError, asyncio.TimeoutError, asyncio.LimitOverrunError, ConnectionError):
                    break
                n = content_length_of(head)
                if n > MAX_REQUEST_BYTES:
                    writer.write(format_http_response(Response.error("request body too large", 413)))
                    await writer.drain()
                    break
                body = await reader.readexactly(n) if n else b""
                req = parse_http_request(head + body)
                if req is None:
                    writer.write(format_http_response(Response.error("malformed request", 400)))
                    await writer.drain()
                    break
                keep = req.headers.get("connection", "").lower() == "keep-alive"
                resp = await self.router.handle(req)
                if resp.stream is not None:
                    writer.write(format_http_response(resp))
                    await writer.drain()
                    try:
                        async for chunk in resp.stream:
                            writer.write(chunk)
                            await writer.drain()
                            if writer.is_closing():
                                break
                    except (ConnectionError, asyncio.CancelledError):
                        pass
                    finally:
                        closer = getattr(resp.stream, "aclose", None)
                        if closer is not None:      # lets the stream's clean-up run (cancels an abandoned request)
                            try:
                                await closer()
                            except Exception:
                                pass
                    break
                writer.write(format_http_response(resp, keep))
                await writer.drain()
                if not keep:
                    break
        finally:
            try:
                writer.close()
                await writer.wait_closed()
            except Exception:
                pass

    async def start(self) -> None:
        if self._engine is not None and hasattr(self._engine, "run") and self._engine_thread is None:
            self._engine_thread = threading.Thread(target=self._engine.run, name="zse-engine", daemon=True)
            self._engine_thread.start()
        self._server = await asyncio.start_server(self._handle_connection, self.host, self.port, limit=MAX_REQUEST_BYTES)
        if self.port == 0:
            self.port = self._server.sockets[0].getsockname()[1]
        if not self.quiet:
            print(f"[zse] serving {self.model_name} on http://{self.host}:{self.port}")

    async def run_forever(self) -> None:
        await self.start()
        async with self._server:
            await self._server.serve_forever()

    def stop(self) -> None:
        self._stopping = True
        if self._engine is not None and hasattr(self._engine, "stop"):
            self._engine.stop()
        if self._server is not None:
            self._server.close()

    def close(self) -> None:
        self.stop()
        self._db.close()

    destroy = close

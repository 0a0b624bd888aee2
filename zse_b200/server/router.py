"""Minimal HTTP/1.1 plumbing for the asyncio server: request parsing, responses, a router with ``{param}`` path
segments, a middleware chain and static files with a traversal guard
(zse-engine/zse_engine/server/router.py:13-349).  No third-party web framework."""
from __future__ import annotations

import json
import mimetypes
import os
import re
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable, Dict, List, Optional, Tuple
from urllib.parse import parse_qs, unquote, urlsplit

STATUS_TEXT = {200: "OK", 201: "Created", 204: "No Content", 400: "Bad Request", 401: "Unauthorized",
               403: "Forbidden", 404: "Not Found", 405: "Method Not Allowed", 413: "Payload Too Large",
               429: "Too Many Requests", 500: "Internal Server Error", 503: "Service Unavailable",
               504: "Gateway Timeout"}
ERROR_TYPES = {400: "invalid_request_error", 401: "authentication_error", 403: "permission_error",
               404: "not_found_error", 429: "rate_limit_error", 500: "server_error", 503: "overloaded_error",
               504: "timeout_error"}


class _JsonObject(dict):
    def __call__(self):
        return self


class _JsonArray(list):
    def __call__(self):
        return self


@dataclass
class Request:
    method: str
    path: str
    headers: Dict[str, str] = field(default_factory=dict)
    body: bytes = b""
    query: Dict[str, str] = field(default_factory=dict)
    params: Dict[str, str] = field(default_factory=dict)
    context: Dict[str, Any] = field(default_factory=dict)     # filled by middleware (auth result, ...)

    @property
    def json(self) -> Optional[Any]:
        """The decoded body (None when absent or malformed).  Objects and arrays can also be CALLED and return
        themselves, so a handler written for the reference's ``request.json()`` method works unchanged."""
        if not self.body:
            return None
        try:
            obj = json.loads(self.body.decode("utf-8"))
        except (ValueError, UnicodeDecodeError):
            return None
        if isinstance(obj, dict):
            return _JsonObject(obj)
        if isinstance(obj, list):
            return _JsonArray(obj)
        return obj

    @property
    def authorization(self) -> Optional[str]:
        return self.headers.get("authorization")

    @property
    def content_type(self) -> str:
        return self.headers.get("content-type", "")

    # the reference's field names (zse-engine/zse_engine/server/router.py:14-23)
    @property
    def query_params(self) -> Dict[str, str]:
        return self.query

    @property
    def path_params(self) -> Dict[str, str]:
        return self.params

    @property
    def api_key(self) -> Any:
        """The key record the auth middleware attached (None on open servers and exempt paths)."""
        return self.context.get("api_key")

    @api_key.setter
    def api_key(self, key: Any) -> None:
        self.context["api_key"] = key


class Route:
    """One registered route: ``match(method, path)`` gives the path parameters or None
    (zse-engine/zse_engine/server/router.py:107-134).  ``*`` as the method matches every method."""

    def __init__(self, method: str, path: str, handler: "Handler"):
        self.method, self.path, self.handler = method.upper(), path, handler
        self.names = re.findall(r"\{(\w+)\}", path)
        self._rx = re.compile("^" + re.sub(r"\{\w+\}", r"([^/]+)", path.rstrip("/") or "/") + "/?$")

    def match(self, method: str, path: str) -> Optional[Dict[str, str]]:
        if self.method not in ("*", method.upper()):
            return None
        m = self._rx.match(path)
        return None if m is None else {n: unquote(v) for n, v in zip(self.names, m.groups())}


@dataclass
class Response:
    status: int = 200
    body: bytes = b""
    headers: Dict[str, str] = field(default_factory=dict)
    stream: Optional[Any] = None          # async iterator of bytes: sent as it is produced (SSE)

    @property
    def _is_streaming(self) -> bool:
        return self.headers.get("Content-Type", "").startswith("text/event-stream")

    @classmethod
    def json_response(cls, obj: Any, status: int = 200) -> "Response":
        return cls(status, json.dumps(obj).encode("utf-8"), {"Content-Type": "application/json"})

    @classmethod
    def text(cls, content: str, status: int = 200, content_type: str = "text/plain; charset=utf-8") -> "Response":
        return cls(status, content.encode("utf-8"), {"Content-Type": content_type})

    @classmethod
    def error(cls, message: str, status: int = 400, code: Optional[str] = None) -> "Response":
        return cls.json_response({"error": {"message": message, "type": ERROR_TYPES.get(status, "error"),
                                            "code": code or str(status)}}, status)

    @classmethod
    def sse(cls, iterator) -> "Response":
        return cls(200, b"", {"Content-Type": "text/event-stream", "Cache-Control": "no-cache",
                              "Connection": "keep-alive"}, iterator)

    # the reference's constructor names (zse-engine/zse_engine/server/router.py:49-98)
    @classmethod
    def json(cls, data: Any, status: int = 200) -> "Response":
        return cls.json_response(data, status)

    @classmethod
    def html(cls, content: str, status: int = 200) -> "Response":
        return cls.text(content, status, "text/html; charset=utf-8")

    @classmethod
    def streaming(cls, iterator=None) -> "Response":
        """Headers of an event stream; ``iterator`` (async, yielding bytes) is sent as the body."""
        r = cls.sse(iterator)
        r.headers["X-Accel-Buffering"] = "no"
        return r


Handler = Callable[[Request], Awaitable[Response]]
Middleware = Callable[[Request, Handler], Awaitable[Response]]


class Router:
    def __init__(self):
        self._routes: List[Route] = []
        self._middleware: List[Middleware] = []
        self._static: List[Tuple[str, str]] = []

    def add(self, method: str, path: str, handler: Handler) -> None:
        self._routes.append(Route(method, path, handler))

    def get(self, path: str, handler: Handler) -> None:
        self.add("GET", path, handler)

    def post(self, path: str, handler: Handler) -> None:
        self.add("POST", path, handler)

    def put(self, path: str, handler: Handler) -> None:
        self.add("PUT", path, handler)

    def delete(self, path: str, handler: Handler) -> None:
        self.add("DELETE", path, handler)

    def use(self, middleware: Middleware) -> None:
        self._middleware.append(middleware)

    def static(self, url_prefix: str, directory: str) -> None:
        self._static.append((url_prefix.rstrip("/") + "/", os.path.abspath(directory)))

    def set_static_dir(self, path: str) -> None:
        """Serves files of ``path`` for non-API paths (the reference's name for ``static("/", path)``)."""
        self.static("/", path)

    def routes(self) -> List[Tuple[str, str]]:
        return [(r.method, r._rx.pattern) for r in self._routes]

    async def handle(self, request: Request) -> Response:
        if request.method == "OPTIONS":
            return Response(204, b"", cors_headers())
        path_matched = False
        for route in self._routes:
            if not route._rx.match(request.path):
                continue
            path_matched = True
            params = route.match(request.method, request.path)
            if params is None:
                continue
            request.params = params
            call = route.handler
            for mw in reversed(self._middleware):
                call = (lambda h, w: (lambda req: w(req, h)))(call, mw)
            try:
                return await call(request)
            except Exception as exc:      # a handler bug must not kill the connection loop
                return Response.error(f"internal error: {type(exc).__name__}: {exc}", 500)
        if path_matched:
            return Response.error(f"method {request.method} not allowed for {request.path}", 405)
        if request.method == "GET":
            static = self._serve_static(request.path)
            if static is not None:
                return static
        return Response.error(f"no route for {request.method} {request.path}", 404)

    def _serve_static(self, path: str) -> Optional[Response]:
        for prefix, root in self._static:
            if path == prefix.rstrip("/") or path == prefix:
                rel = "index.html"
            elif path.startswith(prefix):
                rel = path[len(prefix):]
            else:
                continue
            full = os.path.abspath(os.path.join(root, unquote(rel)))
            if not (full == root or full.startswith(root + os.sep)):
                return Response.error("forbidden", 403)
            if os.path.isfile(full):
                ctype = mimetypes.guess_type(full)[0] or "application/octet-stream"
                with open(full, "rb") as f:
                    return Response(200, f.read(), {"Content-Type": ctype})
        return None


def cors_headers() -> Dict[str, str]:
    return {"Access-Control-Allow-Origin": "*", "Access-Control-Allow-Methods": "GET, POST, PUT, DELETE, OPTIONS",
            "Access-Control-Allow-Headers": "Content-Type, Authorization", "Access-Control-Max-Age": "86400"}


MAX_REQUEST_BYTES = 1 << 20


def parse_http_request(raw: bytes) -> Optional[Request]:
    """Parses a complete request (head + body) from ``raw``; ``None`` if the head is malformed."""
    head, sep, body = raw.partition(b"\r\n\r\n")
    if not sep:
        return None
    lines = head.decode("latin-1").split("\r\n")
    parts = lines[0].split(" ")
    if len(parts) < 2:
        return None
    method, target = parts[0].upper(), parts[1]
    headers = {}
    for line in lines[1:]:
        k, s, v = line.partition(":")
        if s:
            headers[k.strip().lower()] = v.strip()
    url = urlsplit(target)
    query = {k: v[-1] for k, v in parse_qs(url.query).items()}
    return Request(method, unquote(url.path) or "/", headers, body, query)


def content_length_of(head: bytes) -> int:
    m = re.search(rb"(?i)\r\ncontent-length:\s*(\d+)", head)
    return int(m.group(1)) if m else 0


def format_http_response(resp: Response, keep_alive: bool = False) -> bytes:
    headers = dict(cors_headers())
    headers.update(resp.headers)
    if resp.stream is None:
        headers["Content-Length"] = str(len(resp.body))
    headers.setdefault("Connection", "keep-alive" if keep_alive else "close")
    head = f"HTTP/1.1 {resp.status} {STATUS_TEXT.get(resp.status, 'Unknown')}\r\n" + \
        "".join(f"{k}: {v}\r\n" for k, v in headers.items()) + "\r\n"
    return head.encode("latin-1") + (resp.body if resp.stream is None else b"")

"""Unit tests of the server's building blocks - database, authentication, router, HTTP framing, SSE payloads -
without an engine or a socket (the shape of the reference's tests/test_server.py: DB, auth + rate limit, router, SSE
sections).  The routes with a live engine behind them are covered by tests/test_server.py."""
import asyncio
import json
import os
import time

import pytest

from zse_b200.server import sse
from zse_b200.server.auth import ADMIN, AuthManager
from zse_b200.server.database import ServerDatabase
from zse_b200.server.router import (MAX_REQUEST_BYTES, Request, Response, Route, Router, content_length_of,
                                    cors_headers, format_http_response, parse_http_request)


@pytest.fixture()
def db():
    d = ServerDatabase(":memory:")
    yield d
    d.close()


def run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


# ---- database: keys ---------------------------------------------------------------------------------------------
def test_generated_keys_have_the_documented_form_and_are_unique():
    keys = {ServerDatabase.generate_key() for _ in range(50)}
    assert len(keys) == 50
    for k in keys:
        assert k.startswith("sk-zse-") and len(k) == len("sk-zse-") + 64
        int(k[len("sk-zse-"):], 16)


def test_only_the_hash_of_a_key_is_stored(db):
    key, rec = db.create_key("alice")
    assert rec.key_hash == ServerDatabase.hash_key(key) and len(rec.key_hash) == 64
    assert rec.key_prefix == key[:14] and key not in json.dumps(rec.to_public())
    assert "key_hash" not in rec.to_public()


def test_create_validate_list_and_defaults(db):
    key, rec = db.create_key("alice")
    assert rec.name == "alice" and rec.is_active and rec.rate_limit_rpm == 60 and rec.rate_limit_tpm == 100000
    assert rec.allowed_models == "*" and rec.expires_at is None and rec.total_requests == 0
    got = db.validate_key(key)
    assert got is not None and got.id == rec.id
    assert db.validate_key(key + "0") is None and db.validate_key("") is None
    db.create_key("bob", rate_limit_rpm=5, allowed_models="a,b")
    names = [k.name for k in db.list_keys()]
    assert names == ["alice", "bob"]
    assert db.list_keys()[1].rate_limit_rpm == 5 and db.list_keys()[1].allowed_models == "a,b"


def test_expired_key_is_rejected(db):
    key, rec = db.create_key("short", expires_in_days=1e-9)
    assert rec.expires_at is not None
    time.sleep(0.01)
    assert db.validate_key(key) is None
    key2, _ = db.create_key("long", expires_in_days=30)
    assert db.validate_key(key2) is not None


def test_revoke_by_id_and_by_prefix(db):
    k1, r1 = db.create_key("one")
    k2, r2 = db.create_key("two")
    assert db.revoke_key(r1.id) is True and db.revoke_key(r1.id) is False        # second time: nothing to revoke
    assert db.validate_key(k1) is None and db.validate_key(k2) is not None
    assert db.revoke_key(999) is False
    assert db.revoke_key_by_prefix(r2.key_prefix) is True
    assert db.validate_key(k2) is None
    assert db.revoke_key_by_prefix("sk-zse-nothing") is False
    assert [k.is_active for k in db.list_keys()] == [False, False]              # rows stay, flagged


def test_update_key_limits_changes_only_what_is_given(db):
    _, r = db.create_key("k", rate_limit_rpm=10, rate_limit_tpm=1000)
    assert db.update_key_limits(r.id) is False
    assert db.update_key_limits(r.id, rate_limit_rpm=0) is True
    k = db.list_keys()[0]
    assert (k.rate_limit_rpm, k.rate_limit_tpm, k.allowed_models) == (0, 1000, "*")
    assert db.update_key_limits(r.id, allowed_models="m1") is True
    assert db.list_keys()[0].allowed_models == "m1"
    assert db.update_key_limits(12345, rate_limit_rpm=1) is False


def test_database_file_is_created_with_its_directory(tmp_path):
    path = tmp_path / "nested" / "dir" / "server.db"
    d = ServerDatabase(str(path))
    key, _ = d.create_key("persist")
    d.close()
    assert path.exists()
    d2 = ServerDatabase(str(path))                                                # reopen: the key is still valid
    assert d2.validate_key(key) is not None
    d2.close()


# ---- database: usage --------------------------------------------------------------------------------------------
def test_usage_is_accounted_per_key_and_in_total(db):
    _, a = db.create_key("a")
    _, b = db.create_key("b")
    db.record_usage(a.id, 10, 5, model="m", request_id="r1", latency_ms=100.0)
    db.record_usage(a.id, 1, 2, model="m", lora_id="ad", request_id="r2", latency_ms=300.0)
    db.record_usage(b.id, 7, 0, model="n")
    sa = db.get_usage_stats(a.id)
    assert sa == {"total_requests": 2, "prompt_tokens": 11, "completion_tokens": 7, "total_tokens": 18,
                  "avg_latency_ms": 200.0}
    assert db.get_usage_stats()["total_requests"] == 3 and db.get_usage_stats()["total_tokens"] == 25
    assert db.get_usage_stats(999)["total_requests"] == 0
    keys = {k.name: k for k in db.list_keys()}
    assert (keys["a"].total_requests, keys["a"].total_tokens) == (2, 18)
    assert (keys["b"].total_requests, keys["b"].total_tokens) == (1, 7)


def test_usage_window_counts_only_recent_rows(db):
    _, a = db.create_key("a")
    db.record_usage(a.id, 3, 4)
    assert db.get_usage_window(a.id, 60) == (1, 7)
    with db._lock:
        db._conn.execute("UPDATE usage SET timestamp = timestamp - 120")
        db._conn.commit()
    assert db.get_usage_window(a.id, 60) == (0, 0)
    assert db.get_usage_window(a.id, 600) == (1, 7)


def test_recent_usage_is_newest_first_and_limited(db):
    _, a = db.create_key("a")
    for i in range(5):
        db.record_usage(a.id, i, 0, request_id=f"r{i}")
    rows = db.recent_usage(a.id, limit=3)
    assert [r.request_id for r in rows] == ["r4", "r3", "r2"]
    assert rows[0].prompt_tokens == 4 and rows[0].total_tokens == 4 and rows[0].lora_id is None
    assert len(db.recent_usage()) == 5


def test_cleanup_removes_old_usage_only(db):
    _, a = db.create_key("a")
    db.record_usage(a.id, 1, 1, request_id="old")
    with db._lock:
        db._conn.execute("UPDATE usage SET timestamp = timestamp - 40 * 86400")
        db._conn.commit()
    db.record_usage(a.id, 1, 1, request_id="new")
    assert db.cleanup_old_usage(days=30) == 1
    assert [r.request_id for r in db.recent_usage()] == ["new"]
    assert db.list_keys()[0].total_requests == 2                                  # the key's counters are cumulative


# ---- database: chat history -------------------------------------------------------------------------------------
def test_chat_history_sessions(db):
    _, a = db.create_key("a")
    _, b = db.create_key("b")
    ids = [db.save_message(a.id, "s1", "user", "hi", model="m"),
           db.save_message(a.id, "s1", "assistant", "hello", model="m", lora_id="ad"),
           db.save_message(b.id, "s2", "user", "other")]
    assert ids == sorted(ids) and len(set(ids)) == 3
    msgs = db.get_session_messages("s1")
    assert [(m.role, m.content) for m in msgs] == [("user", "hi"), ("assistant", "hello")]
    assert msgs[1].lora_id == "ad" and msgs[0].key_id == a.id
    assert db.get_session_messages("s1", limit=1)[0].content == "hi"
    assert db.get_session_messages("nope") == []
    sessions = db.list_sessions()
    assert {s["session_id"]: s["messages"] for s in sessions} == {"s1": 2, "s2": 1}
    assert [s["session_id"] for s in db.list_sessions(key_id=b.id)] == ["s2"]
    assert db.delete_session("s1") == 2 and db.delete_session("s1") == 0
    assert [s["session_id"] for s in db.list_sessions()] == ["s2"]


def test_sessions_are_listed_most_recent_first(db):
    _, a = db.create_key("a")
    db.save_message(a.id, "old", "user", "1")
    time.sleep(0.01)
    db.save_message(a.id, "new", "user", "2")
    time.sleep(0.01)
    assert [s["session_id"] for s in db.list_sessions()] == ["new", "old"]
    db.save_message(a.id, "old", "assistant", "3")                                # activity moves it up
    assert [s["session_id"] for s in db.list_sessions()] == ["old", "new"]
    assert len(db.list_sessions(limit=1)) == 1


# ---- authentication ---------------------------------------------------------------------------------------------
def test_authenticate_header_forms(db):
    key, rec = db.create_key("k")
    auth = AuthManager(db, admin_key="root-key")
    assert auth.authenticate(None).status_code == 401 and "Missing" in auth.authenticate(None).error
    for bad in ("Basic abc", "Bearer", "Bearer   ", key):
        r = auth.authenticate(bad)
        assert not r.authenticated and r.status_code == 401 and "Bearer <key>" in r.error
    r = auth.authenticate("Bearer " + key)
    assert r.authenticated and r.key.id == rec.id and r.status_code == 200
    r = auth.authenticate("Bearer sk-zse-" + "0" * 64)
    assert not r.authenticated and "Invalid or expired" in r.error
    r = auth.authenticate("Bearer root-key")
    assert r.authenticated and r.key is ADMIN


def test_admin_key_is_optional_and_exact(db):
    assert AuthManager(db).is_admin("Bearer anything") is False                   # no admin key configured
    auth = AuthManager(db, admin_key="root-key")
    assert auth.is_admin("Bearer root-key") is True
    assert auth.is_admin("Bearer root-key2") is False and auth.is_admin(None) is False
    assert auth.is_admin("root-key") is False


def test_request_rate_limit(db):
    key, rec = db.create_key("k", rate_limit_rpm=2, rate_limit_tpm=0)
    auth = AuthManager(db)
    k = db.validate_key(key)
    assert auth.check_rate_limit(k).authenticated
    db.record_usage(rec.id, 1, 1)
    assert auth.check_rate_limit(k).authenticated
    db.record_usage(rec.id, 1, 1)
    r = auth.check_rate_limit(k)
    assert not r.authenticated and r.status_code == 429 and "2/2 requests/min" in r.error
    with db._lock:                                                                # a minute later the window is empty
        db._conn.execute("UPDATE usage SET timestamp = timestamp - 61")
        db._conn.commit()
    assert auth.check_rate_limit(k).authenticated


def test_token_rate_limit_and_unlimited_keys(db):
    key, rec = db.create_key("k", rate_limit_rpm=0, rate_limit_tpm=100)
    auth = AuthManager(db)
    k = db.validate_key(key)
    db.record_usage(rec.id, 60, 39)
    assert auth.check_rate_limit(k).authenticated
    db.record_usage(rec.id, 1, 0)
    r = auth.check_rate_limit(k)
    assert not r.authenticated and r.status_code == 429 and "100/100 tokens/min" in r.error
    key2, rec2 = db.create_key("free", rate_limit_rpm=0, rate_limit_tpm=0)
    for _ in range(5):
        db.record_usage(rec2.id, 10 ** 6, 0)
    assert auth.check_rate_limit(db.validate_key(key2)).authenticated
    assert auth.check_rate_limit(ADMIN).authenticated                             # the admin key has no limits


def test_model_allow_list(db):
    key, _ = db.create_key("k", allowed_models="qwen, llama")
    auth = AuthManager(db)
    k = db.validate_key(key)
    assert auth.check_model_access(k, "qwen").authenticated
    assert auth.check_model_access(k, "llama:my-adapter").authenticated           # model:adapter names the base model
    r = auth.check_model_access(k, "gemma")
    assert not r.authenticated and r.status_code == 403 and "gemma" in r.error
    key2, _ = db.create_key("any")
    assert auth.check_model_access(db.validate_key(key2), "whatever").authenticated


def test_full_auth_check_runs_the_three_stages_in_order(db):
    key, rec = db.create_key("k", rate_limit_rpm=1, allowed_models="m")
    auth = AuthManager(db)
    assert auth.full_auth_check(None, "m").status_code == 401
    assert auth.full_auth_check("Bearer " + key, "other").status_code == 403
    assert auth.full_auth_check("Bearer " + key, "m").authenticated
    assert auth.full_auth_check("Bearer " + key).authenticated                    # no model named: no model check
    db.record_usage(rec.id, 1, 1)
    assert auth.full_auth_check("Bearer " + key, "m").status_code == 429          # the limit comes before the model
    assert auth.full_auth_check("Bearer " + key, "other").status_code == 429


# ---- routes and router ------------------------------------------------------------------------------------------
def test_route_matching_and_parameters():
    r = Route("get", "/v1/items/{item_id}/parts/{part}", None)
    assert r.method == "GET" and r.names == ["item_id", "part"]
    assert r.match("GET", "/v1/items/7/parts/a%20b") == {"item_id": "7", "part": "a b"}
    assert r.match("GET", "/v1/items/7/parts/x/") == {"item_id": "7", "part": "x"}         # trailing slash
    assert r.match("POST", "/v1/items/7/parts/x") is None
    assert r.match("GET", "/v1/items/7/parts") is None and r.match("GET", "/v1/items/7/parts/x/y") is None
    anym = Route("*", "/ping", None)
    assert anym.match("DELETE", "/ping") == {} and anym.match("get", "/ping/") == {}
    root = Route("GET", "/", None)
    assert root.match("GET", "/") == {} and root.match("GET", "/x") is None


def _router():
    rt = Router()

    async def hello(req):
        return Response.json_response({"hello": req.params.get("name"), "q": req.query.get("q")})

    async def boom(req):
        raise ValueError("broken handler")

    rt.get("/hello/{name}", hello)
    rt.post("/boom", boom)
    rt.put("/thing", hello)
    rt.delete("/thing", hello)
    return rt


def test_router_dispatch_404_405_500_and_options():
    rt = _router()
    ok = run(rt.handle(Request("GET", "/hello/bob", query={"q": "1"})))
    assert ok.status == 200 and json.loads(ok.body) == {"hello": "bob", "q": "1"}
    nf = run(rt.handle(Request("GET", "/nothing")))
    assert nf.status == 404 and json.loads(nf.body)["error"]["type"] == "not_found_error"
    na = run(rt.handle(Request("POST", "/hello/bob")))
    assert na.status == 405 and "not allowed" in json.loads(na.body)["error"]["message"]
    err = run(rt.handle(Request("POST", "/boom")))
    assert err.status == 500 and "ValueError: broken handler" in json.loads(err.body)["error"]["message"]
    opt = run(rt.handle(Request("OPTIONS", "/anything/at/all")))
    assert opt.status == 204 and opt.headers["Access-Control-Allow-Origin"] == "*"
    assert run(rt.handle(Request("PUT", "/thing"))).status == 200
    assert run(rt.handle(Request("DELETE", "/thing"))).status == 200
    assert ("GET", Route("GET", "/hello/{name}", None)._rx.pattern) in rt.routes()


def test_middleware_wraps_in_registration_order_and_can_short_circuit():
    rt = _router()
    seen = []

    async def outer(req, nxt):
        seen.append("outer-in")
        req.context["who"] = "outer"
        resp = await nxt(req)
        seen.append("outer-out")
        resp.headers["X-Outer"] = "1"
        return resp

    async def gate(req, nxt):
        seen.append("gate")
        if req.query.get("deny"):
            return Response.error("denied", 403)
        assert req.context["who"] == "outer"
        return await nxt(req)

    rt.use(outer)
    rt.use(gate)
    ok = run(rt.handle(Request("GET", "/hello/x")))
    assert ok.status == 200 and ok.headers["X-Outer"] == "1" and seen == ["outer-in", "gate", "outer-out"]
    seen.clear()
    no = run(rt.handle(Request("GET", "/hello/x", query={"deny": "1"})))
    assert no.status == 403 and no.headers["X-Outer"] == "1" and seen == ["outer-in", "gate", "outer-out"]


def test_static_files_index_types_and_traversal(tmp_path):
    (tmp_path / "index.html").write_text("<h1>home</h1>")
    (tmp_path / "app.js").write_text("console.log(1)")
    (tmp_path / "sub").mkdir()
    (tmp_path / "sub" / "data.bin").write_bytes(b"\x00\x01")
    secret = tmp_path.parent / "secret.txt"
    secret.write_text("no")
    rt = _router()
    rt.set_static_dir(str(tmp_path))
    home = run(rt.handle(Request("GET", "/")))
    assert home.status == 200 and home.body == b"<h1>home</h1>" and home.headers["Content-Type"].startswith("text/html")
    js = run(rt.handle(Request("GET", "/app.js")))
    assert js.status == 200 and "javascript" in js.headers["Content-Type"]
    blob = run(rt.handle(Request("GET", "/sub/data.bin")))
    assert blob.status == 200 and blob.body == b"\x00\x01"
    assert run(rt.handle(Request("GET", "/missing.css"))).status == 404
    assert run(rt.handle(Request("GET", "/../secret.txt"))).status in (403, 404)
    assert run(rt.handle(Request("GET", "/%2e%2e/secret.txt"))).status in (403, 404)
    assert run(rt.handle(Request("POST", "/app.js"))).status == 404                # static files answer GET only
    assert run(rt.handle(Request("GET", "/hello/bob"))).status == 200              # routes come first


def test_static_under_a_prefix(tmp_path):
    (tmp_path / "index.html").write_text("dash")
    rt = Router()
    rt.static("/dashboard", str(tmp_path))
    assert run(rt.handle(Request("GET", "/dashboard"))).body == b"dash"
    assert run(rt.handle(Request("GET", "/dashboard/"))).body == b"dash"
    assert run(rt.handle(Request("GET", "/dashboard/index.html"))).body == b"dash"
    assert run(rt.handle(Request("GET", "/index.html"))).status == 404


# ---- request and response objects -------------------------------------------------------------------------------
def test_request_json_accessors():
    r = Request("POST", "/x", {"authorization": "Bearer k", "content-type": "application/json"}, b'{"a": [1, 2]}',
                {"q": "v"}, {"id": "7"})
    assert r.json == {"a": [1, 2]} and r.json() == {"a": [1, 2]}                  # property and (reference) method
    assert r.authorization == "Bearer k" and r.content_type == "application/json"
    assert r.query_params == {"q": "v"} and r.path_params == {"id": "7"}
    assert r.api_key is None
    r.api_key = "record"
    assert r.api_key == "record" and r.context["api_key"] == "record"
    assert Request("POST", "/x", body=b"[1, 2]").json() == [1, 2]
    assert Request("POST", "/x", body=b"3").json == 3
    assert Request("POST", "/x", body=b"{not json").json is None
    assert Request("POST", "/x", body=b"\xff\xfe").json is None
    assert Request("GET", "/x").json is None and Request("GET", "/x").content_type == ""


def test_response_constructors():
    j = Response.json({"a": 1}, 201)
    assert j.status == 201 and json.loads(j.body) == {"a": 1} and j.headers["Content-Type"] == "application/json"
    t = Response.text("héllo")
    assert t.body == "héllo".encode("utf-8") and "charset=utf-8" in t.headers["Content-Type"]
    h = Response.html("<p>x</p>", 200)
    assert h.headers["Content-Type"].startswith("text/html")
    for status, kind in ((400, "invalid_request_error"), (401, "authentication_error"), (404, "not_found_error"),
                         (429, "rate_limit_error"), (500, "server_error")):
        e = json.loads(Response.error("m", status).body)["error"]
        assert e["message"] == "m" and e["code"] == str(status) and e["type"] == kind
    assert json.loads(Response.error("m", 400, code="bad_thing").body)["error"]["code"] == "bad_thing"
    s = Response.streaming(iter(()))
    assert s._is_streaming and s.headers["Cache-Control"] == "no-cache" and s.headers["X-Accel-Buffering"] == "no"
    assert not j._is_streaming and s.stream is not None


# ---- HTTP framing -----------------------------------------------------------------------------------------------
def test_parse_http_request():
    raw = (b"POST /v1/chat/completions?stream=1&x=a%20b&x=last HTTP/1.1\r\nHost: h\r\nAuthorization: Bearer k\r\n"
           b"Content-Type: application/json\r\nContent-Length: 7\r\n\r\n{\"a\":1}")
    r = parse_http_request(raw)
    assert r.method == "POST" and r.path == "/v1/chat/completions"
    assert r.query == {"stream": "1", "x": "last"}                                # the last value of a repeated name
    assert r.headers["authorization"] == "Bearer k" and r.headers["host"] == "h"  # names are lower-cased
    assert r.body == b'{"a":1}' and r.json == {"a": 1}
    assert parse_http_request(b"GET /a%20b HTTP/1.1\r\n\r\n").path == "/a b"
    assert parse_http_request(b"get / HTTP/1.1\r\n\r\n").method == "GET"
    assert parse_http_request(b"GET / HTTP/1.1\r\nHost: h\r\n") is None            # head not complete
    assert parse_http_request(b"GARBAGE\r\n\r\n") is None
    assert MAX_REQUEST_BYTES == 1 << 20


def test_content_length_of():
    assert content_length_of(b"POST / HTTP/1.1\r\nContent-Length: 42\r\n") == 42
    assert content_length_of(b"POST / HTTP/1.1\r\ncontent-length:7\r\n") == 7
    assert content_length_of(b"GET / HTTP/1.1\r\nHost: x\r\n") == 0


def test_format_http_response():
    out = format_http_response(Response.json_response({"ok": True}))
    head, _, body = out.partition(b"\r\n\r\n")
    lines = head.decode().split("\r\n")
    assert lines[0] == "HTTP/1.1 200 OK" and body == b'{"ok": true}'
    hdr = dict(l.split(": ", 1) for l in lines[1:])
    assert hdr["Content-Length"] == str(len(body)) and hdr["Connection"] == "close"
    assert hdr["Access-Control-Allow-Origin"] == "*" and hdr["Content-Type"] == "application/json"
    keep = format_http_response(Response.text("x"), keep_alive=True)
    assert b"Connection: keep-alive" in keep
    assert format_http_response(Response.error("nope", 404)).startswith(b"HTTP/1.1 404 Not Found")
    assert format_http_response(Response.error("slow", 429)).startswith(b"HTTP/1.1 429 ")
    stream = format_http_response(Response.sse(iter(())))
    assert b"Content-Length" not in stream and b"text/event-stream" in stream and stream.endswith(b"\r\n\r\n")
    assert set(cors_headers()) >= {"Access-Control-Allow-Origin", "Access-Control-Allow-Methods",
                                   "Access-Control-Allow-Headers"}


# ---- SSE payloads -----------------------------------------------------------------------------------------------
def _payload(chunk: bytes):
    assert chunk.startswith(b"data: ") and chunk.endswith(b"\n\n")
    return json.loads(chunk[len(b"data: "):])


def test_sse_chat_chunks():
    first = _payload(sse.chat_chunk("cmpl-1", "m", role="assistant"))
    assert first["object"] == "chat.completion.chunk" and first["id"] == "cmpl-1" and first["model"] == "m"
    assert first["choices"] == [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]
    mid = _payload(sse.chat_chunk("cmpl-1", "m", content="héllo\n"))
    assert mid["choices"][0]["delta"] == {"content": "héllo\n"}
    last = _payload(sse.chat_chunk("cmpl-1", "m", finish_reason="stop"))
    assert last["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "stop"}
    assert abs(first["created"] - time.time()) < 5
    # the reference's names: an empty token text carries no content
    assert _payload(sse.sse_chat_chunk("c", "m", "", finish_reason="length"))["choices"][0]["delta"] == {}
    assert _payload(sse.sse_chat_chunk("c", "m", "tok"))["choices"][0]["delta"] == {"content": "tok"}
    assert _payload(sse.sse_chat_chunk("c", "m", "", role="assistant"))["choices"][0]["delta"] == {"role": "assistant"}


def test_sse_completion_chunks_and_done():
    c = _payload(sse.completion_chunk("cmpl-2", "m", "text"))
    assert c["object"] == "text_completion" and c["choices"] == [{"index": 0, "text": "text", "finish_reason": None}]
    end = _payload(sse.sse_completion_chunk("cmpl-2", "m", "", finish_reason="stop"))
    assert end["choices"][0] == {"index": 0, "text": "", "finish_reason": "stop"}
    assert sse.sse_done() == b"data: [DONE]\n\n" == sse.SSE_DONE
    assert sse.sse_event({"a": "b\nc"}) == b'data: {"a": "b\\nc"}\n\n'            # a newline never splits an event


# ---- chat layouts -----------------------------------------------------------------------------------------------
CONVERSATION = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"},
                {"role": "assistant", "content": "Hello."}, {"role": "user", "content": "Bye"}]


def test_chat_layouts_of_the_model_families():
    from zse_b200.server.api_openai import (TEMPLATES, format_chatml, format_gemma, format_llama, format_llama3,
                                            format_phi3)
    assert set(TEMPLATES) == {"chatml", "llama", "llama3", "phi3", "gemma"}
    assert format_chatml(CONVERSATION) == (
        "<|im_start|>system\nBe brief.<|im_end|>\n<|im_start|>user\nHi<|im_end|>\n"
        "<|im_start|>assistant\nHello.<|im_end|>\n<|im_start|>user\nBye<|im_end|>\n<|im_start|>assistant\n")
    assert format_llama(CONVERSATION) == (
        "[INST] <<SYS>>\nBe brief.\n<</SYS>>\n\nHi [/INST] Hello. </s>[INST] Bye [/INST]")
    assert format_llama([{"role": "user", "content": "Hi"}]) == "[INST] Hi [/INST]"
    assert format_llama3(CONVERSATION[1:2]) == (
        "<|start_header_id|>user<|end_header_id|>\n\nHi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    assert format_phi3(CONVERSATION[1:3]) == "<|user|>\nHi<|end|>\n<|assistant|>\nHello.<|end|>\n<|assistant|>\n"
    g = format_gemma(CONVERSATION[1:])
    assert g == ("<start_of_turn>user\nHi<end_of_turn>\n<start_of_turn>model\nHello.<end_of_turn>\n"
                 "<start_of_turn>user\nBye<end_of_turn>\n<start_of_turn>model\n")        # "assistant" is "model" there
    for fmt in TEMPLATES.values():                                                # every layout ends at the model's turn
        assert fmt([{"content": "no role given"}])                                # ... and defaults the role to user


def test_layout_follows_the_tokenizer_before_the_architecture():
    from zse_b200.server.api_openai import template_for_arch

    class Tok:
        def __init__(self, *tokens):
            self.tokens = set(tokens)

        def token_to_id(self, t):
            return 1 if t in self.tokens else None

    assert template_for_arch("llama", Tok("<|im_start|>")) == "chatml"
    assert template_for_arch("llama", Tok("<|start_header_id|>", "<|eot_id|>")) == "llama3"   # Llama 3 files
    assert template_for_arch("llama", Tok()) == "llama" and template_for_arch("mistral") == "llama"
    assert template_for_arch("qwen2") == "chatml"
    assert template_for_arch("phi3", Tok("<|assistant|>", "<|end|>")) == "phi3"
    assert template_for_arch("phi3") == "chatml"                # without the marker tokens the markers would be text
    assert template_for_arch("gemma2") == "gemma" and template_for_arch("gemma4") == "gemma"
    assert template_for_arch("") == "chatml" and template_for_arch("something-new") == "chatml"


def test_markers_end_the_visible_text():
    from zse_b200.server.api_openai import CHAT_MARKERS, strip_markers
    assert {"<|im_end|>", "<|im_start|>", "<|eot_id|>", "<end_of_turn>", "</s>"} <= set(CHAT_MARKERS)
    assert strip_markers("Hello there.<|im_end|>\n<|im_start|>user") == "Hello there."
    assert strip_markers("Answer  \n</s>trailing") == "Answer"
    assert strip_markers("two<end_of_turn>and<|eot_id|>more") == "two"
    assert strip_markers("nothing to cut  ") == "nothing to cut"

"""The HTTP API of a server that has no model loaded ("mock" mode of the reference's tests/test_server.py): every route
is registered and answers through the same router, authentication and accounting as with an engine, so the whole API
surface can be exercised in milliseconds - requests are handed to the router directly, no socket is opened."""
import asyncio
import json

import pytest

from zse_b200.server.app import ZSEServer
from zse_b200.server.router import Request

ADMIN = {"authorization": "Bearer admin-secret"}


def call(srv, method, path, body=None, headers=None, query=None):
    raw = json.dumps(body).encode() if body is not None else b""
    req = Request(method, path, dict(headers or {}), raw, dict(query or {}))
    resp = asyncio.new_event_loop().run_until_complete(srv.router.handle(req))
    data = json.loads(resp.body) if resp.body and resp.headers.get("Content-Type", "").startswith("application/json") \
        else resp.body
    return resp.status, data


@pytest.fixture()
def srv():
    s = ZSEServer(model_path=None, admin_key="admin-secret", db_path=":memory:", model_name="mock-model", quiet=True,
                  enable_rag=False)
    yield s
    s.database.close()


@pytest.fixture()
def locked():
    s = ZSEServer(model_path=None, admin_key="admin-secret", db_path=":memory:", model_name="mock-model", quiet=True,
                  enable_rag=False, require_auth=True)
    yield s
    s.database.close()


def new_key(srv, **kw):
    status, out = call(srv, "POST", "/v1/admin/keys/create", dict(name="k", **kw), ADMIN)
    assert status == 201
    return out


# ---- health, models, completions --------------------------------------------------------------------------------
def test_health_reports_mock_mode(srv):
    for path in ("/health", "/v1/health"):
        status, out = call(srv, "GET", path)
        assert status == 200 and out == {"status": "ok", "model": "mock-model", "engine": "mock"}
    assert srv.engine is None


def test_models_list_names_the_served_model(srv):
    status, out = call(srv, "GET", "/v1/models")
    assert status == 200 and out["object"] == "list"
    assert [m["id"] for m in out["data"]] == ["mock-model"]
    m = out["data"][0]
    assert m["object"] == "model" and m["owned_by"] == "zse" and m["permission"] == [] and isinstance(m["created"], int)


def test_chat_completion_has_the_openai_shape(srv):
    status, out = call(srv, "POST", "/v1/chat/completions",
                       {"model": "mock-model", "messages": [{"role": "user", "content": "hi"}]})
    assert status == 200 and out["object"] == "chat.completion" and out["model"] == "mock-model"
    assert out["id"].startswith("chatcmpl-") and len(out["id"]) == len("chatcmpl-") + 24 and isinstance(out["created"], int)
    int(out["id"][len("chatcmpl-"):], 16)
    choice = out["choices"][0]
    assert choice["index"] == 0 and choice["finish_reason"] == "stop"
    assert choice["message"] == {"role": "assistant", "content": "This is a mock response (no model loaded)."}
    u = out["usage"]
    assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"] and u["completion_tokens"] == 8


def test_text_completion_has_the_openai_shape(srv):
    status, out = call(srv, "POST", "/v1/completions", {"prompt": "once upon a time", "max_tokens": 4})
    assert status == 200 and out["object"] == "text_completion"
    assert out["choices"][0]["text"].startswith("This is a mock response") and out["id"].startswith("cmpl-")


def test_bad_requests_are_refused_before_generation(srv):
    assert call(srv, "POST", "/v1/chat/completions", {"model": "m"})[0] == 400                 # no messages
    assert call(srv, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
    assert call(srv, "POST", "/v1/completions", {"model": "m"})[0] == 400                      # no prompt
    status, out = call(srv, "POST", "/v1/chat/completions",
                       {"messages": [{"role": "user", "content": "x"}], "temperature": "hot"})
    assert status == 400 and out["error"]["type"] == "invalid_request_error"
    req = Request("POST", "/v1/chat/completions", {}, b"{not json", {})
    resp = asyncio.new_event_loop().run_until_complete(srv.router.handle(req))
    assert resp.status == 400
    assert call(srv, "GET", "/v1/chat/completions")[0] == 405
    assert call(srv, "GET", "/v1/nothing/here")[0] == 404


# ---- keys -------------------------------------------------------------------------------------------------------
def test_admin_routes_need_the_admin_key(srv):
    assert call(srv, "POST", "/v1/admin/keys/create", {"name": "x"})[0] == 403
    assert call(srv, "GET", "/v1/admin/keys/list", headers={"authorization": "Bearer wrong"})[0] == 403
    key = new_key(srv)
    assert call(srv, "GET", "/v1/admin/stats", headers={"authorization": "Bearer " + key["key"]})[0] == 403
    assert call(srv, "GET", "/v1/admin/stats", headers=ADMIN)[0] == 200


def test_key_lifecycle_create_list_update_revoke(srv):
    out = new_key(srv, rate_limit_rpm=7, allowed_models="mock-model")
    assert out["key"].startswith("sk-zse-") and out["prefix"] == out["key"][:14] and out["rate_limit_rpm"] == 7
    status, listed = call(srv, "GET", "/v1/admin/keys/list", headers=ADMIN)
    assert status == 200 and len(listed["keys"]) == 1 and "key" not in listed["keys"][0]       # shown once only
    assert call(srv, "POST", "/v1/admin/keys/update", {"id": out["id"], "rate_limit_rpm": 99}, ADMIN) == \
        (200, {"updated": True})
    assert call(srv, "GET", "/v1/admin/keys/list", headers=ADMIN)[1]["keys"][0]["rate_limit_rpm"] == 99
    assert call(srv, "POST", "/v1/admin/keys/update", {"rate_limit_rpm": 1}, ADMIN)[0] == 400  # no id
    assert call(srv, "POST", "/v1/admin/keys/update", {"id": 555, "rate_limit_rpm": 1}, ADMIN)[0] == 404
    assert call(srv, "POST", "/v1/admin/keys/revoke", {}, ADMIN)[0] == 400
    assert call(srv, "POST", "/v1/admin/keys/revoke", {"id": out["id"]}, ADMIN) == (200, {"revoked": True})
    assert call(srv, "POST", "/v1/admin/keys/revoke", {"id": out["id"]}, ADMIN)[0] == 404
    second = new_key(srv)
    assert call(srv, "POST", "/v1/admin/keys/revoke", {"prefix": second["prefix"]}, ADMIN)[0] == 200
    assert [k["is_active"] for k in call(srv, "GET", "/v1/admin/keys/list", headers=ADMIN)[1]["keys"]] == [False, False]


def test_an_open_server_takes_requests_without_a_key_but_checks_a_key_that_is_shown(srv):
    body = {"messages": [{"role": "user", "content": "x"}]}
    assert call(srv, "POST", "/v1/chat/completions", body)[0] == 200
    assert call(srv, "POST", "/v1/chat/completions", body, {"authorization": "Bearer sk-zse-bogus"})[0] == 401
    key = new_key(srv)
    assert call(srv, "POST", "/v1/chat/completions", body, {"authorization": "Bearer " + key["key"]})[0] == 200


def test_a_locked_server_wants_a_valid_key_for_the_api_but_not_for_health(locked):
    body = {"messages": [{"role": "user", "content": "x"}]}
    status, out = call(locked, "POST", "/v1/chat/completions", body)
    assert status == 401 and "Missing Authorization" in out["error"]["message"]
    assert call(locked, "GET", "/v1/models")[0] == 401
    assert call(locked, "GET", "/health")[0] == 200 and call(locked, "GET", "/v1/health")[0] == 200
    key = new_key(locked)
    auth = {"authorization": "Bearer " + key["key"]}
    assert call(locked, "POST", "/v1/chat/completions", body, auth)[0] == 200
    assert call(locked, "GET", "/v1/models", headers=auth)[0] == 200
    assert call(locked, "POST", "/v1/chat/completions", body, ADMIN)[0] == 200                  # the admin key passes
    call(locked, "POST", "/v1/admin/keys/revoke", {"id": key["id"]}, ADMIN)
    assert call(locked, "POST", "/v1/chat/completions", body, auth)[0] == 401


def test_model_allow_list_and_rate_limit_apply_to_completions(locked):
    body = {"model": "mock-model", "messages": [{"role": "user", "content": "x"}]}
    narrow = new_key(locked, allowed_models="other-model")
    status, out = call(locked, "POST", "/v1/chat/completions", body, {"authorization": "Bearer " + narrow["key"]})
    assert status == 403 and "not allowed" in out["error"]["message"]
    limited = new_key(locked, rate_limit_rpm=2)
    auth = {"authorization": "Bearer " + limited["key"]}
    locked.database.record_usage(limited["id"], 1, 1)
    assert call(locked, "POST", "/v1/chat/completions", body, auth)[0] == 200
    locked.database.record_usage(limited["id"], 1, 1)
    status, out = call(locked, "POST", "/v1/chat/completions", body, auth)
    assert status == 429 and out["error"]["type"] == "rate_limit_error"


# ---- statistics and dashboard sessions --------------------------------------------------------------------------
def test_stats_and_usage_without_an_engine(srv):
    key = new_key(srv)
    srv.database.record_usage(key["id"], 10, 5, model="mock-model", latency_ms=50.0)
    status, out = call(srv, "GET", "/v1/admin/stats", headers=ADMIN)
    assert status == 200 and out["num_keys"] == 1 and out["usage"]["total_tokens"] == 15 and "engine" not in out
    status, out = call(srv, "GET", "/v1/admin/usage", headers=ADMIN, query={"key_id": str(key["id"])})
    assert status == 200 and out["total_requests"] == 1 and out["avg_latency_ms"] == 50.0
    assert call(srv, "GET", "/v1/admin/usage", headers=ADMIN, query={"key_id": "999"})[1]["total_requests"] == 0


def test_dashboard_sessions_round_trip(srv):
    key = new_key(srv)
    auth = {"authorization": "Bearer " + key["key"]}
    assert call(srv, "POST", "/v1/dashboard/session")[0] == 401                                 # a key is needed here
    status, out = call(srv, "POST", "/v1/dashboard/session", headers=auth)
    assert status == 201 and len(out["session_id"]) == 16
    sid = out["session_id"]
    assert call(srv, "POST", f"/v1/dashboard/session/{sid}/message", {"role": "user"}, auth)[0] == 400
    assert call(srv, "POST", f"/v1/dashboard/session/{sid}/message", {"role": "user", "content": "hello"}, auth)[0] == 201
    call(srv, "POST", f"/v1/dashboard/session/{sid}/message",
         {"role": "assistant", "content": "hi there", "model": "mock-model"}, auth)
    status, out = call(srv, "GET", f"/v1/dashboard/session/{sid}", headers=auth)
    assert status == 200 and [(m["role"], m["content"]) for m in out["messages"]] == \
        [("user", "hello"), ("assistant", "hi there")]
    status, out = call(srv, "GET", "/v1/dashboard/sessions", headers=auth)
    assert status == 200 and [(s["session_id"], s["messages"]) for s in out["sessions"]] == [(sid, 2)]
    other = new_key(srv)
    status, out = call(srv, "GET", "/v1/dashboard/sessions", headers={"authorization": "Bearer " + other["key"]})
    assert out["sessions"] == []                                                                # a key sees its own
    assert len(call(srv, "GET", "/v1/dashboard/sessions", headers=ADMIN)[1]["sessions"]) == 1   # the admin sees all
    assert call(srv, "DELETE", f"/v1/dashboard/session/{sid}", headers=auth) == (200, {"deleted": 2})
    assert call(srv, "GET", f"/v1/dashboard/session/{sid}", headers=auth)[1]["messages"] == []


# ---- static files -----------------------------------------------------------------------------------------------
def test_the_dashboard_is_served_from_the_root(srv):
    status, body = call(srv, "GET", "/")
    assert status == 200 and b"<html" in body.lower()
    status, body = call(srv, "GET", "/app.js")
    assert status == 200 and len(body) > 1000
    assert call(srv, "GET", "/style.css")[0] == 200
    assert call(srv, "GET", "/../app.py")[0] in (403, 404)


# ---- LoRA routes without an engine, and with a stand-in manager -------------------------------------------------
def test_lora_routes_without_an_engine(srv):
    assert call(srv, "GET", "/v1/lora/list") == (200, {"adapters": []})
    assert call(srv, "GET", "/v1/lora/stats") == (200, {"num_adapters": 0})
    assert call(srv, "POST", "/v1/lora/load", {"adapter_id": "a", "path": "/x"})[0] == 403      # admin only
    status, out = call(srv, "POST", "/v1/lora/load", {"adapter_id": "a", "path": "/x"}, ADMIN)
    assert status == 503 and "no engine" in out["error"]["message"]
    assert call(srv, "POST", "/v1/lora/unload", {"adapter_id": "a"})[0] == 403
    assert call(srv, "POST", "/v1/lora/unload", {"adapter_id": "a"}, ADMIN)[0] == 400


class _FakeAdapter:
    adapter_id, rank, alpha, target_modules, num_layers, total_bytes = "a1", 8, 16.0, ["q_proj"], 2, 4096


class _FakeManager:
    def __init__(self):
        self.loaded = {}

    def list_adapters(self):
        return [{"adapter_id": k} for k in self.loaded]

    def stats(self):
        return {"num_adapters": len(self.loaded)}

    def load_adapter(self, aid, path):
        if aid in self.loaded:
            raise ValueError(f"adapter '{aid}' is already loaded")
        self.loaded[aid] = path
        return _FakeAdapter()

    def unload_adapter(self, aid):
        return self.loaded.pop(aid, None) is not None


class _FakeEngine:
    tokenizer = None

    def __init__(self):
        self.lora_manager = _FakeManager()


def test_lora_load_and_unload_through_the_routes(tmp_path):
    eng = _FakeEngine()
    s = ZSEServer(engine=eng, admin_key="admin-secret", db_path=":memory:", quiet=True, enable_rag=False)
    try:
        f = tmp_path / "a.zse-lora"
        f.write_bytes(b"x")
        assert call(s, "POST", "/v1/lora/load", {"adapter_id": "a1"}, ADMIN)[0] == 400           # path missing
        assert call(s, "POST", "/v1/lora/load", {"adapter_id": "a1", "path": str(tmp_path / "none")}, ADMIN)[0] == 404
        status, out = call(s, "POST", "/v1/lora/load", {"adapter_id": "a1", "path": str(f)}, ADMIN)
        assert status == 201 and out == {"adapter_id": "a1", "rank": 8, "alpha": 16.0, "target_modules": ["q_proj"],
                                          "num_layers": 2, "bytes": 4096}
        status, out = call(s, "POST", "/v1/lora/load", {"adapter_id": "a1", "path": str(f)}, ADMIN)
        assert status == 400 and "already loaded" in out["error"]["message"]
        assert call(s, "GET", "/v1/lora/list")[1] == {"adapters": [{"adapter_id": "a1"}]}
        assert call(s, "GET", "/v1/lora/stats")[1] == {"num_adapters": 1}
        assert call(s, "POST", "/v1/lora/unload", {"adapter_id": "a1"}, ADMIN) == (200, {"unloaded": "a1"})
        assert call(s, "POST", "/v1/lora/unload", {"adapter_id": "a1"}, ADMIN)[0] == 404
        assert call(s, "GET", "/health")[1]["engine"] == "running"
        # every loaded adapter is also a model name "<model>:<adapter>"
        call(s, "POST", "/v1/lora/load", {"adapter_id": "a2", "path": str(f)}, ADMIN)
        assert [m["id"] for m in call(s, "GET", "/v1/models")[1]["data"]] == ["zse-model", "zse-model:a2"]
    finally:
        s.database.close()


# ---- /metrics ---------------------------------------------------------------------------------------------------
def _metrics(text):
    out = {}
    for line in text.decode().splitlines():
        if line and not line.startswith("#"):
            name, value = line.split(" ")
            out[name] = float(value)
    return out


def test_metrics_in_prometheus_text_format(srv, locked):
    key = new_key(srv)
    srv.database.record_usage(key["id"], 10, 5)
    req = Request("GET", "/metrics")
    resp = asyncio.new_event_loop().run_until_complete(srv.router.handle(req))
    assert resp.status == 200 and resp.headers["Content-Type"].startswith("text/plain; version=0.0.4")
    text = resp.body.decode()
    assert "# TYPE zse_engine_up gauge" in text and "# HELP zse_api_tokens_total" in text and text.endswith("\n")
    m = _metrics(resp.body)
    assert m["zse_engine_up"] == 0 and m["zse_api_requests_total"] == 1 and m["zse_api_tokens_total"] == 15
    # where keys are required the numbers are for the admin only
    assert call(locked, "GET", "/metrics")[0] == 403
    assert call(locked, "GET", "/metrics", headers=ADMIN)[0] == 200


def test_session_save_route_of_the_reference(srv):
    key = new_key(srv)
    auth = {"authorization": "Bearer " + key["key"]}
    body = {"session_id": "s-1", "role": "user", "content": "hello", "model": "mock-model"}
    assert call(srv, "POST", "/v1/dashboard/session/save", body)[0] == 401
    assert call(srv, "POST", "/v1/dashboard/session/save", body, auth) == (200, {"ok": True})
    assert call(srv, "POST", "/v1/dashboard/session/save", dict(body, content=""), auth)[0] == 400
    assert call(srv, "POST", "/v1/dashboard/session/save", {"role": "user", "content": "x"}, auth)[0] == 400
    call(srv, "POST", "/v1/dashboard/session/save", dict(body, role="assistant", content="hi", lora_id="ad"), auth)
    msgs = call(srv, "GET", "/v1/dashboard/session/s-1", headers=auth)[1]["messages"]
    assert [(m["role"], m["content"]) for m in msgs] == [("user", "hello"), ("assistant", "hi")]
    # "save" is a route of its own, not a session id
    assert call(srv, "GET", "/v1/dashboard/session/save", headers=auth)[1]["messages"] == []


# ---- retrieval routes without a model (lexical search only) -----------------------------------------------------
@pytest.fixture()
def rag_srv():
    s = ZSEServer(model_path=None, admin_key="admin-secret", db_path=":memory:", model_name="mock-model", quiet=True,
                  enable_rag=True)
    yield s
    s.database.close()


def test_document_lifecycle_and_lexical_search(rag_srv):
    import base64
    s = rag_srv
    assert call(s, "GET", "/v1/rag/documents") == (200, {"documents": []})
    assert call(s, "POST", "/v1/rag/upload", {"text": "no name"})[0] == 400
    assert call(s, "POST", "/v1/rag/upload", {"filename": "a.txt"})[0] == 400
    assert call(s, "POST", "/v1/rag/upload", {"filename": "a.txt", "content": "not base64!!"})[0] == 400
    text_a = "The paged key value cache stores attention keys in fixed size blocks. " * 6
    text_b = "Speculative decoding drafts several tokens and verifies them in one pass. " * 6
    status, a = call(s, "POST", "/v1/rag/upload", {"filename": "cache.txt", "text": text_a})
    assert status == 201 and a["chunk_count"] >= 1 and a["doc_type"] == "text"
    status, b = call(s, "POST", "/v1/rag/upload",
                     {"filename": "spec.md", "content": base64.b64encode(text_b.encode()).decode()})
    assert status == 201 and b["doc_id"] != a["doc_id"]
    docs = call(s, "GET", "/v1/rag/documents")[1]["documents"]
    assert sorted(d["name"] for d in docs) == ["cache.txt", "spec.md"]
    status, doc = call(s, "GET", f"/v1/rag/document/{a['doc_id']}")
    assert status == 200 and doc["name"] == "cache.txt" and doc["chunks"][0]["content"].startswith("The paged key")
    assert call(s, "GET", "/v1/rag/document/9999")[0] == 404 and call(s, "GET", "/v1/rag/document/abc")[0] == 404
    # search: BM25 only (no model to embed with)
    assert call(s, "POST", "/v1/rag/search", {})[0] == 400
    status, out = call(s, "POST", "/v1/rag/search", {"query": "speculative drafts tokens", "top_k": 3})
    assert status == 200 and out["query"] == "speculative drafts tokens" and out["results"]
    assert out["results"][0]["doc_name"] == "spec.md"
    status, out = call(s, "POST", "/v1/rag/search", {"query": "paged cache blocks", "top_k": 1})
    assert len(out["results"]) == 1 and out["results"][0]["doc_name"] == "cache.txt"
    stats = call(s, "GET", "/v1/rag/stats")[1]
    assert stats["documents"] == 2 and stats["chunks"] >= 2 and stats["dense_enabled"] is False
    # replace, then delete
    status, r = call(s, "PUT", f"/v1/rag/document/{a['doc_id']}",
                     {"filename": "cache.txt", "text": "Entirely different words about tokenizers and vocabularies. " * 5})
    assert status == 200
    assert call(s, "PUT", "/v1/rag/document/9999", {"filename": "x.txt", "text": "y"})[0] == 404
    out = call(s, "POST", "/v1/rag/search", {"query": "tokenizers vocabularies", "top_k": 2})[1]
    assert out["results"][0]["doc_name"] == "cache.txt"
    assert call(s, "DELETE", f"/v1/rag/document/{b['doc_id']}") == (200, {"deleted": b["doc_id"]})
    assert call(s, "DELETE", f"/v1/rag/document/{b['doc_id']}")[0] == 404
    assert len(call(s, "GET", "/v1/rag/documents")[1]["documents"]) == 1
    # dense back-fill is for the admin, and has nothing to embed with here
    assert call(s, "POST", "/v1/rag/backfill_dense")[0] == 403
    assert call(s, "POST", "/v1/rag/backfill_dense", headers=ADMIN) == (200, {"embedded": 0})

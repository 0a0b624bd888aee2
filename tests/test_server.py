"""HTTP server end to end on the CPU path: a real socket on an ephemeral port, the tiny random model behind it.
Covers the surface the reference exposes (zse-engine/zse_engine/server/*): OpenAI chat/completions (plain and SSE),
models, health, auth + rate limits, admin keys, LoRA routes, RAG routes, static files, CORS pre-flight."""
import asyncio
import base64
import json
import threading
import time

import pytest

from zse_b200.config import EngineConfig
from zse_b200.engine import ZStreamerEngine
from zse_b200.format import synth
from zse_b200.server.app import ZSEServer

ADMIN = "sk-zse-admin-test"


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("srv")
    model = str(d / "tiny.zse")
    synth.write_random_model(model, synth.shape_config("tiny"), seed=5)
    eng = ZStreamerEngine(model, config=EngineConfig(device="cpu", max_batch_seqs=8, max_seq_len=256, quiet=True))
    srv = ZSEServer(engine=eng, host="127.0.0.1", port=0, admin_key=ADMIN, db_path=str(d / "server.db"),
                    model_name="tiny", quiet=True)
    loop = asyncio.new_event_loop()
    started = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        loop.run_until_complete(srv.start())
        started.set()
        loop.run_forever()

    t = threading.Thread(target=run, daemon=True)
    t.start()
    assert started.wait(30)
    yield srv
    srv.stop()
    loop.call_soon_threadsafe(loop.stop)
    t.join(5)


def http(srv, method, path, body=None, headers=None, raw=False, timeout=60):
    import socket
    data = b"" if body is None else (body if isinstance(body, bytes) else json.dumps(body).encode())
    h = {"Host": "x", "Content-Length": str(len(data)), "Connection": "close"}
    if body is not None:
        h["Content-Type"] = "application/json"
    h.update(headers or {})
    req = f"{method} {path} HTTP/1.1\r\n" + "".join(f"{k}: {v}\r\n" for k, v in h.items()) + "\r\n"
    with socket.create_connection(("127.0.0.1", srv.port), timeout=timeout) as s:
        s.sendall(req.encode() + data)
        buf = b""
        while True:
            chunk = s.recv(65536)
            if not chunk:
                break
            buf += chunk
    head, _, payload = buf.partition(b"\r\n\r\n")
    status = int(head.split(b" ", 2)[1])
    hdrs = {k.strip().lower(): v.strip() for k, v in
            (line.decode().split(":", 1) for line in head.split(b"\r\n")[1:] if b":" in line)}
    if raw:
        return status, hdrs, payload
    return status, hdrs, (json.loads(payload) if payload and hdrs.get("content-type", "").startswith("application/json")
                          else payload)


def test_health_models_static_and_cors(server):
    st, _, body = http(server, "GET", "/health")
    assert st == 200 and body["status"] == "ok" and body["engine"] == "running"
    st, _, body = http(server, "GET", "/v1/models")
    assert st == 200 and body["object"] == "list" and body["data"][0]["id"] == "tiny"
    st, h, page = http(server, "GET", "/", raw=True)
    assert st == 200 and b"<html" in page.lower() and "text/html" in h["content-type"]
    assert http(server, "GET", "/../../etc/passwd", raw=True)[0] in (400, 403, 404)
    st, h, _ = http(server, "OPTIONS", "/v1/chat/completions", raw=True)
    assert st in (200, 204) and "access-control-allow-origin" in h
    assert http(server, "GET", "/v1/nope")[0] == 404


def test_chat_completion_and_usage(server):
    st, _, body = http(server, "POST", "/v1/chat/completions",
                       {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6,
                        "temperature": 0})
    assert st == 200 and body["object"] == "chat.completion"
    ch = body["choices"][0]
    assert ch["message"]["role"] == "assistant" and isinstance(ch["message"]["content"], str)
    assert ch["finish_reason"] in ("length", "stop")
    u = body["usage"]
    assert u["completion_tokens"] <= 6 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    # greedy is deterministic
    again = http(server, "POST", "/v1/chat/completions",
                 {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6,
                  "temperature": 0})[2]
    assert again["choices"][0]["message"]["content"] == ch["message"]["content"]


def test_text_completion_and_validation(server):
    st, _, body = http(server, "POST", "/v1/completions", {"model": "tiny", "prompt": "abc", "max_tokens": 4,
                                                           "temperature": 0})
    assert st == 200 and body["object"] == "text_completion" and "text" in body["choices"][0]
    assert http(server, "POST", "/v1/completions", {"model": "tiny"})[0] == 400
    assert http(server, "POST", "/v1/chat/completions", {"model": "tiny", "messages": []})[0] == 400
    assert http(server, "POST", "/v1/chat/completions", b"{not json")[0] == 400


def test_streaming_chunks(server):
    st, h, payload = http(server, "POST", "/v1/chat/completions",
                          {"model": "tiny", "messages": [{"role": "user", "content": "stream please"}],
                           "max_tokens": 5, "temperature": 0, "stream": True}, raw=True)
    assert st == 200 and h["content-type"].startswith("text/event-stream")
    events = [e[6:] for e in payload.decode().split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop")
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    plain = http(server, "POST", "/v1/chat/completions",
                 {"model": "tiny", "messages": [{"role": "user", "content": "stream please"}], "max_tokens": 5,
                  "temperature": 0})[2]
    assert text == plain["choices"][0]["message"]["content"]


def test_admin_keys_auth_and_rate_limit(server):
    adm = {"Authorization": f"Bearer {ADMIN}"}
    assert http(server, "POST", "/v1/admin/keys/create", {"name": "t"})[0] in (401, 403)
    st, _, made = http(server, "POST", "/v1/admin/keys/create", {"name": "t", "rate_limit_rpm": 2}, adm)
    assert st in (200, 201) and made["key"].startswith("sk-zse-")
    key = {"Authorization": f"Bearer {made['key']}"}
    st, _, keys = http(server, "GET", "/v1/admin/keys/list", headers=adm)
    assert st == 200 and any(k["name"] == "t" for k in keys["keys"])
    assert all("key_hash" not in k for k in keys["keys"])
    body = {"model": "tiny", "prompt": "x", "max_tokens": 2, "temperature": 0}
    assert http(server, "POST", "/v1/completions", body, key)[0] == 200
    assert http(server, "POST", "/v1/completions", body, key)[0] == 200
    st, _, err = http(server, "POST", "/v1/completions", body, key)
    assert st == 429 and "error" in err                       # third request inside the minute
    assert http(server, "POST", "/v1/completions", body, {"Authorization": "Bearer sk-zse-bogus"})[0] == 401
    st, _, stats = http(server, "GET", "/v1/admin/stats", headers=adm)
    assert st == 200 and "engine" in stats
    kid = made.get("id") or next(k["id"] for k in keys["keys"] if k["name"] == "t")
    assert http(server, "POST", "/v1/admin/keys/revoke", {"id": kid}, adm)[0] == 200
    assert http(server, "POST", "/v1/completions", body, key)[0] == 401


def test_lora_routes(server, tmp_path):
    adm = {"Authorization": f"Bearer {ADMIN}"}
    st, _, body = http(server, "GET", "/v1/lora/list")
    assert st == 200 and body["adapters"] == []
    assert http(server, "POST", "/v1/lora/load", {"adapter_id": "a", "path": "/nope"})[0] == 403
    assert http(server, "POST", "/v1/lora/load", {"adapter_id": "a", "path": "/nope"}, adm)[0] == 404
    from zse_b200.lora.weights import random_adapter_file
    path = str(tmp_path / "a.zse-lora")
    random_adapter_file(path, server.engine.model_config, rank=4, alpha=8.0, seed=1)
    st, _, info = http(server, "POST", "/v1/lora/load", {"adapter_id": "a", "path": path}, adm)
    assert st == 201 and info["rank"] == 4
    assert "a" in [x["adapter_id"] if isinstance(x, dict) else x
                   for x in http(server, "GET", "/v1/lora/list")[2]["adapters"]]
    base = http(server, "POST", "/v1/completions", {"model": "tiny", "prompt": "lora", "max_tokens": 6,
                                                    "temperature": 0})[2]["choices"][0]["text"]
    st, _, tuned = http(server, "POST", "/v1/completions", {"model": "tiny:a", "prompt": "lora", "max_tokens": 6,
                                                            "temperature": 0})
    assert st == 200 and isinstance(tuned["choices"][0]["text"], str)
    assert http(server, "POST", "/v1/completions", {"model": "tiny", "prompt": "lora", "max_tokens": 6,
                                                    "temperature": 0, "lora_id": "missing"})[0] in (400, 404)
    assert http(server, "POST", "/v1/lora/unload", {"adapter_id": "a"}, adm)[0] == 200
    after = http(server, "POST", "/v1/completions", {"model": "tiny", "prompt": "lora", "max_tokens": 6,
                                                     "temperature": 0})[2]["choices"][0]["text"]
    assert after == base


def test_rag_routes_and_rag_flag(server):
    text = "The warranty of the Falcon drone lasts twenty four months.\n\nReturns are accepted within thirty days."
    st, _, up = http(server, "POST", "/v1/rag/upload", {"filename": "policy.txt",
                                                        "content": base64.b64encode(text.encode()).decode()})
    assert st == 201 and up["chunk_count"] >= 1
    doc_id = up["doc_id"]
    assert http(server, "POST", "/v1/rag/upload", {"filename": "x.txt", "content": "%%%"})[0] == 400
    assert http(server, "POST", "/v1/rag/upload", {"content": "aGk="})[0] == 400
    st, _, res = http(server, "POST", "/v1/rag/search", {"query": "how long is the drone warranty", "top_k": 2})
    assert st == 200 and res["results"][0]["doc_name"] == "policy.txt"
    assert http(server, "POST", "/v1/rag/search", {})[0] == 400
    st, _, docs = http(server, "GET", "/v1/rag/documents")
    assert st == 200 and [d["name"] for d in docs["documents"]] == ["policy.txt"]
    st, _, doc = http(server, "GET", f"/v1/rag/document/{doc_id}")
    assert st == 200 and doc["chunks"][0]["content"].startswith("The warranty")
    st, _, rep = http(server, "PUT", f"/v1/rag/document/{doc_id}", {"filename": "policy.txt", "text": "New policy text."})
    assert st == 200 and rep["doc_id"] != doc_id
    assert http(server, "GET", f"/v1/rag/document/{doc_id}")[0] == 404
    st, _, stats = http(server, "GET", "/v1/rag/stats")
    assert st == 200 and stats["documents"] == 1
    st, _, body = http(server, "POST", "/v1/chat/completions",
                       {"model": "tiny", "messages": [{"role": "user", "content": "new policy"}], "max_tokens": 3,
                        "temperature": 0, "rag": True})
    assert st == 200 and body["usage"]["prompt_tokens"] > 10      # the retrieved context went into the prompt
    assert http(server, "DELETE", f"/v1/rag/document/{rep['doc_id']}")[0] == 200
    assert http(server, "DELETE", f"/v1/rag/document/{rep['doc_id']}")[0] == 404
    assert http(server, "POST", "/v1/rag/backfill_dense", {})[0] == 403


def test_client_that_goes_away_mid_stream_is_cancelled(server):
    """A streaming client closes its socket after the first chunks: the request must be cancelled (not generated to
    the end for nobody) and its cache blocks returned."""
    import socket
    eng = server._engine
    before = eng.stats().total_tokens_generated
    body = json.dumps({"model": "tiny", "prompt": "go on for a long time", "max_tokens": 230, "stream": True,
                       "temperature": 0}).encode()
    req = (f"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\n"
           f"Content-Length: {len(body)}\r\n\r\n").encode() + body
    s = socket.create_connection(("127.0.0.1", server.port), timeout=30)
    s.sendall(req)
    got = b""
    while got.count(b"data: ") < 2:
        got += s.recv(4096)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_LINGER, __import__("struct").pack("ii", 1, 0))   # close with a reset
    s.close()
    deadline = time.time() + 20
    while time.time() < deadline:
        if eng.scheduler.num_active == 0 and eng.kv_cache.num_sequences == 0:
            break
        time.sleep(0.02)
    assert eng.scheduler.num_active == 0 and eng.kv_cache.num_sequences == 0
    produced = eng.stats().total_tokens_generated - before
    assert produced < 200, produced            # it did not run to its 230 tokens
    status, _, health = http(server, "GET", "/health")
    assert status == 200 and health["status"] == "ok"


def test_chat_template_follows_the_tokenizer():
    from zse_b200.server.api_openai import TEMPLATES, template_for_arch

    class Tok:
        def __init__(self, *tokens):
            self.tokens = set(tokens)

        def token_to_id(self, t):
            return 1 if t in self.tokens else None

    assert template_for_arch("llama") == "llama" and template_for_arch("qwen2") == "chatml"
    assert template_for_arch("llama", Tok("<|start_header_id|>", "<|eot_id|>")) == "llama3"
    assert template_for_arch("llama", Tok("<|im_start|>")) == "chatml"            # a ChatML fine-tune of a Llama
    assert template_for_arch("phi3", Tok("<|assistant|>", "<|end|>")) == "phi3"
    assert template_for_arch("phi3", Tok()) == "chatml" and template_for_arch("gemma2", Tok()) == "gemma"
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    assert TEMPLATES["llama3"](msgs).endswith("hi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    assert TEMPLATES["phi3"](msgs) == "<|system|>\nbe brief<|end|>\n<|user|>\nhi<|end|>\n<|assistant|>\n"

"""OpenAI-compatible inference routes: ``POST /v1/chat/completions``, ``POST /v1/completions``, ``GET /v1/models``
(zse-engine/zse_engine/server/api_openai.py:21-431).

Request fields: ``messages`` / ``prompt``, ``model`` (``"<model>:<adapter>"`` selects a LoRA adapter, as does
``lora_id``), ``temperature`` 1.0, ``top_p`` 0.9, ``top_k`` 50, ``max_tokens`` 128, ``stream``, ``seed``,
``repetition_penalty``, ``rag``.  Chat templates: ChatML (default; Qwen2, Phi), Llama ``[INST]``, Gemma.
Streaming uses SSE fed by the engine thread through ``loop.call_soon_threadsafe``; a request that does not finish
in 120 s answers 504, a full queue 503.  Unlike the reference, finished requests are recorded in the usage table
when the caller authenticated with an API key.
"""
from __future__ import annotations

import asyncio
import secrets
import time
from typing import Dict, List, Optional

from .router import Request, Response
from .sse import SSE_DONE, chat_chunk, completion_chunk

CHAT_MARKERS = ("<|im_end|>", "<|im_start|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "</s>")
REQUEST_TIMEOUT_S = 120.0


def format_chatml(messages: List[Dict]) -> str:
    parts = [f"<|im_start|>{m.get('role', 'user')}\n{m.get('content', '')}<|im_end|>" for m in messages]
    parts.append("<|im_start|>assistant\n")
    return "\n".join(parts)


def format_llama(messages: List[Dict]) -> str:
    out, system = [], ""
    for m in messages:
        role, content = m.get("role", "user"), m.get("content", "")
        if role == "system":
            system = content
        elif role == "user":
            if system:
                out.append(f"[INST] <<SYS>>\n{system}\n<</SYS>>\n\n{content} [/INST]")
                system = ""
            else:
                out.append(f"[INST] {content} [/INST]")
        elif role == "assistant":
            out.append(f" {content} </s>")
    return "".join(out)


def format_gemma(messages: List[Dict]) -> str:
    parts = [f"<start_of_turn>{'model' if m.get('role') == 'assistant' else m.get('role', 'user')}\n"
             f"{m.get('content', '')}<end_of_turn>" for m in messages]
    parts.append("<start_of_turn>model\n")
    return "\n".join(parts)


def format_llama3(messages: List[Dict]) -> str:
    parts = [f"<|start_header_id|>{m.get('role', 'user')}<|end_header_id|>\n\n{m.get('content', '')}<|eot_id|>"
             for m in messages]
    return "".join(parts) + "<|start_header_id|>assistant<|end_header_id|>\n\n"


def format_phi3(messages: List[Dict]) -> str:
    parts = [f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}<|end|>\n" for m in messages]
    return "".join(parts) + "<|assistant|>\n"


TEMPLATES = {"chatml": format_chatml, "llama": format_llama, "llama3": format_llama3, "phi3": format_phi3,
             "gemma": format_gemma}


def template_for_arch(arch: str, tokenizer=None) -> str:
    """The chat layout of a model.  The tokenizer decides when it has one of the layouts' marker tokens (a Llama-3
    file and a Llama-2 file share the architecture name but not the template); otherwise the architecture does."""
    has = (lambda t: tokenizer.token_to_id(t) is not None) if tokenizer is not None else (lambda t: False)
    try:
        if has("<|im_start|>"):
            return "chatml"
        if has("<|start_header_id|>") and has("<|eot_id|>"):
            return "llama3"
        if has("<start_of_turn>"):
            return "gemma"
        if has("<|assistant|>") and has("<|end|>"):
            return "phi3"
    except Exception:
        pass
    a = (arch or "").lower()
    if "llama" in a or "mistral" in a:
        return "llama"
    if "gemma" in a:
        return "gemma"
    return "chatml"


def strip_markers(text: str) -> str:
    for m in CHAT_MARKERS:
        if m in text:
            text = text.split(m)[0]
    return text.rstrip()


class OpenAIAPI:
    def __init__(self, engine, model_name: str = "zse-model", tokenizer=None, db=None, rag_engine=None):
        self._engine = engine
        self._model_name = model_name
        self._tokenizer = tokenizer
        self._db = db
        self._rag_engine = rag_engine
        arch = getattr(getattr(engine, "model_config", None), "arch", "") if engine is not None else ""
        self._chat_template = template_for_arch(arch, tokenizer)
        self._created = int(time.time())

    def set_rag_engine(self, rag_engine) -> None:
        self._rag_engine = rag_engine

    def register(self, router) -> None:
        router.post("/v1/chat/completions", self.handle_chat_completions)
        router.post("/v1/completions", self.handle_completions)
        router.get("/v1/models", self.handle_list_models)

    # ---- helpers ----------------------------------------------------------------------------------------
    def _params(self, body: dict):
        model = str(body.get("model", self._model_name))
        lora_id = body.get("lora_id")
        if lora_id is None and ":" in model:
            lora_id = model.split(":", 1)[1] or None
        try:
            p = dict(temperature=float(body.get("temperature", 1.0)), top_p=float(body.get("top_p", 0.9)),
                     top_k=int(body.get("top_k", 50)), max_tokens=int(body.get("max_tokens", 128)),
                     repetition_penalty=float(body.get("repetition_penalty", 1.0)))
        except (TypeError, ValueError):
            return None, None, None, None
        seed = body.get("seed")
        p["seed"] = int(seed) if seed is not None else None
        p["lora_id"] = lora_id
        return model, p, bool(body.get("stream", False)), lora_id

    def _decode(self, ids: List[int]) -> str:
        if self._tokenizer is not None:
            return strip_markers(self._tokenizer.decode(ids))
        return " ".join(str(t) for t in ids)

    def _record(self, request: Request, model: str, lora_id, rid: str, n_prompt: int, n_out: int, t0: float) -> None:
        key = request.context.get("api_key")
        if self._db is not None and key is not None and getattr(key, "id", 0) > 0:
            self._db.record_usage(key.id, n_prompt, n_out, model, lora_id, rid, (time.monotonic() - t0) * 1000.0)

    async def _generate(self, request: Request, prompt: str, completion_id: str, model: str, params: dict,
                        stream: bool, chat: bool) -> Response:
        if self._engine is None:                 # mock mode (no model loaded): echo service for API tests
            text = "This is a mock response (no model loaded)."
            return self._final(completion_id, model, text, "stop", 0, len(text.split()), chat)
        loop = asyncio.get_running_loop()
        t0 = time.monotonic()
        if stream:
            return await self._stream(request, loop, prompt, completion_id, model, params, chat, t0)
        done = asyncio.Event()
        box: Dict[str, object] = {}

        def on_finish(out):
            box["out"] = out
            loop.call_soon_threadsafe(done.set)

        try:
            rid = self._engine.add_request(prompt=prompt, on_finish=on_finish, **params)
        except ValueError as exc:
            return Response.error(str(exc), 400)
        if rid is None:
            return Response.error("Server is busy (request queue full). Retry later.", 503)
        try:
            await asyncio.wait_for(done.wait(), REQUEST_TIMEOUT_S)
        except asyncio.TimeoutError:
            self._engine.cancel_request(rid)
            return Response.error("Request timed out", 504)
        out = box["out"]
        if out.finish_reason.value == "error":
            return Response.error(out.error or "generation failed", 500)
        text = self._decode(out.output_tokens)
        self._record(request, model, params.get("lora_id"), rid, len(out.prompt_tokens), len(out.output_tokens), t0)
        return self._final(completion_id, model, text, out.finish_reason.value, len(out.prompt_tokens),
                           len(out.output_tokens), chat)

    def _final(self, completion_id, model, text, finish, n_prompt, n_out, chat) -> Response:
        usage = {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}
        if chat:
            choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": finish}
            obj = "chat.completion"
        else:
            choice = {"index": 0, "text": text, "finish_reason": finish}
            obj = "text_completion"
        return Response.json_response({"id": completion_id, "object": obj, "created": int(time.time()), "model": model,
                                       "choices": [choice], "usage": usage})

    async def _stream(self, request, loop, prompt, completion_id, model, params, chat, t0) -> Response:
        q: asyncio.Queue = asyncio.Queue()

        def on_token(tok: int):
            loop.call_soon_threadsafe(q.put_nowait, ("tok", tok))

        def on_finish(out):
            loop.call_soon_threadsafe(q.put_nowait, ("end", out))

        try:
            rid = self._engine.add_request(prompt=prompt, on_token=on_token, on_finish=on_finish, **params)
        except ValueError as exc:
            return Response.error(str(exc), 400)
        if rid is None:
            return Response.error("Server is busy (request queue full). Retry later.", 503)
        stops = set(self._engine.default_stop_tokens()) if hasattr(self._engine, "default_stop_tokens") else set()

        async def gen():
            ids: List[int] = []
            sent = ""
            finished = False
            try:
                if chat:
                    yield chat_chunk(completion_id, model, role="assistant")
                deadline = time.monotonic() + REQUEST_TIMEOUT_S
                while True:
                    try:
                        kind, val = await asyncio.wait_for(q.get(), max(0.1, deadline - time.monotonic()))
                    except asyncio.TimeoutError:
                        break
                    if kind == "tok":
                        if val in stops:
                            continue
                        ids.append(val)
                        text = self._decode(ids)
                        if len(text) > len(sent) and not text.endswith("\ufffd"):
                            piece, sent = text[len(sent):], text
                            yield chat_chunk(completion_id, model, content=piece) if chat else \
                                completion_chunk(completion_id, model, piece)
                    else:
                        out = val
                        finished = True
                        self._record(request, model, params.get("lora_id"), rid, len(out.prompt_tokens),
                                     len(out.output_tokens), t0)
                        # text held back while it ended inside a multi-byte character goes out with the last chunk
                        text = self._decode(ids)
                        if len(text) > len(sent):
                            piece, sent = text[len(sent):], text
                            yield chat_chunk(completion_id, model, content=piece) if chat else \
                                completion_chunk(completion_id, model, piece)
                        fin = out.finish_reason.value
                        yield chat_chunk(completion_id, model, finish_reason=fin) if chat else \
                            completion_chunk(completion_id, model, "", fin)
                        break
                yield SSE_DONE
            finally:
                # the time-out above, or the client went away in the middle of the stream (the connection handler
                # closes this generator): stop generating for nobody
                if not finished:
                    self._engine.cancel_request(rid)

        return Response.sse(gen())

    # ---- routes -----------------------------------------------------------------------------------------
    def _format_chat_messages(self, messages: List[Dict]) -> str:
        """The prompt text for a chat in this model's template (ChatML unless the architecture says otherwise)."""
        return TEMPLATES[self._chat_template](messages)

    async def handle_chat_completions(self, request: Request) -> Response:
        body = request.json
        if not isinstance(body, dict):
            return Response.error("Request body required")
        messages = body.get("messages")
        if not messages or not isinstance(messages, list):
            return Response.error("'messages' field is required and must be a list")
        model, params, stream, _ = self._params(body)
        if params is None:
            return Response.error("invalid sampling parameter")
        if body.get("rag") and self._rag_engine is not None:
            messages = self._rag_engine.augment_messages(messages)
        prompt = self._format_chat_messages(messages)
        return await self._generate(request, prompt, f"chatcmpl-{secrets.token_hex(12)}", model, params, stream, True)

    async def handle_completions(self, request: Request) -> Response:
        body = request.json
        if not isinstance(body, dict):
            return Response.error("Request body required")
        prompt = body.get("prompt")
        if isinstance(prompt, list):
            prompt = prompt[0] if prompt else None
        if not prompt or not isinstance(prompt, str):
            return Response.error("'prompt' field is required")
        model, params, stream, _ = self._params(body)
        if params is None:
            return Response.error("invalid sampling parameter")
        return await self._generate(request, prompt, f"cmpl-{secrets.token_hex(12)}", model, params, stream, False)

    async def handle_list_models(self, request: Request) -> Response:
        entry = lambda mid: {"id": mid, "object": "model", "created": self._created, "owned_by": "zse", "permission": []}
        data = [entry(self._model_name)]
        lm = getattr(self._engine, "lora_manager", None) if self._engine is not None else None
        if lm is not None:
            data += [entry(f"{self._model_name}:{a['adapter_id']}") for a in lm.list_adapters()]
        return Response.json_response({"object": "list", "data": data})

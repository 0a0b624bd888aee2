"""Server-sent-event payloads of the OpenAI streaming protocol (zse-engine/zse_engine/server/sse.py:13-85)."""
from __future__ import annotations

import json
import time
from typing import Optional


def sse_event(obj) -> bytes:
    return b"data: " + json.dumps(obj).encode("utf-8") + b"\n\n"


SSE_DONE = b"data: [DONE]\n\n"


def chat_chunk(completion_id: str, model: str, content: Optional[str] = None, role: Optional[str] = None,
               finish_reason: Optional[str] = None) -> bytes:
    delta = {}
    if role is not None:
        delta["role"] = role
    if content is not None:
        delta["content"] = content
    return sse_event({"id": completion_id, "object": "chat.completion.chunk", "created": int(time.time()),
                      "model": model, "choices": [{"index": 0, "delta": delta, "finish_reason": finish_reason}]})


def completion_chunk(completion_id: str, model: str, text: str = "", finish_reason: Optional[str] = None) -> bytes:
    return sse_event({"id": completion_id, "object": "text_completion", "created": int(time.time()), "model": model,
                      "choices": [{"index": 0, "text": text, "finish_reason": finish_reason}]})


# the reference's names (zse-engine/zse_engine/server/sse.py:18-85)
def sse_done() -> bytes:
    return SSE_DONE


def sse_chat_chunk(completion_id: str, model: str, token_text: str, finish_reason: Optional[str] = None,
                   role: Optional[str] = None) -> bytes:
    return chat_chunk(completion_id, model, token_text if token_text else None, role, finish_reason)


def sse_completion_chunk(completion_id: str, model: str, token_text: str,
                         finish_reason: Optional[str] = None) -> bytes:
    return completion_chunk(completion_id, model, token_text, finish_reason)

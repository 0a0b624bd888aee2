"""SQLite persistence of the server: API keys, usage accounting, chat history
(zse-engine/zse_engine/server/database.py:66-445).  WAL mode, one connection guarded by a lock; keys look like
``sk-zse-<64 hex>`` and only their SHA-256 is stored."""
from __future__ import annotations

import hashlib
import os
import secrets
import sqlite3
import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

SCHEMA = """
CREATE TABLE IF NOT EXISTS api_keys (
    id INTEGER PRIMARY KEY AUTOINCREMENT, key_hash TEXT NOT NULL UNIQUE, key_prefix TEXT NOT NULL,
    name TEXT NOT NULL DEFAULT '', created_at REAL NOT NULL, expires_at REAL, is_active INTEGER NOT NULL DEFAULT 1,
    rate_limit_rpm INTEGER NOT NULL DEFAULT 60, rate_limit_tpm INTEGER NOT NULL DEFAULT 100000,
    allowed_models TEXT NOT NULL DEFAULT '*', total_requests INTEGER NOT NULL DEFAULT 0,
    total_tokens INTEGER NOT NULL DEFAULT 0);
CREATE TABLE IF NOT EXISTS usage (
    id INTEGER PRIMARY KEY AUTOINCREMENT, key_id INTEGER NOT NULL, timestamp REAL NOT NULL,
    prompt_tokens INTEGER NOT NULL DEFAULT 0, completion_tokens INTEGER NOT NULL DEFAULT 0,
    total_tokens INTEGER NOT NULL DEFAULT 0, model TEXT NOT NULL DEFAULT '', lora_id TEXT,
    request_id TEXT NOT NULL DEFAULT '', latency_ms REAL NOT NULL DEFAULT 0);
CREATE INDEX IF NOT EXISTS idx_usage_key_ts ON usage(key_id, timestamp);
CREATE TABLE IF NOT EXISTS chat_history (
    id INTEGER PRIMARY KEY AUTOINCREMENT, key_id INTEGER NOT NULL, session_id TEXT NOT NULL, role TEXT NOT NULL,
    content TEXT NOT NULL, model TEXT NOT NULL DEFAULT '', lora_id TEXT, created_at REAL NOT NULL);
CREATE INDEX IF NOT EXISTS idx_chat_session ON chat_history(session_id, created_at);
CREATE INDEX IF NOT EXISTS idx_chat_key ON chat_history(key_id, created_at);
"""


@dataclass
class APIKey:
    id: int
    key_hash: str
    key_prefix: str
    name: str
    created_at: float
    expires_at: Optional[float]
    is_active: bool
    rate_limit_rpm: int
    rate_limit_tpm: int
    allowed_models: str
    total_requests: int
    total_tokens: int

    def to_public(self) -> dict:
        return {"id": self.id, "prefix": self.key_prefix, "name": self.name, "created_at": self.created_at,
                "expires_at": self.expires_at, "is_active": self.is_active, "rate_limit_rpm": self.rate_limit_rpm,
                "rate_limit_tpm": self.rate_limit_tpm, "allowed_models": self.allowed_models,
                "total_requests": self.total_requests, "total_tokens": self.total_tokens}


@dataclass
class UsageRecord:
    """Token usage of one request (a row of the ``usage`` table; zse-engine/zse_engine/server/database.py:39-50)."""
    id: int
    key_id: int
    timestamp: float
    prompt_tokens: int
    completion_tokens: int
    total_tokens: int
    model: str
    lora_id: Optional[str]
    request_id: str
    latency_ms: float


@dataclass
class ChatMessage:
    id: int
    key_id: int
    session_id: str
    role: str
    content: str
    model: str
    lora_id: Optional[str]
    created_at: float


class ServerDatabase:
    def __init__(self, db_path: str = "~/.zse/server.db"):
        self._path = db_path if db_path == ":memory:" else os.path.expanduser(db_path)
        if self._path != ":memory:":
            os.makedirs(os.path.dirname(self._path) or ".", exist_ok=True)
        self._conn = sqlite3.connect(self._path, check_same_thread=False)
        self._conn.row_factory = sqlite3.Row
        self._lock = threading.Lock()
        with self._lock:
            if self._path != ":memory:":
                self._conn.execute("PRAGMA journal_mode=WAL")
            self._conn.executescript(SCHEMA)
            self._conn.commit()

    # ---- keys -------------------------------------------------------------------------------------------
    @staticmethod
    def hash_key(key: str) -> str:
        return hashlib.sha256(key.encode("utf-8")).hexdigest()

    @staticmethod
    def generate_key() -> str:
        return "sk-zse-" + secrets.token_hex(32)

    def create_key(self, name: str = "", rate_limit_rpm: int = 60, rate_limit_tpm: int = 100000,
                   allowed_models: str = "*", expires_in_days: Optional[float] = None) -> Tuple[str, APIKey]:
        key = self.generate_key()
        now = time.time()
        exp = now + expires_in_days * 86400 if expires_in_days else None
        with self._lock:
            cur = self._conn.execute(
                "INSERT INTO api_keys (key_hash, key_prefix, name, created_at, expires_at, rate_limit_rpm, "
                "rate_limit_tpm, allowed_models) VALUES (?,?,?,?,?,?,?,?)",
                (self.hash_key(key), key[:14], name, now, exp, rate_limit_rpm, rate_limit_tpm, allowed_models))
            self._conn.commit()
            row = self._conn.execute("SELECT * FROM api_keys WHERE id=?", (cur.lastrowid,)).fetchone()
        return key, self._key(row)

    def validate_key(self, key: str) -> Optional[APIKey]:
        with self._lock:
            row = self._conn.execute("SELECT * FROM api_keys WHERE key_hash=?", (self.hash_key(key),)).fetchone()
        if row is None:
            return None
        k = self._key(row)
        if not k.is_active or (k.expires_at is not None and k.expires_at < time.time()):
            return None
        return k

    def list_keys(self) -> List[APIKey]:
        with self._lock:
            return [self._key(r) for r in self._conn.execute("SELECT * FROM api_keys ORDER BY id")]

    def revoke_key(self, key_id: int) -> bool:
        with self._lock:
            cur = self._conn.execute("UPDATE api_keys SET is_active=0 WHERE id=? AND is_active=1", (key_id,))
            self._conn.commit()
            return cur.rowcount > 0

    def revoke_key_by_prefix(self, prefix: str) -> bool:
        with self._lock:
            cur = self._conn.execute("UPDATE api_keys SET is_active=0 WHERE key_prefix LIKE ? AND is_active=1",
                                     (prefix + "%",))
            self._conn.commit()
            return cur.rowcount > 0

    def update_key_limits(self, key_id: int, rate_limit_rpm: Optional[int] = None,
                          rate_limit_tpm: Optional[int] = None, allowed_models: Optional[str] = None) -> bool:
        sets, vals = [], []
        for col, v in (("rate_limit_rpm", rate_limit_rpm), ("rate_limit_tpm", rate_limit_tpm),
                       ("allowed_models", allowed_models)):
            if v is not None:
                sets.append(f"{col}=?")
                vals.append(v)
        if not sets:
            return False
        with self._lock:
            cur = self._conn.execute(f"UPDATE api_keys SET {', '.join(sets)} WHERE id=?", (*vals, key_id))
            self._conn.commit()
            return cur.rowcount > 0

    @staticmethod
    def _key(r) -> APIKey:
        return APIKey(r["id"], r["key_hash"], r["key_prefix"], r["name"], r["created_at"], r["expires_at"],
                      bool(r["is_active"]), r["rate_limit_rpm"], r["rate_limit_tpm"], r["allowed_models"],
                      r["total_requests"], r["total_tokens"])

    # ---- usage ------------------------------------------------------------------------------------------
    def record_usage(self, key_id: int, prompt_tokens: int, completion_tokens: int, model: str = "",
                     lora_id: Optional[str] = None, request_id: str = "", latency_ms: float = 0.0) -> None:
        total = prompt_tokens + completion_tokens
        with self._lock:
            self._conn.execute(
                "INSERT INTO usage (key_id, timestamp, prompt_tokens, completion_tokens, total_tokens, model, lora_id, "
                "request_id, latency_ms) VALUES (?,?,?,?,?,?,?,?,?)",
                (key_id, time.time(), prompt_tokens, completion_tokens, total, model, lora_id, request_id, latency_ms))
            self._conn.execute("UPDATE api_keys SET total_requests=total_requests+1, total_tokens=total_tokens+? "
                               "WHERE id=?", (total, key_id))
            self._conn.commit()

    def get_usage_window(self, key_id: int, window_seconds: float = 60.0) -> Tuple[int, int]:
        with self._lock:
            r = self._conn.execute("SELECT COUNT(*) AS n, COALESCE(SUM(total_tokens),0) AS t FROM usage WHERE key_id=? "
                                   "AND timestamp>=?", (key_id, time.time() - window_seconds)).fetchone()
        return int(r["n"]), int(r["t"])

    def get_usage_stats(self, key_id: Optional[int] = None) -> Dict:
        where, args = ("WHERE key_id=?", (key_id,)) if key_id is not None else ("", ())
        with self._lock:
            r = self._conn.execute(
                f"SELECT COUNT(*) AS n, COALESCE(SUM(prompt_tokens),0) AS p, COALESCE(SUM(completion_tokens),0) AS c, "
                f"COALESCE(SUM(total_tokens),0) AS t, COALESCE(AVG(latency_ms),0) AS l FROM usage {where}",
                args).fetchone()
        return {"total_requests": int(r["n"]), "prompt_tokens": int(r["p"]), "completion_tokens": int(r["c"]),
                "total_tokens": int(r["t"]), "avg_latency_ms": float(r["l"])}

    def recent_usage(self, key_id: Optional[int] = None, limit: int = 100) -> List[UsageRecord]:
        """The latest usage rows, newest first."""
        where, args = ("WHERE key_id=?", (key_id,)) if key_id is not None else ("", ())
        with self._lock:
            rows = self._conn.execute(f"SELECT * FROM usage {where} ORDER BY id DESC LIMIT ?",
                                      args + (int(limit),)).fetchall()
        return [UsageRecord(r["id"], r["key_id"], r["timestamp"], r["prompt_tokens"], r["completion_tokens"],
                            r["total_tokens"], r["model"], r["lora_id"], r["request_id"], r["latency_ms"])
                for r in rows]

    def cleanup_old_usage(self, days: int = 30) -> int:
        with self._lock:
            cur = self._conn.execute("DELETE FROM usage WHERE timestamp<?", (time.time() - days * 86400,))
            self._conn.commit()
            return cur.rowcount

    # ---- chat history -----------------------------------------------------------------------------------
    def save_message(self, key_id: int, session_id: str, role: str, content: str, model: str = "",
                     lora_id: Optional[str] = None) -> int:
        with self._lock:
            cur = self._conn.execute("INSERT INTO chat_history (key_id, session_id, role, content, model, lora_id, "
                                     "created_at) VALUES (?,?,?,?,?,?,?)",
                                     (key_id, session_id, role, content, model, lora_id, time.time()))
            self._conn.commit()
            return cur.lastrowid

    def get_session_messages(self, session_id: str, limit: int = 1000) -> List[ChatMessage]:
        with self._lock:
            rows = self._conn.execute("SELECT * FROM chat_history WHERE session_id=? ORDER BY created_at, id LIMIT ?",
                                      (session_id, limit)).fetchall()
        return [ChatMessage(r["id"], r["key_id"], r["session_id"], r["role"], r["content"], r["model"], r["lora_id"],
                            r["created_at"]) for r in rows]

    def list_sessions(self, key_id: Optional[int] = None, limit: int = 100) -> List[dict]:
        where, args = ("WHERE key_id=?", (key_id,)) if key_id is not None else ("", ())
        with self._lock:
            rows = self._conn.execute(
                f"SELECT session_id, COUNT(*) AS n, MIN(created_at) AS first, MAX(created_at) AS last FROM chat_history "
                f"{where} GROUP BY session_id ORDER BY last DESC LIMIT ?", (*args, limit)).fetchall()
        return [{"session_id": r["session_id"], "messages": r["n"], "created_at": r["first"], "updated_at": r["last"]}
                for r in rows]

    def delete_session(self, session_id: str) -> int:
        with self._lock:
            cur = self._conn.execute("DELETE FROM chat_history WHERE session_id=?", (session_id,))
            self._conn.commit()
            return cur.rowcount

    def close(self) -> None:
        with self._lock:
            if self._conn is not None:
                self._conn.close()
                self._conn = None

"""Bearer-key authentication, sliding-window rate limits and per-key model allow-lists
(zse-engine/zse_engine/server/auth.py:23-165).  The admin key bypasses limits."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .database import APIKey, ServerDatabase

ADMIN = APIKey(0, "", "admin", "admin", 0.0, None, True, 0, 0, "*", 0, 0)


@dataclass
class AuthResult:
    authenticated: bool
    key: Optional[APIKey] = None
    error: Optional[str] = None
    status_code: int = 200


class AuthManager:
    def __init__(self, db: ServerDatabase, admin_key: Optional[str] = None):
        self._db, self._admin_key = db, admin_key

    @staticmethod
    def _token(authorization: Optional[str]) -> Optional[str]:
        if not authorization:
            return None
        scheme, _, tok = authorization.partition(" ")
        return tok.strip() if scheme == "Bearer" and tok.strip() else None

    def authenticate(self, authorization: Optional[str]) -> AuthResult:
        if not authorization:
            return AuthResult(False, error="Missing Authorization header", status_code=401)
        tok = self._token(authorization)
        if tok is None:
            return AuthResult(False, error="Invalid Authorization format. Use: Bearer <key>", status_code=401)
        if self._admin_key and tok == self._admin_key:
            return AuthResult(True, ADMIN)
        key = self._db.validate_key(tok)
        if key is None:
            return AuthResult(False, error="Invalid or expired API key", status_code=401)
        return AuthResult(True, key)

    def check_rate_limit(self, key: APIKey) -> AuthResult:
        if key.id == 0 or (key.rate_limit_rpm == 0 and key.rate_limit_tpm == 0):
            return AuthResult(True, key)
        reqs, toks = self._db.get_usage_window(key.id, 60)
        if key.rate_limit_rpm > 0 and reqs >= key.rate_limit_rpm:
            return AuthResult(False, key, f"Rate limit exceeded: {reqs}/{key.rate_limit_rpm} requests/min", 429)
        if key.rate_limit_tpm > 0 and toks >= key.rate_limit_tpm:
            return AuthResult(False, key, f"Token limit exceeded: {toks}/{key.rate_limit_tpm} tokens/min", 429)
        return AuthResult(True, key)

    def check_model_access(self, key: APIKey, model: str) -> AuthResult:
        if key.allowed_models == "*":
            return AuthResult(True, key)
        allowed = [m.strip() for m in key.allowed_models.split(",")]
        if model in allowed or model.split(":")[0] in allowed:
            return AuthResult(True, key)
        return AuthResult(False, key, f"Model '{model}' not allowed for this key. Allowed: {key.allowed_models}", 403)

    def is_admin(self, authorization: Optional[str]) -> bool:
        tok = self._token(authorization)
        return bool(self._admin_key) and tok == self._admin_key

    def full_auth_check(self, authorization: Optional[str], model: str = "") -> AuthResult:
        res = self.authenticate(authorization)
        if not res.authenticated:
            return res
        res = self.check_rate_limit(res.key)
        if not res.authenticated:
            return res
        return self.check_model_access(res.key, model) if model else res

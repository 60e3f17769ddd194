"""User store with PBKDF2 password hashes, signed session tokens and lock-out after failed log-ins
(reference ``security/auth.py:33-70``).  Tokens are HMAC-SHA256 signed JSON (JWT-compatible layout) so PyJWT is not needed."""
from __future__ import annotations

import base64
import hashlib
import hmac
import json
import os
import secrets
import time
from typing import Dict, Optional


def _b64(b: bytes) -> str:
    return base64.urlsafe_b64encode(b).rstrip(b"=").decode()


def _unb64(s: str) -> bytes:
    return base64.urlsafe_b64decode(s + "=" * (-len(s) % 4))


class AuthManager:
    def __init__(self, secret: Optional[str] = None, max_attempts: int = 5, lockout_s: int = 900, session_s: int = 3600,
                 iterations: int = 120_000):
        self.secret = (secret or os.environ.get("ATS_AUTH_SECRET") or secrets.token_hex(32)).encode()
        self.users: Dict[str, Dict[str, object]] = {}
        self.max_attempts, self.lockout_s, self.session_s, self.iterations = max_attempts, lockout_s, session_s, iterations
        self.revoked: set = set()

    def _hash(self, password: str, salt: bytes) -> bytes:
        return hashlib.pbkdf2_hmac("sha256", password.encode(), salt, self.iterations)

    def create_user(self, username: str, password: str, role: str = "user") -> None:
        if username in self.users:
            raise ValueError("user exists")
        if len(password) < 8:
            raise ValueError("password must have at least 8 characters")
        salt = secrets.token_bytes(16)
        self.users[username] = {"salt": salt, "hash": self._hash(password, salt), "role": role, "failed": 0, "locked_until": 0.0}

    def authenticate(self, username: str, password: str) -> Optional[str]:
        u = self.users.get(username)
        now = time.time()
        if u is None:
            self._hash(password, b"0" * 16)  # same work for unknown users
            return None
        if now < u["locked_until"]:
            return None
        if hmac.compare_digest(self._hash(password, u["salt"]), u["hash"]):
            u["failed"] = 0
            return self._issue(username, u["role"])
        u["failed"] += 1
        if u["failed"] >= self.max_attempts:
            u["locked_until"] = now + self.lockout_s
            u["failed"] = 0
        return None

    def _issue(self, username: str, role: str) -> str:
        head = _b64(json.dumps({"alg": "HS256", "typ": "JWT"}).encode())
        body = _b64(json.dumps({"sub": username, "role": role, "exp": time.time() + self.session_s, "jti": secrets.token_hex(8)}).encode())
        sig = _b64(hmac.new(self.secret, f"{head}.{body}".encode(), hashlib.sha256).digest())
        return f"{head}.{body}.{sig}"

    def verify(self, token: str) -> Optional[Dict[str, object]]:
        try:
            head, body, sig = token.split(".")
            good = _b64(hmac.new(self.secret, f"{head}.{body}".encode(), hashlib.sha256).digest())
            if not hmac.compare_digest(sig, good):
                return None
            claims = json.loads(_unb64(body))
            if claims["exp"] < time.time() or claims["jti"] in self.revoked:
                return None
            return claims
        except Exception:
            return None

    def logout(self, token: str) -> None:
        c = self.verify(token)
        if c:
            self.revoked.add(c["jti"])

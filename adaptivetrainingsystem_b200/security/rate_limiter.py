"""Sliding-window rate limiter and the secured chat wrapper (reference ``security/rate_limiter.py:8-45, 107-247``)."""
from __future__ import annotations

import threading
import time
from collections import defaultdict, deque
from typing import Callable, Deque, Dict, Optional, Tuple

from .auth import AuthManager
from .input_validator import InputValidator


class RateLimiter:
    def __init__(self, max_requests: int = 30, window_s: float = 60.0, clock: Callable[[], float] = time.monotonic):
        self.max_requests, self.window_s, self.clock = max_requests, window_s, clock
        self._hits: Dict[str, Deque[float]] = defaultdict(deque)
        self._lock = threading.Lock()

    def allow(self, key: str) -> Tuple[bool, float]:
        """-> (allowed, seconds until the next slot frees up)."""
        now = self.clock()
        with self._lock:
            q = self._hits[key]
            while q and now - q[0] >= self.window_s:
                q.popleft()
            if len(q) < self.max_requests:
                q.append(now)
                return True, 0.0
            return False, self.window_s - (now - q[0])

    def remaining(self, key: str) -> int:
        now = self.clock()
        with self._lock:
            q = self._hits[key]
            return self.max_requests - sum(1 for t in q if now - t < self.window_s)


class SecureConversationalChat:
    """Authenticated, validated and rate-limited front door of a generation callable ``generate(prompt) -> str``."""

    def __init__(self, generate: Callable[[str], str], auth: Optional[AuthManager] = None,
                 validator: Optional[InputValidator] = None, limiter: Optional[RateLimiter] = None):
        self.generate = generate
        self.auth = auth or AuthManager()
        self.validator = validator or InputValidator()
        self.limiter = limiter or RateLimiter()

    def login(self, username: str, password: str) -> Optional[str]:
        return self.auth.authenticate(username, password)

    def chat(self, token: str, prompt: str) -> Dict[str, object]:
        claims = self.auth.verify(token)
        if claims is None:
            return {"ok": False, "error": "not authenticated"}
        ok, wait = self.limiter.allow(str(claims["sub"]))
        if not ok:
            return {"ok": False, "error": "rate limited", "retry_after_s": wait}
        valid, problems = self.validator.validate(prompt)
        if not valid:
            return {"ok": False, "error": "invalid input", "problems": problems}
        return {"ok": True, "response": self.generate(self.validator.sanitize(prompt))}

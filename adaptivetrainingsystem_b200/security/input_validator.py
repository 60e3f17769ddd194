"""Prompt validation for the chat front end: length limits, control characters, injection / script patterns
(reference ``security/input_validator.py:17-45``)."""
from __future__ import annotations

import re
from typing import List, Tuple

PATTERNS = [r"<\s*script", r"javascript\s*:", r"on\w+\s*=\s*[\"']", r"\{\{.*\}\}", r"\$\{.*\}", r";\s*(rm|del|drop)\s", r"\.\./\.\./",
            r"<\|im_(start|end)\|>", r"\x00"]


class InputValidator:
    def __init__(self, max_length: int = 8192, max_line_length: int = 4096):
        self.max_length, self.max_line_length = max_length, max_line_length
        self._rx = [re.compile(p, re.IGNORECASE | re.DOTALL) for p in PATTERNS]

    def validate(self, text: str) -> Tuple[bool, List[str]]:
        problems: List[str] = []
        if not isinstance(text, str) or not text.strip():
            return False, ["empty input"]
        if len(text) > self.max_length:
            problems.append(f"input longer than {self.max_length} characters")
        if any(len(l) > self.max_line_length for l in text.splitlines()):
            problems.append("line too long")
        if sum(1 for c in text if ord(c) < 32 and c not in "\n\r\t") > 0:
            problems.append("control characters")
        for rx in self._rx:
            if rx.search(text):
                problems.append(f"blocked pattern {rx.pattern!r}")
        return not problems, problems

    def sanitize(self, text: str) -> str:
        text = "".join(c for c in text if ord(c) >= 32 or c in "\n\r\t")
        text = re.sub(r"<\|im_(start|end)\|>", "", text)
        return text[: self.max_length]

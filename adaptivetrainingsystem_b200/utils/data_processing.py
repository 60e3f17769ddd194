"""Data helpers: OASST tree -> conversation JSONL conversion and dataset validation statistics
(reference ``utils/data_processing.py``; ``Dataset_download.py`` message-tree extraction)."""
from __future__ import annotations

import json
import os
from collections import Counter, defaultdict
from typing import Any, Dict, Iterable, List, Optional


def oasst_trees_to_conversations(messages: Iterable[Dict[str, Any]], lang: Optional[str] = "en") -> List[Dict[str, Any]]:
    """Flat OASST1 message rows (message_id, parent_id, role, text, lang, rank) -> one conversation per root-to-leaf path
    following the best-ranked reply at every level."""
    by_parent: Dict[Optional[str], List[Dict[str, Any]]] = defaultdict(list)
    for m in messages:
        if lang is None or m.get("lang", lang) == lang:
            by_parent[m.get("parent_id")].append(m)
    out = []
    for root in by_parent[None]:
        conv, node = [], root
        while node is not None:
            conv.append({"role": "user" if node.get("role") == "prompter" else "assistant", "content": node.get("text", "")})
            kids = sorted(by_parent.get(node["message_id"], []), key=lambda k: (k.get("rank") is None, k.get("rank") or 0))
            node = kids[0] if kids else None
        if len(conv) >= 2:
            out.append({"messages": conv})
    return out


def write_jsonl(rows: Iterable[Dict[str, Any]], path: str) -> int:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    n = 0
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n


def validate_data_comprehensive(path: str, tokenizer=None, max_lines: int = 100000) -> Dict[str, Any]:
    stats: Dict[str, Any] = {"path": path, "exists": os.path.exists(path), "lines": 0, "valid": 0, "invalid": 0,
                             "roles": Counter(), "turns": Counter(), "tokens": 0}
    if not stats["exists"]:
        return stats
    with open(path, errors="ignore") as f:
        for i, line in enumerate(f):
            if i >= max_lines:
                break
            line = line.strip()
            if not line:
                continue
            stats["lines"] += 1
            try:
                obj = json.loads(line)
                msgs = obj.get("messages")
                if isinstance(msgs, list) and msgs and all(isinstance(m.get("content"), str) for m in msgs):
                    stats["valid"] += 1
                    stats["turns"][len(msgs)] += 1
                    for m in msgs:
                        stats["roles"][m.get("role", "?")] += 1
                        if tokenizer is not None:
                            stats["tokens"] += len(tokenizer.encode(m["content"]))
                elif isinstance(obj.get("text"), str):
                    stats["valid"] += 1
                else:
                    stats["invalid"] += 1
            except Exception:
                stats["invalid"] += 1
    stats["roles"], stats["turns"] = dict(stats["roles"]), dict(stats["turns"])
    return stats


def validate_data_paths(paths: Iterable[str]) -> Dict[str, bool]:
    return {p: os.path.exists(p) for p in paths}

"""Readers and writers for the corpus file formats of the data-acquisition scripts (no network access here).

The reference downloads OpenAssistant trees and scrapes Wikipedia / Gutenberg / arXiv / StackOverflow / PubMed / Reddit /
PhilPapers / CC-News into plain-text files (reference ``Dataset_download.py:1-560``, ``multi_source_dataset.py:1-1551``).
What the rest of the framework needs from those scripts is their OUTPUT formats, so that files produced elsewhere load here:

* conversations: JSON lines ``{"conversation_id", "messages": [{"role", "content"}, ...]}``;
* base-training text: UTF-8 ``.txt`` with documents separated by a line that holds only ``<|endoftext|>`` (or blank-line
  separated paragraphs when no separator line is present), optionally with a ``# source: <name>`` header line per document.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, Iterator, List, Optional

from ..utils.data_processing import oasst_trees_to_conversations, write_jsonl

DOC_SEPARATOR = "<|endoftext|>"
KNOWN_SOURCES = ("wikipedia", "gutenberg", "arxiv", "stackoverflow", "pubmed", "reddit", "philpapers", "ccnews")


def iter_text_documents(path: str) -> Iterator[Dict[str, str]]:
    """Yield ``{"source", "text"}`` for every document of a scraped ``.txt`` corpus file."""
    default_source = os.path.splitext(os.path.basename(path))[0].lower()
    source, buf = default_source, []
    saw_separator = False

    def flush():
        text = "\n".join(buf).strip()
        buf.clear()
        return {"source": source, "text": text} if text else None
    with open(path, "r", encoding="utf-8", errors="replace") as f:
        for line in f:
            line = line.rstrip("\n")
            if line.strip() == DOC_SEPARATOR:
                saw_separator = True
                d = flush()
                if d:
                    yield d
                source = default_source
            elif line.startswith("# source:") and not buf:
                source = line.split(":", 1)[1].strip().lower() or default_source
            elif not line.strip() and not saw_separator and buf and not buf[-1].strip():
                d = flush()  # two blank lines: paragraph-separated file without separator lines
                if d:
                    yield d
            else:
                buf.append(line)
    d = flush()
    if d:
        yield d


def write_text_corpus(docs: Iterable[Dict[str, str]], path: str) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for d in docs:
            if d.get("source"):
                f.write(f"# source: {d['source']}\n")
            f.write(d["text"].strip() + "\n" + DOC_SEPARATOR + "\n")
            n += 1
    return n


def iter_conversations(path: str) -> Iterator[Dict[str, Any]]:
    """JSON-lines conversations; lines that are not valid conversations are skipped."""
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                continue
            msgs = row.get("messages")
            if isinstance(msgs, list) and msgs and all(isinstance(m, dict) and "role" in m and "content" in m for m in msgs):
                yield row


def convert_oasst_export(messages_path: str, out_path: str, lang: Optional[str] = "en") -> int:
    """OpenAssistant message export (JSON lines, one message per line with ``message_id`` / ``parent_id``) ->
    conversation JSON lines."""
    rows: List[Dict[str, Any]] = []
    with open(messages_path, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    return write_jsonl(oasst_trees_to_conversations(rows, lang=lang), out_path)


def corpus_statistics(paths: Iterable[str]) -> Dict[str, Dict[str, int]]:
    """Documents and characters per source over a list of corpus files."""
    stats: Dict[str, Dict[str, int]] = {}
    for p in paths:
        for d in iter_text_documents(p):
            s = stats.setdefault(d["source"], {"documents": 0, "characters": 0})
            s["documents"] += 1
            s["characters"] += len(d["text"])
    return stats

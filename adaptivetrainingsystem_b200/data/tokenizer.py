"""Conversation tokenizer: a BPE/byte base vocabulary plus role and control tokens, ChatML-style message framing,
truncation strategies and threaded batch encoding.

Interface of the reference (``core/tokenizer.py``): 13 special tokens appended after the base vocabulary (``:76-90``),
vocabulary padded to a multiple of 128 (``:99-101``), ``pad_token_id`` (``:96``), message framing
``<|im_start|><|role|>content<|im_end|>`` (``:305-355``), truncation strategies (``:392-414``), ``encode_batch`` with
threads (``:492-523``).  The reference needs tiktoken's ``cl100k_base`` file from the network on first use; here the
base encoder is pluggable: tiktoken when its cache is present, otherwise a self-contained byte-level encoder (256 byte
tokens), so the framework works offline.  The pad id is a dedicated special token, not 0 (id 0 is a real token).
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence

SPECIAL_TOKENS = ["<|pad|>", "<|im_start|>", "<|im_end|>", "<|system|>", "<|user|>", "<|assistant|>", "<|tool|>",
                  "<|bos|>", "<|eos|>", "<|unk|>", "<|sep|>", "<|mask|>", "<|endoftext|>"]
ROLE_ALIASES = {"prompter": "user", "human": "user", "bot": "assistant", "gpt": "assistant"}


class ByteEncoder:
    """256 byte tokens; lossless for any UTF-8 text."""
    n_vocab = 256
    name = "bytes"

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: Iterable[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


def _load_tiktoken(name: str):
    try:
        import tiktoken
        enc = tiktoken.get_encoding(name)  # raises offline when the vocabulary file is not cached

        class _TT:
            n_vocab = enc.n_vocab

            def __init__(self):
                self.name = name

            def encode(self, text):
                return enc.encode(text, disallowed_special=())

            def decode(self, ids):
                return enc.decode([i for i in ids if i < enc.n_vocab])
        return _TT()
    except Exception:
        return None


class ConversationTokenizer:
    def __init__(self, model_name: str = "cl100k_base", base=None, allow_fallback: bool = True):
        self.tokenizer = base or _load_tiktoken(model_name)
        if self.tokenizer is None:
            if not allow_fallback:
                raise RuntimeError(f"tokenizer {model_name!r} is not available offline")
            self.tokenizer = ByteEncoder()
        self.base_vocab_size = int(self.tokenizer.n_vocab)
        self.special_tokens: Dict[str, int] = {t: self.base_vocab_size + i for i, t in enumerate(SPECIAL_TOKENS)}
        self._special_by_id = {v: k for k, v in self.special_tokens.items()}
        raw = self.base_vocab_size + len(SPECIAL_TOKENS)
        self.vocab_size = (raw + 127) // 128 * 128
        self.pad_token_id = self.special_tokens["<|pad|>"]
        self.eos_token_id = self.special_tokens["<|eos|>"]
        self.bos_token_id = self.special_tokens["<|bos|>"]

    # -- basic ------------------------------------------------------------------------------------------------
    def get_role_token(self, role: str) -> int:
        role = ROLE_ALIASES.get(role, role)
        return self.special_tokens.get(f"<|{role}|>", self.special_tokens["<|user|>"])

    def encode(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text))

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        out, run = [], []
        for i in ids:
            i = int(i)
            if i in self._special_by_id:
                if run:
                    out.append(self.tokenizer.decode(run))
                    run = []
                if not skip_special_tokens:
                    out.append(self._special_by_id[i])
            elif i < self.base_vocab_size:
                run.append(i)
        if run:
            out.append(self.tokenizer.decode(run))
        return "".join(out)

    # -- conversations ------------------------------------------------------------------------------------------
    def encode_message(self, role: str, content: str) -> List[int]:
        st = self.special_tokens
        return [st["<|im_start|>"], self.get_role_token(role)] + self.encode(content.strip()) + [st["<|im_end|>"]]

    def encode_conversation(self, messages: Sequence[Dict[str, str]], max_length: Optional[int] = None,
                            truncation: str = "right", add_generation_prompt: bool = False) -> Dict[str, List]:
        """-> {input_ids, roles (per token), attention_mask}.  Truncation: right | left | middle | keep_system."""
        ids: List[int] = []
        roles: List[str] = []
        spans = []
        for m in messages:
            toks = self.encode_message(m["role"], m["content"])
            spans.append((ROLE_ALIASES.get(m["role"], m["role"]), len(ids), len(ids) + len(toks)))
            ids.extend(toks)
            roles.extend([ROLE_ALIASES.get(m["role"], m["role"])] * len(toks))
        if add_generation_prompt:
            ids.extend([self.special_tokens["<|im_start|>"], self.get_role_token("assistant")])
            roles.extend(["assistant"] * 2)
        if max_length is not None and len(ids) > max_length:
            ids, roles = self._truncate(ids, roles, spans, max_length, truncation)
        return {"input_ids": ids, "roles": roles, "attention_mask": [1] * len(ids)}

    @staticmethod
    def _truncate(ids, roles, spans, n, how):
        if how == "left":
            return ids[-n:], roles[-n:]
        if how == "middle":
            a = n // 2
            return ids[:a] + ids[-(n - a):], roles[:a] + roles[-(n - a):]
        if how == "keep_system" and spans and spans[0][0] == "system" and spans[0][2] < n:
            s_end = spans[0][2]
            return ids[:s_end] + ids[-(n - s_end):], roles[:s_end] + roles[-(n - s_end):]
        return ids[:n], roles[:n]

    def encode_batch(self, texts: Sequence[str], num_threads: int = 8) -> List[List[int]]:
        if len(texts) < 32 or num_threads <= 1:
            return [self.encode(t) for t in texts]
        with ThreadPoolExecutor(max_workers=num_threads) as ex:
            return list(ex.map(self.encode, texts))

    def get_vocab_size(self) -> int:
        return self.vocab_size

    def info(self) -> Dict[str, object]:
        return {"base": getattr(self.tokenizer, "name", "custom"), "base_vocab_size": self.base_vocab_size,
                "vocab_size": self.vocab_size, "special_tokens": dict(self.special_tokens)}

"""Datasets and loaders with the reference batch schema ``{input_ids, labels, attention_mask, loss_weights}``
(reference ``core/dataset.py:216-231, 503-508``): labels are the ids shifted left by one, so the trainer never shifts.

* :class:`SyntheticTokenDataset` -- uniform random ids from a seed (the benchmark workload);
* :class:`BaseTrainingDataset` -- ``.txt`` / ``{"text": ...}`` JSONL packed into ``seq_length + 1`` chunks
  (reference ``dataset.py:118-206``);
* :class:`ConversationDataset` -- ``{"messages": [{role, content}...]}`` JSONL, right-truncated / padded, role-aware
  ``loss_weights`` with ``assistant_loss_weight`` (reference ``dataset.py:388-556``);
* :class:`HybridDatasetManager` -- ``base_only | finetuning_only | hybrid | interleaved`` (reference ``dataset.py:619-752``);
  several files are really concatenated (the reference keeps only the first).
"""
from __future__ import annotations

import json
import os
import random
from typing import Any, Dict, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import ConcatDataset, DataLoader, Dataset, DistributedSampler

IGNORE_INDEX = -100


def _make_item(ids: torch.Tensor, weights: Optional[torch.Tensor] = None, pad_mask: Optional[torch.Tensor] = None):
    """ids has seq_length + 1 entries."""
    inp, lab = ids[:-1].clone(), ids[1:].clone()
    mask = torch.ones_like(inp, dtype=torch.float32) if pad_mask is None else pad_mask[:-1].float()
    w = torch.ones_like(inp, dtype=torch.float32) if weights is None else weights[1:].float()
    if pad_mask is not None:
        lab = torch.where(pad_mask[1:].bool(), lab, torch.full_like(lab, IGNORE_INDEX))
        w = w * pad_mask[1:].float()
    return {"input_ids": inp, "labels": lab, "attention_mask": mask, "loss_weights": w}


class SyntheticTokenDataset(Dataset):
    """Token ids uniform in [0, vocab) drawn from ``seed``; item i is reproducible on its own."""

    def __init__(self, vocab_size: int, seq_length: int, num_samples: int = 1024, seed: int = 0):
        self.vocab_size, self.seq_length, self.num_samples, self.seed = vocab_size, seq_length, num_samples, seed

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, i: int):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.randint(0, self.vocab_size, (self.seq_length + 1,), generator=g)
        return _make_item(ids)

    def total_tokens(self) -> int:
        return self.num_samples * self.seq_length


class BaseTrainingDataset(Dataset):
    def __init__(self, paths: Sequence[str], tokenizer, seq_length: int, max_chunks: Optional[int] = None):
        self.seq_length = seq_length
        stream: List[int] = []
        eos = getattr(tokenizer, "eos_token_id", None)
        for p in paths:
            for text in _iter_texts(p):
                stream.extend(_encode(tokenizer, text))
                if eos is not None:
                    stream.append(eos)
        n = len(stream) // (seq_length + 1)
        if max_chunks:
            n = min(n, max_chunks)
        self.chunks = torch.tensor(stream[: n * (seq_length + 1)], dtype=torch.long).view(n, seq_length + 1)

    def __len__(self) -> int:
        return self.chunks.shape[0]

    def __getitem__(self, i: int):
        return _make_item(self.chunks[i])

    def total_tokens(self) -> int:
        return self.chunks.numel()


class StreamingBaseTrainingDataset(torch.utils.data.IterableDataset):
    """Same packing, produced lazily for files above ``streaming_threshold_gb`` (reference ``dataset.py:241-330``)."""

    def __init__(self, paths: Sequence[str], tokenizer, seq_length: int):
        self.paths, self.tokenizer, self.seq_length = list(paths), tokenizer, seq_length

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        buf: List[int] = []
        n = self.seq_length + 1
        for p in self.paths:
            for text in _iter_texts(p):
                buf.extend(_encode(self.tokenizer, text))
                while len(buf) >= n:
                    yield _make_item(torch.tensor(buf[:n], dtype=torch.long))
                    buf = buf[n:]


class ConversationDataset(Dataset):
    def __init__(self, paths: Sequence[str], tokenizer, seq_length: int, assistant_loss_weight: float = 1.5,
                 max_conversations: Optional[int] = None):
        self.tokenizer, self.seq_length, self.alw = tokenizer, seq_length, assistant_loss_weight
        self.conversations: List[List[Dict[str, str]]] = []
        self.stats = {"loaded": 0, "invalid": 0}
        for p in paths:
            with open(p) as f:
                for line in f:
                    line = line.strip()
                    if not line:
                        continue
                    try:
                        obj = json.loads(line)
                    except json.JSONDecodeError:
                        self.stats["invalid"] += 1
                        continue
                    msgs = obj.get("messages") if isinstance(obj, dict) else None
                    if self._valid(msgs):
                        self.conversations.append(msgs)
                        self.stats["loaded"] += 1
                    else:
                        self.stats["invalid"] += 1
                    if max_conversations and len(self.conversations) >= max_conversations:
                        break

    @staticmethod
    def _valid(msgs) -> bool:
        if not isinstance(msgs, list) or not msgs:
            return False
        for m in msgs:
            if not isinstance(m, dict) or not isinstance(m.get("content"), str) or not m["content"].strip():
                return False
            if m.get("role") not in ("system", "user", "assistant", "prompter", "human", "bot"):
                return False
        return True

    def __len__(self) -> int:
        return len(self.conversations)

    def __getitem__(self, i: int):
        ids, weights = [], []
        for m in self.conversations[i]:
            role = {"prompter": "user", "human": "user", "bot": "assistant"}.get(m["role"], m["role"])
            if hasattr(self.tokenizer, "encode_message"):
                toks = self.tokenizer.encode_message(role, m["content"])
            else:
                toks = _encode(self.tokenizer, m["content"])
            ids.extend(toks)
            weights.extend([self.alw if role == "assistant" else 1.0] * len(toks))
        n = self.seq_length + 1
        ids, weights = ids[:n], weights[:n]
        valid = len(ids)
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        ids = ids + [pad] * (n - valid)
        weights = weights + [0.0] * (n - valid)
        mask = torch.zeros(n)
        mask[:valid] = 1
        return _make_item(torch.tensor(ids, dtype=torch.long), torch.tensor(weights), mask)

    def total_tokens(self) -> int:
        return len(self) * self.seq_length


class InterleavedDataset(Dataset):
    """Deterministic mix of two datasets with a target ratio of the first (reference ``dataset.py:759-800``)."""

    def __init__(self, a: Dataset, b: Dataset, ratio_a: float = 0.5, seed: int = 0):
        self.a, self.b = a, b
        rng = random.Random(seed)
        n = len(a) + len(b)
        self.plan = []
        ia = ib = 0
        for _ in range(n):
            take_a = (rng.random() < ratio_a and ia < len(a)) or ib >= len(b)
            if take_a and ia < len(a):
                self.plan.append((0, ia))
                ia += 1
            elif ib < len(b):
                self.plan.append((1, ib))
                ib += 1

    def __len__(self) -> int:
        return len(self.plan)

    def __getitem__(self, i: int):
        which, j = self.plan[i]
        return (self.a if which == 0 else self.b)[j]


class HybridDatasetManager:
    def __init__(self, config, tokenizer):
        self.config, self.tokenizer = config, tokenizer

    def _base(self, paths):
        paths = [p for p in (paths or []) if os.path.exists(p)]
        if not paths:
            return None
        size_gb = sum(os.path.getsize(p) for p in paths) / 2 ** 30
        if size_gb > getattr(self.config, "streaming_threshold_gb", 10.0):
            return StreamingBaseTrainingDataset(paths, self.tokenizer, self.config.seq_length)
        return BaseTrainingDataset(paths, self.tokenizer, self.config.seq_length)

    def _conv(self, paths):
        paths = [p for p in (paths or []) if os.path.exists(p)]
        if not paths:
            return None
        return ConversationDataset(paths, self.tokenizer, self.config.seq_length, self.config.assistant_loss_weight,
                                   getattr(self.config, "max_conversations_per_file", None))

    def get_datasets(self):
        c = self.config
        mode = getattr(c, "training_mode", "finetuning_only")
        ft_paths = c.finetuning_paths or ([c.train_data_path] if c.train_data_path else [])
        ft_eval = c.finetuning_eval_paths or ([c.eval_data_path] if c.eval_data_path else [])
        if mode == "base_only":
            return self._base(c.base_training_paths), self._base(c.base_eval_paths)
        if mode == "finetuning_only":
            return self._conv(ft_paths), self._conv(ft_eval)
        base, conv = self._base(c.base_training_paths), self._conv(ft_paths)
        ev = self._conv(ft_eval) or self._base(c.base_eval_paths)
        if base is None or conv is None:
            return base or conv, ev
        if mode == "hybrid":
            return ConcatDataset([base, conv]), ev
        if mode == "interleaved":
            return InterleavedDataset(base, conv, c.base_finetuning_ratio, c.seed), ev
        raise ValueError(f"unknown training_mode {mode}")


def setup_datasets(config, tokenizer):
    return HybridDatasetManager(config, tokenizer).get_datasets()


def collate(items: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    return {k: torch.stack([it[k] for it in items]) for k in items[0]}


def create_dataloader(dataset, config, shuffle: bool = True, rank: Optional[int] = None, world: Optional[int] = None) -> DataLoader:
    """drop_last, pinned memory, and a DistributedSampler when several data-parallel ranks exist."""
    import torch.distributed as dist
    bs = config.micro_batch_size or config.batch_size
    iterable = isinstance(dataset, torch.utils.data.IterableDataset)
    sampler = None
    if not iterable:
        w = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        r = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        if w > 1:
            sampler = DistributedSampler(dataset, num_replicas=w, rank=r, shuffle=shuffle, seed=getattr(config, "seed", 0), drop_last=True)
    nw = 0 if iterable else min(getattr(config, "num_workers", 0), 8)
    return DataLoader(dataset, batch_size=bs, shuffle=(shuffle and sampler is None and not iterable), sampler=sampler,
                      drop_last=True, collate_fn=collate, num_workers=nw,
                      pin_memory=bool(getattr(config, "pin_memory", False)) and torch.cuda.is_available(),
                      prefetch_factor=(getattr(config, "prefetch_factor", 2) if nw > 0 else None))


create_fast_dataloader = create_dataloader


def _iter_texts(path: str) -> Iterator[str]:
    if path.endswith((".jsonl", ".json")):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                try:
                    obj = json.loads(line)
                except json.JSONDecodeError:
                    continue
                if isinstance(obj, dict) and isinstance(obj.get("text"), str):
                    yield obj["text"]
    else:
        with open(path, errors="ignore") as f:
            for para in f.read().split("\n\n"):
                if para.strip():
                    yield para


def _encode(tokenizer, text: str) -> List[int]:
    if hasattr(tokenizer, "encode"):
        out = tokenizer.encode(text)
    else:
        out = tokenizer.tokenizer.encode(text)
    return list(out)

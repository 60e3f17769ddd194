"""Continuous batching: a fixed pool of cache rows, requests of any length admitted and retired between decode steps.

The pool is one ``KVCache`` of ``max_batch`` rows and one captured decode step over it (``GraphDecoder``).  A row is a
sequence slot handed out by ``KVSlotManager``.  Every call of :meth:`ContinuousBatcher.step`

1. admits waiting requests into free rows: the prompt is prefilled straight into the row (a one-row view of the pool's cache), the
   row's length and RoPE position are set in device memory, and the first token is sampled from the prefill logits;
2. replays the decode graph once for all rows (each row attends over its own length; a free row has length 0 and its output is
   ignored), samples one token per row in one launch;
3. retires rows that produced a stop token or their token budget and frees their slots.

The reference's own generator serves one sequence at a time and re-runs the context for every token (``Chat.py:355-465``); its
vendored serving engine keeps a slot table per batch (``colossalai/inference/kv_cache/kvcache_manager.py:11-106`` allocator,
``kv_cache/batch_infer_state.py:13-118`` per-batch lengths and start locations), which is the bookkeeping done here on rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..models.transformer import KVCache
from .engine import GenerationEngine, GraphDecoder, KVSlotManager, SamplingParams, sample_next


@dataclass
class Request:
    rid: int
    prompt: torch.Tensor                      # [Lp] token ids (host or device)
    max_new_tokens: int
    tokens: List[int] = field(default_factory=list)
    slot: int = -1
    done: bool = False


class _RowView(KVCache):
    """One row of the pool's cache presented as a cache of batch 1 (prefill writes land in the pool)."""

    def __init__(self, pool: KVCache, row: int):  # noqa: D401  (no buffers of its own)
        self.k = [t[row:row + 1] for t in pool.k]
        self.v = [t[row:row + 1] for t in pool.v]
        self.length = 0
        self.max_len = pool.max_len
        self.device_lengths = None
        self.device_positions = None


class ContinuousBatcher:
    def __init__(self, engine: GenerationEngine, max_batch: int = 64, max_len: int = 2048, params: Optional[SamplingParams] = None):
        self.engine, self.model = engine, engine.model
        self.params = params or SamplingParams.from_mode("greedy")
        self.max_batch, self.max_len = max_batch, max_len
        self.device = next(self.model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("continuous batching replays a CUDA graph of the decode step: a CUDA device is required")
        if getattr(self.model, "_ep_comm", None) is not None:
            # admission prefills one request on one rank, which the expert-parallel exchange (a collective of all ranks) cannot serve
            raise RuntimeError("continuous batching runs on one GPU (or on replicas): the model must not be expert-parallel")
        self.cache = self.model.make_cache(max_batch, max_len)
        self.slots = KVSlotManager(max_batch)
        self.decoder = GraphDecoder(self.model, self.cache)        # captured once; rows come and go underneath it
        self.cache.device_lengths.zero_()
        self.cache.device_positions.zero_()
        self.active = torch.zeros(max_batch, dtype=torch.int32, device=self.device)     # 1 for rows that hold a live sequence
        self.last = torch.zeros(max_batch, dtype=torch.long, device=self.device)        # the token each row feeds next
        self.history = torch.zeros(max_batch, self.params.repetition_window, dtype=torch.long, device=self.device)
        self.by_slot: Dict[int, Request] = {}
        self.waiting: List[Request] = []
        self.finished: Dict[int, Request] = {}
        self._next_id = 0
        self._stop = set(int(t) for t in (self.params.stop_token_ids or ()))
        self.steps = 0
        self.generator = torch.Generator(device=self.device).manual_seed(self.params.seed) if self.params.seed is not None else None

    # -- requests --------------------------------------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], max_new_tokens: Optional[int] = None) -> int:
        ids = torch.as_tensor(prompt, dtype=torch.long).flatten()
        budget = int(max_new_tokens if max_new_tokens is not None else self.params.max_new_tokens)
        if ids.numel() < 1 or ids.numel() + budget > self.max_len:
            raise ValueError(f"prompt of {ids.numel()} tokens + {budget} new tokens does not fit rows of {self.max_len}")
        r = Request(self._next_id, ids, budget)
        self._next_id += 1
        self.waiting.append(r)
        return r.rid

    @property
    def pending(self) -> int:
        return len(self.waiting) + len(self.by_slot)

    # -- one scheduling step ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def _admit(self) -> None:
        while self.waiting and self.slots.available:
            r = self.waiting.pop(0)
            slot = int(self.slots.alloc(1)[0])
            ids = r.prompt.to(self.device).view(1, -1)
            logits = self.engine.prefill(ids, _RowView(self.cache, slot))
            n = ids.shape[1]
            self.cache.device_lengths[slot] = n
            self.cache.device_positions[slot] = n
            w = self.history.shape[1]
            self.history[slot].fill_(int(ids[0, 0]))      # left padding of a short prompt repeats its first token
            self.history[slot, -min(n, w):] = ids[0, -min(n, w):]
            first = sample_next(logits, self.params, self.history[slot:slot + 1], self.generator)
            self.last[slot:slot + 1] = first
            self.history[slot] = torch.roll(self.history[slot], -1)
            self.history[slot, -1:] = first
            r.slot = slot
            self.by_slot[slot] = r
            self.active[slot] = 1
            self._accept(slot, int(first))

    def _accept(self, slot: int, token: int) -> None:
        """Host-side bookkeeping of one generated token (the device-side state was updated for all rows at once)."""
        r = self.by_slot[slot]
        r.tokens.append(token)
        if token in self._stop or len(r.tokens) >= r.max_new_tokens:
            self._retire(slot)

    def _retire(self, slot: int) -> None:
        r = self.by_slot.pop(slot)
        r.done = True
        self.finished[r.rid] = r
        self.active[slot] = 0
        self.cache.device_lengths[slot] = 0
        self.cache.device_positions[slot] = 0
        self.slots.free(torch.tensor([slot]))

    @torch.no_grad()
    def step(self) -> int:
        """Admit, decode one token for every live row, retire.  Returns the number of live rows that were decoded."""
        self._admit()
        live = sorted(self.by_slot)
        if not live:
            return 0
        self.decoder.tokens.copy_(self.last.view(-1, 1))
        self.decoder.graph.replay()
        # the captured step advanced every row's counters: free rows go back to zero so that they never walk off their buffer
        self.cache.device_lengths.mul_(self.active)
        self.cache.device_positions.mul_(self.active)
        nxt_dev = sample_next(self.decoder.logits, self.params, self.history, self.generator)
        self.last.copy_(nxt_dev)
        self.history = torch.roll(self.history, -1, dims=1)
        self.history[:, -1] = nxt_dev
        nxt = nxt_dev.tolist()                       # the one device-to-host read of the step
        for slot in live:
            self._accept(slot, int(nxt[slot]))
        self.steps += 1
        return len(live)

    def run(self, prompts: Sequence[Sequence[int]], max_new_tokens: Optional[int] = None) -> List[List[int]]:
        """Serve all prompts; returns the generated ids in the order of ``prompts``."""
        rids = [self.submit(p, max_new_tokens) for p in prompts]
        while self.pending:
            self.step()
        return [self.finished.pop(r).tokens for r in rids]

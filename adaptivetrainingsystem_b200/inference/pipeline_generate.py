"""KV-cached generation across pipeline stages.

Every stage keeps the K/V cache of its own layers only.  A step moves one activation tensor per micro-batch from stage to stage
(``[b, prompt, hidden]`` during the prefill, ``[b, 1, hidden]`` afterwards); the last stage applies the final norm and the output
head to the last position, samples, and sends the new token ids back to the first stage.  The batch is cut into micro-batches
that follow each other through the stages, so with at least as many micro-batches as stages every stage has work while the
tokens of the other micro-batches travel back -- the schedule the reference's vendored tree implements with pickled metadata per
message (``colossalai/pipeline/schedule/generate.py:34-441``); here every message has a fixed shape and nothing is pickled.

Collective over the pipeline group: every stage calls :meth:`PipelineGenerator.generate` with the same arguments; every stage
returns the same ``[batch, new_tokens]`` tensor.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from ..models.transformer import KVCache
from ..parallel.pipeline import PipelineStage
from .engine import SamplingParams, sample_next


class _StageCache(KVCache):
    """A cache that holds buffers for this stage's layers only (the other entries are empty placeholders)."""

    def __init__(self, num_layers: int, own: range, batch: int, max_len: int, n_kv: int, head_dim: int, dtype, device):
        empty = torch.empty(0, dtype=dtype, device=device)
        self.k = [torch.zeros(batch, max_len, n_kv, head_dim, dtype=dtype, device=device) if i in own else empty for i in range(num_layers)]
        self.v = [torch.zeros(batch, max_len, n_kv, head_dim, dtype=dtype, device=device) if i in own else empty for i in range(num_layers)]
        self.length = 0
        self.max_len = max_len
        self.device_lengths = None
        self.device_positions = None


class PipelineGenerator:
    def __init__(self, stage: PipelineStage, group=None, ranks: Optional[List[int]] = None):
        """``ranks``: the global ranks of the pipeline stages in stage order (default: 0 .. stages - 1 of ``group``)."""
        self.stage, self.group = stage, group
        self.S, self.s = stage.num_stages, stage.stage
        self.ranks = list(ranks) if ranks is not None else list(range(self.S))
        m = stage.model
        p = next(q for q in m.parameters() if q.numel() > 0)
        self.device, self.dtype = p.device, p.dtype
        self.hidden = m.config.hidden_size
        self._inflight: list = []   # (request, tensor kept alive until the send has completed)

    # -- wire ------------------------------------------------------------------------------------------------------------
    def _send(self, t: torch.Tensor, stage: int) -> None:
        # never blocking: a stage may be sending activations forward while the last stage is sending it tokens
        t = t.contiguous()
        self._inflight.append((dist.isend(t, self.ranks[stage], group=self.group), t))
        # completed sends are dropped without ever waiting here (waiting inside the loop could close a cycle of waits between stages)
        self._inflight = [(w, k) for (w, k) in self._inflight if not w.is_completed()]

    def _recv(self, shape, dtype, stage: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, self.ranks[stage], group=self.group)
        return t

    # -- one stage pass over one micro-batch -------------------------------------------------------------------------------
    def _run(self, x: torch.Tensor, cache: KVCache, decode: bool) -> torch.Tensor:
        m, st = self.stage.model, self.stage
        if st.is_first:
            from .. import ops
            x = ops.embedding(x, m.embed_tokens.weight, math.sqrt(m.config.hidden_size) if m.config.use_stable_embedding else 1.0)
        n = x.shape[1]
        for blk in m.layers[st.start:st.end]:
            x, _ = blk(x, m.rope, None, cache, None, decode)
        cache.advance(n)
        return x

    def _head(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops
        m = self.stage.model
        logits = ops.linear(m.norm(x[:, -1:, :]), m.lm_head)
        if m.config.scale_lm_head_output:
            logits = logits / math.sqrt(m.config.hidden_size)
        return logits[:, -1, :]

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, params: Optional[SamplingParams] = None, micro_batches: int = 1) -> torch.Tensor:
        """input_ids [B, Lp] (equal-length prompts, the same tensor on every stage) -> generated ids [B, max_new_tokens]."""
        params = params or SamplingParams.from_mode("greedy")
        B, Lp = input_ids.shape
        M = max(1, min(micro_batches, B))
        if B % M:
            raise ValueError(f"batch {B} is not divisible into {M} micro-batches")
        b = B // M
        new = params.max_new_tokens
        m, st = self.stage.model, self.stage
        cfg = m.config
        n_kv = m.layers[st.start].self_attn.n_kv if st.end > st.start else cfg.num_kv_heads
        caches = [_StageCache(cfg.num_layers, range(st.start, st.end), b, Lp + new, n_kv, cfg.head_dim, self.dtype, self.device)
                  for _ in range(M)]
        ids = input_ids.to(self.device)
        gen = torch.Generator(device=self.device).manual_seed(params.seed) if params.seed is not None else None
        out = torch.zeros(B, new, dtype=torch.long, device=self.device)
        first, last = 0, self.S - 1
        for step in range(new):
            L = Lp if step == 0 else 1
            for i in range(M):
                rows = slice(i * b, (i + 1) * b)
                if st.is_first:
                    if step == 0:
                        x = ids[rows]
                    elif self.S > 1:
                        x = self._recv((b, 1), torch.long, last)          # the token this micro-batch produced one step ago
                    else:
                        x = out[rows, step - 1:step]
                else:
                    x = self._recv((b, L, self.hidden), self.dtype, self.s - 1)
                x = self._run(x, caches[i], decode=step > 0)
                if not st.is_last:
                    self._send(x, self.s + 1)
                    continue
                nxt = sample_next(self._head(x), params, None, gen)
                out[rows, step] = nxt
                if self.S > 1 and step + 1 < new:
                    self._send(nxt.view(b, 1), first)
        for w, _ in self._inflight:
            w.wait()
        self._inflight = []
        if self.S > 1:   # every stage returns the tokens
            dist.broadcast(out, self.ranks[last], group=self.group)
        return out

"""Inference runtime: batched prefill + decode with a grouped-query KV cache, sampling (repetition penalty,
temperature, top-k, top-p, greedy), stop conditions and streaming.

The reference's generator re-runs the whole context for every new token and has no cache (reference
``Chat.py:355-465``); its sampling API and generation modes (``Chat.py:60-85``) are kept, the loop is new:

* prefill runs the training kernels over the prompt (causal flash attention) and fills the cache;
* each decode step feeds one token per sequence: QKV GEMM -> RoPE at the cache offset -> attention of the single
  query against the cached K/V -> MoE FFN (router, dispatch, grouped SwiGLU GEMM, combine; expert-parallel ranks
  exchange the routed tokens through peer memory) -> next-token logits only for the last position;
* a slot allocator (``KVSlotManager``) hands out cache rows to ``inference/scheduler.py: ContinuousBatcher``, which admits and
  retires requests of any length between replays of one captured decode step (the vendored inference engine of the
  reference keeps the same bookkeeping, ``colossalai/inference/kv_cache/kvcache_manager.py:11-106``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import torch

from ..models.transformer import DeepSeekTransformer, KVCache

GENERATION_MODES: Dict[str, Dict[str, float]] = {
    "standard": dict(temperature=0.8, top_p=0.9, top_k=50, repetition_penalty=1.1),
    "creative": dict(temperature=1.0, top_p=0.95, top_k=100, repetition_penalty=1.05),
    "precise": dict(temperature=0.3, top_p=0.7, top_k=20, repetition_penalty=1.2),
    "analytical": dict(temperature=0.5, top_p=0.8, top_k=40, repetition_penalty=1.15),
    "greedy": dict(temperature=0.0, top_p=1.0, top_k=0, repetition_penalty=1.0),
}


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 50
    top_p: float = 0.9
    repetition_penalty: float = 1.1
    repetition_window: int = 50
    max_new_tokens: int = 512
    stop_token_ids: Sequence[int] = field(default_factory=tuple)
    seed: Optional[int] = None

    @classmethod
    def from_mode(cls, mode: str, **kw) -> "SamplingParams":
        return cls(**{**GENERATION_MODES[mode], **kw})


def sample_next(logits: torch.Tensor, params: SamplingParams, history: Optional[torch.Tensor] = None,
                generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """logits [B, V] -> token ids [B].  Order of operations as in the reference (``Chat.py:391-425``): repetition
    penalty over the last ``repetition_window`` tokens, temperature, top-k, top-p, multinomial; ``temperature <= 0``
    is greedy.  On a GPU the whole chain is one kernel launch per step (bisection on the logit values instead of a sort)."""
    if logits.is_cuda and logits.dim() == 2:
        from ..ops import serving
        hist = history[:, -params.repetition_window:] if history is not None and history.numel() else None
        return serving.sample_tokens(logits, params.temperature, params.top_k, params.top_p, params.repetition_penalty, hist,
                                     generator=generator)
    lg = logits.float()
    if history is not None and params.repetition_penalty != 1.0 and history.numel():
        h = history[:, -params.repetition_window:]
        picked = torch.gather(lg, 1, h)
        picked = torch.where(picked > 0, picked / params.repetition_penalty, picked * params.repetition_penalty)
        lg = lg.scatter(1, h, picked)
    if params.temperature <= 0:
        return lg.argmax(-1)
    lg = lg / params.temperature
    if params.top_k and params.top_k < lg.shape[-1]:
        kth = torch.topk(lg, params.top_k, dim=-1).values[:, -1:]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    if params.top_p < 1.0:
        sl, si = torch.sort(lg, dim=-1, descending=True)
        cp = torch.softmax(sl, -1).cumsum(-1)
        drop = cp - torch.softmax(sl, -1) > params.top_p
        sl = sl.masked_fill(drop, float("-inf"))
        lg = torch.full_like(lg, float("-inf")).scatter(1, si, sl)
    probs = torch.softmax(lg, -1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(1)


class KVSlotManager:
    """Free-list of cache rows for continuous batching: ``alloc(n)`` returns n free slots (lowest first),
    ``alloc_contiguous(n)`` a run of n, ``free(slots)`` returns them."""

    def __init__(self, size: int):
        self.size = size
        self.free_mask = torch.ones(size, dtype=torch.bool)

    @property
    def available(self) -> int:
        return int(self.free_mask.sum())

    def alloc(self, n: int) -> Optional[torch.Tensor]:
        idx = torch.nonzero(self.free_mask, as_tuple=False).flatten()
        if idx.numel() < n:
            return None
        sel = idx[:n]
        self.free_mask[sel] = False
        return sel

    def alloc_contiguous(self, n: int) -> Optional[torch.Tensor]:
        if n > self.size:
            return None
        run = torch.nn.functional.conv1d(self.free_mask.float().view(1, 1, -1), torch.ones(1, 1, n)).flatten()
        starts = torch.nonzero(run == n, as_tuple=False).flatten()
        if not starts.numel():
            return None
        s = int(starts[0])
        self.free_mask[s:s + n] = False
        return torch.arange(s, s + n)

    def free(self, slots: torch.Tensor) -> None:
        self.free_mask[slots] = True


class GenerationEngine:
    def __init__(self, model: DeepSeekTransformer, tokenizer=None, max_batch: int = 64, max_len: Optional[int] = None,
                 pack_experts: bool = False, use_kv_cache: bool = True, kv_cache_dtype: str = "auto"):
        """``use_kv_cache=False`` is the reference's generation loop (``Chat.py:379-452``: the whole sequence is run again for
        every token), kept for comparison; ``kv_cache_dtype``: ``"auto"`` / the model's dtype (an 8-bit cache is not built)."""
        self.model = model.eval()
        self.use_kv_cache = bool(use_kv_cache)
        own = {torch.bfloat16: ("bf16", "bfloat16"), torch.float32: ("fp32", "float32"), torch.float16: ("fp16", "float16")}
        dt = next(model.parameters()).dtype
        if kv_cache_dtype not in ("auto", None) and kv_cache_dtype not in own.get(dt, ()) and not (kv_cache_dtype == "bf16" and dt == torch.float32):
            raise ValueError(f"kv_cache_dtype {kv_cache_dtype!r}: the cache holds the model's dtype ({dt}); an 8-bit cache is not built")
        self.tokenizer = tokenizer
        self.max_batch = max_batch
        self.max_len = max_len or model.config.seq_length
        self.stats: Dict[str, float] = {}
        if pack_experts:
            self.pack_expert_weights()

    @torch.no_grad()
    def pack_expert_weights(self) -> int:
        """Re-store every expert weight tile by tile (``ops.gemm.pack_kmajor``) for serving: a decode step reads each expert
        weight exactly once, and whole-page reads stream it faster than 128-byte row pieces.  The model can no longer be
        trained or saved in the reference layout afterwards (``ops.gemm.unpack_kmajor`` restores a tensor).  Returns the
        number of tensors packed."""
        from ..ops import gemm as G
        n = 0
        for mod in self.model.modules():
            w1, w2 = getattr(mod, "experts_w1", None), getattr(mod, "experts_w2", None)
            if w1 is None or w2 is None or getattr(w1, "_ats_packed", False) or not w1.is_cuda:
                continue
            if w1.shape[1] % 256 or w1.shape[2] % 64 or w2.shape[1] % 128 or w2.shape[2] % 64:
                continue
            for w in (w1, w2):
                w.requires_grad_(False)
                w.data = G.pack_kmajor(w.data)
                w._ats_packed = True
                n += 1
        if n and torch.cuda.is_available():
            # the plain copies went back to PyTorch's caching allocator; the peer-memory exchange buffers of expert
            # parallelism are allocated outside it and need that memory returned to the driver
            torch.cuda.empty_cache()
        return n

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """Runs the prompt, fills the cache, returns the logits of the last position [B, V]."""
        logits = self.model(input_ids, cache=cache, last_token_only=True, return_aux_loss=False)
        return logits[:, -1, :]

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """tokens [B] -> logits [B, V] for the next position."""
        logits = self.model(tokens.view(-1, 1), cache=cache, last_token_only=True, return_aux_loss=False)
        return logits[:, -1, :]

    @torch.no_grad()
    def graph_decoder(self, cache: KVCache) -> "GraphDecoder":
        """Capture one decode step (all layers, launch-bound at batch <= 64) into a CUDA graph bound to ``cache``."""
        return GraphDecoder(self.model, cache)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, params: Optional[SamplingParams] = None,
                 on_token: Optional[Callable[[int, torch.Tensor], None]] = None, use_graph: Optional[bool] = None) -> Dict[str, object]:
        """input_ids [B, Lp] (equal-length prompts) -> dict(tokens [B, <=max_new], prefill_s, decode_s, ...).
        Timed with device synchronisation on both sides of each phase."""
        params = params or SamplingParams()
        dev = input_ids.device
        B, Lp = input_ids.shape
        if not self.use_kv_cache:
            return self._generate_without_cache(input_ids, params, on_token)
        total = Lp + params.max_new_tokens
        cache = self.model.make_cache(B, total)
        gen = None
        if params.seed is not None:
            gen = torch.Generator(device=dev).manual_seed(params.seed)
        sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)
        sync()
        t0 = time.perf_counter()
        logits = self.prefill(input_ids, cache)
        sync()
        t1 = time.perf_counter()
        history = input_ids
        out: List[torch.Tensor] = []
        decoder = None
        if use_graph is None:
            use_graph = dev.type == "cuda" and next(self.model.parameters()).dtype == torch.bfloat16 and params.max_new_tokens > 8
        if use_graph:
            decoder = self.graph_decoder(cache)  # capture is part of the timed decode phase
        finished = torch.zeros(B, dtype=torch.bool, device=dev)
        stop = torch.tensor(list(params.stop_token_ids), device=dev, dtype=torch.long) if params.stop_token_ids else None
        steps = 0
        for step in range(params.max_new_tokens):
            nxt = sample_next(logits, params, history, gen)
            if stop is not None:
                finished |= (nxt[:, None] == stop[None, :]).any(-1)
            out.append(nxt)
            steps += 1
            if on_token is not None:
                on_token(step, nxt)
            if stop is not None and bool(finished.all()):
                break
            history = torch.cat([history, nxt[:, None]], dim=1)
            if step + 1 < params.max_new_tokens:
                logits = decoder.step(nxt) if decoder is not None else self.decode_step(nxt, cache)
        sync()
        t2 = time.perf_counter()
        self.stats = {"prefill_s": t1 - t0, "decode_s": t2 - t1, "prefill_tokens_per_s": B * Lp / max(t1 - t0, 1e-9),
                      "decode_tokens_per_s": B * max(steps - 1, 1) / max(t2 - t1, 1e-9), "steps": steps}
        return {"tokens": torch.stack(out, dim=1), **self.stats}

    @torch.no_grad()
    def _generate_without_cache(self, input_ids: torch.Tensor, params: SamplingParams, on_token=None) -> Dict[str, object]:
        """Every step runs the whole sequence again (quadratic in the length): the reference's loop, for comparison only."""
        dev = input_ids.device
        gen = torch.Generator(device=dev).manual_seed(params.seed) if params.seed is not None else None
        sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)
        stop = torch.tensor(list(params.stop_token_ids), device=dev, dtype=torch.long) if params.stop_token_ids else None
        finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=dev)
        history, out = input_ids, []
        sync()
        t0 = time.perf_counter()
        for step in range(params.max_new_tokens):
            logits = self.model(history, last_token_only=True, return_aux_loss=False)[:, -1, :]
            nxt = sample_next(logits, params, history, gen)
            out.append(nxt)
            if on_token is not None:
                on_token(step, nxt)
            if stop is not None:
                finished |= (nxt[:, None] == stop[None, :]).any(-1)
                if bool(finished.all()):
                    break
            history = torch.cat([history, nxt[:, None]], dim=1)
        sync()
        dt = time.perf_counter() - t0
        self.stats = {"prefill_s": 0.0, "decode_s": dt, "prefill_tokens_per_s": 0.0,
                      "decode_tokens_per_s": input_ids.shape[0] * len(out) / max(dt, 1e-9), "steps": len(out), "kv_cache": False}
        return {"tokens": torch.stack(out, dim=1), **self.stats}

    # ---------------------------------------------------------------------------------------------------------------
    def generate_text(self, prompt: str, params: Optional[SamplingParams] = None) -> str:
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer is needed for text generation")
        dev = next(self.model.parameters()).device
        ids = torch.tensor([self.tokenizer.encode(prompt)], dtype=torch.long, device=dev)
        res = self.generate(ids, params)
        return self.tokenizer.decode(res["tokens"][0].tolist())

    def stream(self, prompt: str, params: Optional[SamplingParams] = None) -> Iterator[str]:
        """Yields decoded text piece by piece (one model step per yielded token)."""
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer is needed for text generation")
        params = params or SamplingParams()
        dev = next(self.model.parameters()).device
        ids = torch.tensor([self.tokenizer.encode(prompt)], dtype=torch.long, device=dev)
        cache = self.model.make_cache(1, ids.shape[1] + params.max_new_tokens)
        with torch.no_grad():
            logits = self.prefill(ids, cache)
            history = ids
            for _ in range(params.max_new_tokens):
                nxt = sample_next(logits, params, history)
                if params.stop_token_ids and int(nxt) in set(params.stop_token_ids):
                    return
                yield self.tokenizer.decode([int(nxt)])
                history = torch.cat([history, nxt[:, None]], dim=1)
                logits = self.decode_step(nxt, cache)


class GraphDecoder:
    """One decode step of the whole model as a CUDA graph.  A decode step at serving batch sizes is a few hundred small
    launches whose host-side cost exceeds their device time; replaying a captured graph removes that cost.  Everything that
    changes from step to step lives in device memory: the input tokens (a static buffer), the cache fill level and the RoPE
    positions (``KVCache.device_lengths`` / ``device_positions``, advanced inside the graph)."""

    def __init__(self, model: DeepSeekTransformer, cache: KVCache, warmup: int = 2):
        self.model, self.cache = model, cache
        dev = cache.k[0].device
        B = cache.k[0].shape[0]
        self.tokens = torch.zeros(B, 1, dtype=torch.long, device=dev)
        start = cache.length
        cache.enable_device_lengths()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):  # builds every lazily created buffer / function attribute outside the capture
                self._run()
        torch.cuda.current_stream(dev).wait_stream(side)
        cache.device_lengths.fill_(start)   # the warm-up wrote K / V beyond the fill level: harmless, rewind the counters
        cache.device_positions.fill_(start)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = self._run()
        cache.device_lengths.fill_(start)   # capture does not execute, but keep the invariant explicit
        cache.device_positions.fill_(start)

    def _run(self) -> torch.Tensor:
        logits = self.model(self.tokens, cache=self.cache, last_token_only=True, return_aux_loss=False)[:, -1, :]
        self.cache.device_advance()
        return logits

    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] -> logits [B, V] (a static buffer that the next step overwrites)."""
        if self.cache.length + 1 > self.cache.max_len:
            raise RuntimeError(f"KV cache overflow: {self.cache.length}+1 > {self.cache.max_len}")
        self.tokens.copy_(tokens.view(-1, 1))
        self.graph.replay()
        self.cache.length += 1
        return self.logits

"""Decoder-only language model: dense, Mixture-of-Experts, Mixture-of-Depths or hybrid.

Architecture and semantics follow the reference model (reference ``core/model.py``): pre-norm blocks with
RMSNorm (``:228-304``), grouped-query attention with half-split RoPE (``:470-853``), bias-free SwiGLU FFN with a
fused ``gate_up_proj`` (``:1027-1088``), top-k MoE with softmax over all experts and renormalised kept
probabilities plus the ``E * sum f_e P_e`` auxiliary loss (``:1090-1302``), Mixture-of-Depths routing
(``:860-1020``), tied or untied output head (``:1957-1973``).

What differs on purpose (the reference documents these but does not implement them):

* expert capacity is enforced (tokens beyond ``capacity_factor`` are dropped in token order);
* Mixture-of-Depths really skips compute: the selected tokens are gathered, run through the FFN and scattered
  back; selection is per sequence (``mod_per_sequence``), not over the whole batch;
* a KV cache is threaded through block and model with correct rotary offsets.

Parameters are stored fused for the kernels (one ``qkv_proj``, stacked expert weights) and exposed under the
reference's state-dict names (``layers.N.self_attn.q_proj.weight``, ``layers.N.ffn.experts.E.gate_up_proj.weight``
...) by ``state_dict`` / ``load_state_dict`` hooks, so checkpoints are interchangeable.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..config import ModelConfig
from .. import ops
from ..ops import moe as moe_ops
from ..ops import mod as mod_ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)

    def with_skip(self, x: torch.Tensor):
        """-> (norm(x), x) as one autograd node: the gradients of the normalised branch and of the residual branch are
        summed inside the norm's backward kernel."""
        return ops.rms_norm_skip(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    """Bias-optional LayerNorm kept for API parity (reference ``core/model.py:307-327``)."""

    def __init__(self, dim: int, eps: float = 1e-5, bias: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class RotaryEmbedding(nn.Module):
    """cos/sin tables [max_pos, d/2] in fp32 (frequencies computed in fp64), grown on demand."""

    def __init__(self, dim: int, max_position: int = 2048, theta: float = 10000.0, scaling_factor: float = 1.0):
        super().__init__()
        self.dim, self.theta, self.scaling_factor = dim, theta, scaling_factor
        cos, sin = ops.rope_tables(max_position, dim, theta, scaling_factor)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def ensure(self, length: int, device) -> None:
        # the tables stay fp32 even when the module was cast with .to(bfloat16): the kernels read them as float
        if length > self.cos.shape[0] or self.cos.device != torch.device(device) or self.cos.dtype != torch.float32:
            n = max(length, self.cos.shape[0])
            if length > self.cos.shape[0]:
                n = max(length, 2 * self.cos.shape[0])
            cos, sin = ops.rope_tables(n, self.dim, self.theta, self.scaling_factor, device)
            self.cos, self.sin = cos, sin

    def forward(self, length: int, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
        self.ensure(length, device or self.cos.device)
        return self.cos[:length], self.sin[:length]


class KVCache:
    """Contiguous per-layer K/V buffers ``[B, max_len, Hkv, D]`` plus the filled length."""

    def __init__(self, num_layers: int, batch: int, max_len: int, n_kv: int, head_dim: int, dtype, device):
        self.k = [torch.zeros(batch, max_len, n_kv, head_dim, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(batch, max_len, n_kv, head_dim, dtype=dtype, device=device) for _ in range(num_layers)]
        self.length = 0
        self.max_len = max_len
        # device-side copy of the fill level, used when the decode step is replayed from a CUDA graph (a Python integer
        # would be frozen into the captured launches): per-sequence lengths for the attention kernel, positions for RoPE
        self.device_lengths: Optional[torch.Tensor] = None
        self.device_positions: Optional[torch.Tensor] = None

    def enable_device_lengths(self) -> None:
        dev = self.k[0].device
        B = self.k[0].shape[0]
        self.device_lengths = torch.full((B,), self.length, dtype=torch.int32, device=dev)
        self.device_positions = torch.full((B,), self.length, dtype=torch.int32, device=dev)

    def device_advance(self) -> None:
        """One decoded token: called inside the captured step."""
        self.device_lengths += 1
        self.device_positions += 1

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        n = k.shape[1]
        if self.length + n > self.max_len:
            raise RuntimeError(f"KV cache overflow: {self.length}+{n} > {self.max_len}")
        self.k[layer][:, self.length:self.length + n] = k
        self.v[layer][:, self.length:self.length + n] = v
        return self.k[layer][:, : self.length + n], self.v[layer][:, : self.length + n]

    def advance(self, n: int) -> None:
        self.length += n

    def reset(self) -> None:
        self.length = 0


class GroupedQueryAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.n_q, self.n_kv, self.d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        width = (self.n_q + 2 * self.n_kv) * self.d
        self.qkv_proj = nn.Parameter(torch.empty(width, cfg.hidden_size))
        self.o_proj = nn.Parameter(torch.empty(cfg.hidden_size, self.n_q * self.d))
        # set by parallel.strategy: tensor parallelism (this rank's heads only, outputs all-reduced) and head-scatter sequence
        # parallelism (this rank's tokens only, heads exchanged for tokens around the attention)
        self.tp_group = None
        self.sp_group = None
        self.sp_size, self.sp_rank = 1, 0

    def _project_out(self, a: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        if self.tp_group is None:
            return ops.linear(a, self.o_proj, residual=residual)
        from ..parallel.tensor_parallel import _ReduceFromRegion
        return _ReduceFromRegion.apply(ops.linear(a, self.o_proj), self.tp_group) + residual

    def _forward_sequence_parallel(self, h, residual, rope):
        """Every rank holds L / W tokens: rotary positions are global, heads are traded for tokens around the attention."""
        from ..parallel.sequence_parallel import scatter_heads_gather_sequence, scatter_sequence_gather_heads
        B, L, _ = h.shape
        W, r = self.sp_size, self.sp_rank
        rope.ensure(W * L, h.device)
        qkv = ops.linear(h, self.qkv_proj, reduce_group=self.tp_group)
        qkv = ops.rope_packed(qkv, rope.cos, rope.sin, self.n_q, self.n_kv, self.d, pos_offset=r * L)
        nq, nk = self.n_q * self.d, self.n_kv * self.d
        q = scatter_heads_gather_sequence(qkv[..., :nq].reshape(B, L, self.n_q, self.d), self.sp_group)
        k = scatter_heads_gather_sequence(qkv[..., nq:nq + nk].reshape(B, L, self.n_kv, self.d), self.sp_group)
        v = scatter_heads_gather_sequence(qkv[..., nq + nk:].reshape(B, L, self.n_kv, self.d), self.sp_group)
        a = scatter_sequence_gather_heads(ops.attention(q, k, v, causal=True), self.sp_group)
        return self._project_out(a.reshape(B, L, nq), residual)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, rope: RotaryEmbedding,
                attention_mask: Optional[torch.Tensor] = None, cache: Optional[KVCache] = None,
                positions: Optional[torch.Tensor] = None, post_norm: Optional["RMSNorm"] = None):
        """-> x (= attention output projected + residual).  With ``post_norm`` (graph-replayed decode steps only) -> (x, h) where
        h = post_norm(x) came out of the launch that folded the output projection, or ``None`` when that form did not apply."""
        B, L, _ = h.shape
        if self.sp_group is not None and cache is None and attention_mask is None and positions is None:
            return self._forward_sequence_parallel(h, residual, rope)
        offset = cache.length if cache is not None else 0
        graph_decode = cache is not None and cache.device_lengths is not None and L == 1
        if graph_decode:
            # fill level and positions come from device memory, nothing of this call depends on Python state
            rope.ensure(cache.max_len, h.device)
            qkv = None
            if self.tp_group is None:  # the fold of the split projection also rotates q and k
                q2 = ops.serving.qkv_rope(h.reshape(B, -1), self.qkv_proj, rope.cos, rope.sin, cache.device_positions, self.n_q, self.n_kv, self.d)
                qkv = q2.view(B, 1, -1) if q2 is not None else None
            if qkv is None:
                qkv = ops.linear(h, self.qkv_proj, reduce_group=self.tp_group)
                qkv = ops.rope_packed(qkv, rope.cos, rope.sin, self.n_q, self.n_kv, self.d, positions=cache.device_positions.view(B, 1))
            a = ops.decode_attention(qkv, cache.k[self.layer_idx], cache.v[self.layer_idx], cache.device_lengths, self.n_q, self.n_kv, self.d)
            if post_norm is not None and self.tp_group is None:  # the fold of the output projection adds the residual and normalises
                fused = ops.serving.out_proj_norm(a.reshape(B, -1), self.o_proj, residual.reshape(B, -1), post_norm.weight, post_norm.eps)
                if fused is not None:
                    return fused[0].view(residual.shape), fused[1].view(residual.shape)
            x = self._project_out(a, residual)
            return (x, None) if post_norm is not None else x
        rope.ensure(offset + L if positions is None else int(self.cfg.seq_length), h.device)
        qkv = ops.linear(h, self.qkv_proj, reduce_group=self.tp_group)
        nq, nk = self.n_q * self.d, self.n_kv * self.d
        if (cache is None and attention_mask is None and positions is None and self.d % 16 == 0
                and ops.attention_packed_available(qkv, self.d, L)):
            # training / scoring path: rotation and attention are one autograd node on the projection buffer
            a = ops.rope_attention_packed(qkv, rope.cos, rope.sin, self.n_q, self.n_kv, self.d, pos_offset=0)
            return self._project_out(a.reshape(B, L, nq), residual)
        qkv = ops.rope_packed(qkv, rope.cos, rope.sin, self.n_q, self.n_kv, self.d, pos_offset=offset, positions=positions)
        if cache is None and attention_mask is None and ops.attention_packed_available(qkv, self.d, L):
            a = ops.attention_packed(qkv, self.n_q, self.n_kv, self.d)
            return self._project_out(a.reshape(B, L, nq), residual)
        if (cache is not None and L == 1 and attention_mask is None and positions is None
                and ops.decode_attention_available(qkv, self.n_q, self.n_kv, self.d)):
            # single-token step: the kernel appends K / V to the cache and attends in one pass over the cache
            a = ops.decode_attention(qkv, cache.k[self.layer_idx], cache.v[self.layer_idx], cache.length, self.n_q, self.n_kv, self.d)
            return self._project_out(a, residual)
        q = qkv[..., :nq].view(B, L, self.n_q, self.d)
        k = qkv[..., nq:nq + nk].view(B, L, self.n_kv, self.d)
        v = qkv[..., nq + nk:].view(B, L, self.n_kv, self.d)
        if cache is not None:
            k, v = cache.append(self.layer_idx, k, v)
        a = ops.attention(q, k, v, causal=True, q_offset=offset, key_mask=attention_mask)
        return self._project_out(a.reshape(B, L, nq), residual)


class DenseSwiGLU(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size))
        self.down_proj = nn.Parameter(torch.empty(cfg.hidden_size, cfg.intermediate_size))
        self.tp_group = None  # set by parallel.strategy.apply_tensor_parallel: this rank's columns, outputs all-reduced

    def forward(self, h: torch.Tensor, residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import _ReduceFromRegion
            # the all-reduce of the input gradient starts inside the MLP's backward and runs under its weight-gradient products
            y = _ReduceFromRegion.apply(ops.swiglu_mlp(h, self.gate_up_proj, self.down_proj, reduce_group=self.tp_group), self.tp_group)
            return (y + residual if residual is not None else y), None
        return ops.swiglu_mlp(h, self.gate_up_proj, self.down_proj, residual), None


class SwiGLUExpert(nn.Module):
    """A single expert as a stand-alone module (used by tests and by expert add/prune bookkeeping)."""

    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(2 * inter, hidden))
        self.down_proj = nn.Parameter(torch.empty(hidden, inter))
        nn.init.normal_(self.gate_up_proj, std=0.02)
        nn.init.normal_(self.down_proj, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.swiglu_mlp(x, self.gate_up_proj, self.down_proj)


class MoEFFNLayer(nn.Module):
    """Top-k routed experts.  ``experts_w1`` [E_local, 2I, H] / ``experts_w2`` [E_local, H, I] hold the experts
    of this rank (all of them without expert parallelism)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, ep_size: int = 1, ep_rank: int = 0):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.num_experts = cfg.num_experts
        self.top_k = cfg.moe_top_k
        self.capacity_factor = cfg.capacity_factor
        self.routing_temperature = cfg.routing_temperature
        self.routing_noise_std = cfg.routing_noise_std
        self.load_balancing_weight = cfg.load_balancing_weight
        self.router_z_loss_weight = float(getattr(cfg, "router_z_loss_weight", 0.0))
        self.expert_dropout = 0.0
        self.ep_size, self.ep_rank = ep_size, ep_rank
        assert cfg.num_experts % ep_size == 0, "num_experts must be divisible by the expert-parallel degree"
        e_local = cfg.num_experts // ep_size
        self.gate = nn.Linear(cfg.hidden_size, cfg.num_experts, bias=False)
        self.experts_w1 = nn.Parameter(torch.empty(e_local, 2 * cfg.intermediate_size, cfg.hidden_size))
        self.experts_w2 = nn.Parameter(torch.empty(e_local, cfg.hidden_size, cfg.intermediate_size))
        self.experts_w1._ats_expert = True
        self.experts_w2._ats_expert = True
        self.register_buffer("expert_demand", torch.zeros(cfg.num_experts, dtype=torch.float64), persistent=False)
        self.register_buffer("tokens_seen", torch.zeros((), dtype=torch.float64), persistent=False)
        self.register_buffer("dropped_slots", torch.zeros((), dtype=torch.float64), persistent=False)
        self.ep = None  # set by parallel.expert_parallel.attach when world size > 1

    def forward(self, h: torch.Tensor, residual: Optional[torch.Tensor] = None, next_norm=None):
        """-> (output, auxiliary loss); with ``next_norm`` = (weight, eps) on a decode-sized step whose combine launch also
        normalised its result for the next block -> (output, None, normalised output)."""
        shape = h.shape
        x = h.reshape(-1, shape[-1])
        T = x.shape[0]
        E, k = self.num_experts, self.top_k
        if not self.training and moe_ops.serving_path_ok(x, E, k):
            # decode-sized step: routing, permutation and combine are three small launches around the grouped GEMMs; the
            # exchange between expert-parallel ranks happens inside them (no auxiliary loss, no statistics while serving)
            res2 = residual.reshape(-1, shape[-1]) if residual is not None else None
            if self.ep is not None:
                served = self.ep.moe_serving(x, self.gate.weight, k, self.routing_temperature, self.experts_w1, self.experts_w2, res2,
                                             next_norm=next_norm)
            else:
                served = moe_ops.moe_ffn_serving(x, self.gate.weight, k, self.routing_temperature, self.experts_w1, self.experts_w2, res2,
                                                 next_norm=next_norm)
            if served is not None:
                if next_norm is not None:
                    out, normed = served[0]
                    return out.view(shape), None, (normed.view(shape) if normed is not None else None)
                return served[0].view(shape), None
        logits = moe_ops.gate_logits(x, self.gate.weight)
        fused_route = logits.is_cuda and not (self.training and self.routing_noise_std > 0) and logits.dtype == torch.float32
        if fused_route:
            idx, w, aux = moe_ops.route_and_balance(logits, k, self.routing_temperature, self.load_balancing_weight)
        else:
            idx, w, clean = moe_ops.route(logits, k, self.routing_temperature, self.routing_noise_std, self.training)
        if self.training and self.expert_dropout > 0:
            keep = (torch.rand_like(w) >= self.expert_dropout).float()
            keep[:, 0] = 1.0
            w = w * keep
            w = w / w.sum(-1, keepdim=True).clamp(min=1e-20)
        if not fused_route:
            aux = moe_ops.load_balancing_loss(clean, idx, E, self.load_balancing_weight)
        if self.router_z_loss_weight > 0 and self.training:
            # router z-loss: mean squared log-partition of the (un-noised) gate logits; it keeps the logits from drifting to magnitudes
            # where the soft-max saturates (reference: colossalai/moe/routers.py:94-110)
            aux = aux + self.router_z_loss_weight * torch.logsumexp(logits.float(), dim=-1).pow(2).mean()
        cap = moe_ops.expert_capacity(T, E, k, self.capacity_factor, self.cfg.drop_tokens)
        res2 = residual.reshape(-1, shape[-1]) if residual is not None else None
        if self.ep is not None:
            out, totals = self.ep.moe_ffn(x, idx, w.to(torch.float32), self.experts_w1, self.experts_w2, cap, res2)
        else:
            out, totals = moe_ops._MoEFFNFn.apply(x, idx, w.to(torch.float32), self.experts_w1, self.experts_w2, cap, res2)
        if self.training or torch.is_grad_enabled():  # routing statistics are a training-time instrument
            with torch.no_grad():
                self.expert_demand += totals.to(torch.float64)
                self.tokens_seen += T
                self.dropped_slots += (totals - totals.clamp(max=cap)).sum().to(torch.float64)
        return out.view(shape), aux

    @torch.no_grad()
    def get_routing_stats(self, reset: bool = False) -> Dict[str, Any]:
        d = self.expert_demand.cpu()
        tot = float(d.sum())
        usage = (d / tot).tolist() if tot > 0 else [0.0] * self.num_experts
        mean = 1.0 / self.num_experts
        stats = {
            "expert_usage": usage,
            "usage_std": float(torch.tensor(usage).std()) if tot > 0 else 0.0,
            "min_usage": min(usage), "max_usage": max(usage),
            "imbalance_ratio": (max(usage) / max(min(usage), 1e-9)) if tot > 0 else 1.0,
            "load_balance": 1.0 - float(torch.tensor(usage).sub(mean).abs().sum()) / 2 if tot > 0 else 1.0,
            "dropped_fraction": float(self.dropped_slots.cpu()) / tot if tot > 0 else 0.0,
            "tokens_seen": float(self.tokens_seen.cpu()),
        }
        if reset:
            self.expert_demand.zero_()
            self.tokens_seen.zero_()
            self.dropped_slots.zero_()
        return stats


class MoDRouter(nn.Module):
    """Token router of Mixture-of-Depths: a linear score per token.  Training / prefill: the top ``capacity``
    fraction of every sequence is processed.  The auxiliary loss trains the sigmoid of the score to predict
    membership in that top set so that causal decoding can use ``score > 0`` without looking ahead."""

    def __init__(self, hidden: int, capacity_factor: float = 0.5, temperature: float = 1.0):
        super().__init__()
        self.router = nn.Linear(hidden, 1, bias=True)
        self.capacity_factor = capacity_factor
        self.temperature = temperature
        self.register_buffer("selected_tokens", torch.zeros((), dtype=torch.float64), persistent=False)
        self.register_buffer("total_tokens", torch.zeros((), dtype=torch.float64), persistent=False)

    def keep_count(self, seq_len: int) -> int:
        return max(1, min(seq_len, int(math.ceil(seq_len * self.capacity_factor))))

    def forward(self, h: torch.Tensor, per_sequence: bool = True, decode: bool = False):
        """-> (sel [B, keep] ascending positions, weight [B, keep], aux loss, scores [B, L])"""
        B, L, _ = h.shape
        scores = (F.linear(h.float(), self.router.weight.float(), self.router.bias.float()).squeeze(-1)) / self.temperature
        if decode:
            return None, None, scores.new_zeros(()), scores
        keep = self.keep_count(L)
        if per_sequence:
            if scores.is_cuda and not torch.is_grad_enabled():
                sel = _mod_select_cuda(scores.detach(), keep)
            else:
                sel = torch.topk(scores.detach(), keep, dim=1).indices.sort(dim=1).values
        else:  # whole-batch selection (reference behaviour, core/model.py:937-938); padded to a rectangle
            flat = scores.detach().reshape(-1)
            top = torch.topk(flat, keep * B).indices
            member = torch.zeros_like(flat, dtype=torch.bool)
            member[top] = True
            sel = torch.topk(member.view(B, L).float() * 2 + scores.detach().sigmoid(), keep, dim=1).indices.sort(dim=1).values
        weight = torch.sigmoid(torch.gather(scores, 1, sel.long()))
        target = torch.zeros_like(scores)
        target.scatter_(1, sel.long(), 1.0)
        aux = F.binary_cross_entropy_with_logits(scores, target)
        with torch.no_grad():
            self.selected_tokens += float(B * keep)
            self.total_tokens += float(B * L)
        return sel, weight, aux, scores

    @torch.no_grad()
    def get_stats(self) -> Dict[str, float]:
        tot = float(self.total_tokens.cpu())
        ratio = float(self.selected_tokens.cpu()) / tot if tot > 0 else self.capacity_factor
        return {"selected_ratio": ratio, "compute_ratio": ratio, "skip_ratio": 1.0 - ratio,
                "capacity_factor": self.capacity_factor}


def _mod_select_cuda(scores: torch.Tensor, keep: int) -> torch.Tensor:
    from ..ops.functional import _L, _P, _S, _CK
    B, L = scores.shape
    if L > 8192:
        return torch.topk(scores, keep, dim=1).indices.sort(dim=1).values
    sel = torch.empty(B, keep, dtype=torch.int32, device=scores.device)
    member = torch.empty(B * L, dtype=torch.int32, device=scores.device)
    _CK(_L().ats_mod_select(_P(scores.contiguous().float()), _P(sel), _P(member), B, L, keep, _S(scores.device)), "mod_select")
    return sel


class MoDFFN(nn.Module):
    """Dense SwiGLU FFN applied only to the tokens its router selects; the rest take the residual path."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.router = MoDRouter(cfg.hidden_size, cfg.mod_capacity_factor, cfg.mod_routing_temperature)
        self.gate_up_proj = nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size))
        self.down_proj = nn.Parameter(torch.empty(cfg.hidden_size, cfg.intermediate_size))

    def forward(self, h: torch.Tensor, residual: Optional[torch.Tensor] = None, decode: bool = False):
        B, L, H = h.shape
        base = residual if residual is not None else torch.zeros_like(h)
        if decode:
            _, _, _, scores = self.router(h, decode=True)
            gate = (scores > 0).to(h.dtype).unsqueeze(-1) * torch.sigmoid(scores).to(h.dtype).unsqueeze(-1)
            y = ops.swiglu_mlp(h, self.gate_up_proj, self.down_proj)
            return base + y * gate, None
        if self.cfg.mod_per_sequence and mod_ops.kernel_path_ok(h, L):
            # training / prefill on the GPU: scores, selection, gather, weighted scatter-add and all their gradients are kernels
            r = self.router
            picked, weight, aux, sel, slot_of, _ = mod_ops.route(h, r.router.weight, r.router.bias, r.temperature, r.keep_count(L))
            y = ops.swiglu_mlp(picked, self.gate_up_proj, self.down_proj)
            with torch.no_grad():
                r.selected_tokens += float(sel.numel())
                r.total_tokens += float(B * L)
            return mod_ops.scatter(residual, y, weight, sel, slot_of, L), aux * self.cfg.mod_aux_weight
        sel, weight, aux, _ = self.router(h, per_sequence=self.cfg.mod_per_sequence)
        idx = sel.long()
        picked = torch.gather(h, 1, idx.unsqueeze(-1).expand(-1, -1, H))
        y = ops.swiglu_mlp(picked, self.gate_up_proj, self.down_proj)
        y = y * weight.to(y.dtype).unsqueeze(-1)
        out = base.scatter_add(1, idx.unsqueeze(-1).expand(-1, -1, H), y)
        return out, aux * self.cfg.mod_aux_weight


class TransformerBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, ep_size: int = 1, ep_rank: int = 0):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.input_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = GroupedQueryAttention(cfg, layer_idx)
        self.post_attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        if cfg.is_moe_layer(layer_idx):
            self.ffn: nn.Module = MoEFFNLayer(cfg, layer_idx, ep_size, ep_rank)
            self.ffn_kind = "moe"
        elif cfg.is_mod_layer(layer_idx):
            self.ffn = MoDFFN(cfg)
            self.ffn_kind = "mod"
        else:
            self.ffn = DenseSwiGLU(cfg)
            self.ffn_kind = "dense"

    def _body(self, x, rope, attention_mask, cache, positions, decode):
        h, x = self.input_norm.with_skip(x)
        x = self.self_attn(h, x, rope, attention_mask, cache, positions)
        h, x = self.post_attn_norm.with_skip(x)
        if self.ffn_kind == "mod":
            x, aux = self.ffn(h, x, decode=decode)
        else:
            x, aux = self.ffn(h, x)
        if aux is None:
            aux = x.new_zeros((), dtype=torch.float32)
        return x, aux

    def decode_step(self, x, rope, cache, h_pre=None, next_norm=None):
        """One graph-replayed decode step of this block with the norms folded into their producers: ``h_pre`` is this block's
        normalised input when the block before already produced it, ``next_norm`` = (weight, eps) of the norm that follows this
        block.  -> (x, normalised x for the next block or None)."""
        if h_pre is None:
            h, x = self.input_norm.with_skip(x)
        else:
            h = h_pre
        res = self.self_attn(h, x, rope, None, cache, None, post_norm=self.post_attn_norm)
        x, h = res if isinstance(res, tuple) else (res, None)
        if h is None:
            h, x = self.post_attn_norm.with_skip(x)
        h_next = None
        if self.ffn_kind == "moe":
            res = self.ffn(h, x, next_norm=next_norm)
            x = res[0]
            h_next = res[2] if len(res) > 2 else None
        elif self.ffn_kind == "mod":
            x, _ = self.ffn(h, x, decode=True)
        else:
            x, _ = self.ffn(h, x)
        return x, h_next

    def forward(self, x, rope, attention_mask=None, cache=None, positions=None, decode=False):
        if self.cfg.gradient_checkpointing and self.training and torch.is_grad_enabled() and cache is None:
            return checkpoint(self._body, x, rope, attention_mask, None, positions, decode, use_reentrant=False)
        return self._body(x, rope, attention_mask, cache, positions, decode)


class DeepSeekTransformer(nn.Module):
    """``forward(input_ids, attention_mask=None, return_hidden_states=False, return_aux_loss=None)`` returns
    logits, or ``(logits, total_aux_loss, aux_losses)`` for MoE / MoD models (reference ``core/model.py:1901-1973``).
    ``forward_loss`` fuses the output head with the loss and never materialises the logits."""

    def __init__(self, config: ModelConfig, ep_size: int = 1, ep_rank: int = 0):
        super().__init__()
        self.config = config
        self.ep_size, self.ep_rank = ep_size, ep_rank
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([TransformerBlock(config, i, ep_size, ep_rank) for i in range(config.num_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.rope = RotaryEmbedding(config.head_dim, config.seq_length, config.rope_theta, config.rope_scaling_factor)
        if config.tie_word_embeddings:
            self.lm_head_weight = None
        else:
            self.lm_head_weight = nn.Parameter(torch.empty(config.vocab_size, config.hidden_size))
        self.reset_parameters()
        self._register_state_dict_hook(_export_reference_names)
        self.register_load_state_dict_pre_hook(_import_reference_names)

    # -- init -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self, generator: Optional[torch.Generator] = None) -> None:
        cfg = self.config
        std = cfg.init_std
        n_layers = cfg.num_layers

        def normal_(t, s):
            t.copy_(torch.randn(t.shape, generator=generator, dtype=torch.float32,
                                device=t.device if generator is None else None).mul_(s).to(t.dtype))
        normal_(self.embed_tokens.weight, std)
        if self.lm_head_weight is not None:
            normal_(self.lm_head_weight, std)
        for l, blk in enumerate(self.layers):
            if cfg.init_mode == "scaled":  # depth-scaled init of the reference model (core/model.py:645-660, 1057-1068)
                s_qkv = std
                s_out = std / math.sqrt(2.0 * n_layers)
            else:
                s_qkv, s_out = std, std
            normal_(blk.self_attn.qkv_proj, s_qkv)
            normal_(blk.self_attn.o_proj, s_out)
            blk.input_norm.weight.fill_(1.0)
            blk.post_attn_norm.weight.fill_(1.0)
            if blk.ffn_kind == "moe":
                normal_(blk.ffn.gate.weight, std if cfg.init_mode != "scaled" else 0.01)
                # experts are drawn for the GLOBAL expert index so that every EP layout sees the same model
                e_local = blk.ffn.experts_w1.shape[0]
                for j in range(e_local):
                    normal_(blk.ffn.experts_w1[j], std)
                    normal_(blk.ffn.experts_w2[j], s_out * cfg.expert_output_scaling)
            else:
                normal_(blk.ffn.gate_up_proj, std)
                normal_(blk.ffn.down_proj, s_out)
                if blk.ffn_kind == "mod":
                    normal_(blk.ffn.router.router.weight, std)
                    blk.ffn.router.router.bias.zero_()
        self.norm.weight.fill_(1.0)

    @property
    def lm_head(self) -> torch.Tensor:
        return self.embed_tokens.weight if self.lm_head_weight is None else self.lm_head_weight

    # -- forward --------------------------------------------------------------------------------------------
    def hidden_states(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                      cache: Optional[KVCache] = None, positions: Optional[torch.Tensor] = None,
                      decode: bool = False):
        cfg = self.config
        scale = math.sqrt(cfg.hidden_size) if cfg.use_stable_embedding else 1.0
        x = ops.embedding(input_ids, self.embed_tokens.weight, scale)
        if cfg.dropout > 0 and self.training:
            x = F.dropout(x, cfg.dropout)
        aux_losses: List[torch.Tensor] = []
        if (cache is not None and cache.device_lengths is not None and input_ids.shape[1] == 1 and attention_mask is None and positions is None
                and not self.training and not torch.is_grad_enabled() and ops.serving.FUSE_DECODE):
            # graph-replayed decode step: every norm that can ride on the launch before it does (no auxiliary losses while serving)
            h_pre = None
            n = len(self.layers)
            for i, blk in enumerate(self.layers):
                nxt = self.layers[i + 1].input_norm if i + 1 < n else self.norm
                x, h_pre = blk.decode_step(x, self.rope, cache, h_pre, (nxt.weight, nxt.eps))
            return (h_pre if h_pre is not None else self.norm(x)), aux_losses
        for blk in self.layers:
            x, aux = blk(x, self.rope, attention_mask, cache, positions, decode)
            aux_losses.append(aux.float().clamp(max=1.0))
        if cache is not None and not (cache.device_lengths is not None and input_ids.shape[1] == 1):
            cache.advance(input_ids.shape[1])  # (a graph-replayed decode step advances the device-side counters instead)
        x = self.norm(x)
        return x, aux_losses

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                return_hidden_states: bool = False, return_aux_loss: Optional[bool] = None,
                cache: Optional[KVCache] = None, last_token_only: bool = False):
        x, aux_losses = self.hidden_states(input_ids, attention_mask, cache, decode=cache is not None and input_ids.shape[1] == 1)
        if last_token_only:
            x = x[:, -1:, :]
        logits = ops.linear(x, self.lm_head)
        if self.config.scale_lm_head_output:
            logits = logits / math.sqrt(self.config.hidden_size)
        has_aux = self.config.use_moe or self.config.use_mod
        want_aux = has_aux if return_aux_loss is None else return_aux_loss
        total_aux = torch.stack(aux_losses).sum() if aux_losses else logits.new_zeros(())
        if return_hidden_states:
            return (logits, x, total_aux, aux_losses) if want_aux else (logits, x)
        if want_aux:
            return logits, total_aux, aux_losses
        return logits

    def forward_loss(self, input_ids: torch.Tensor, labels: torch.Tensor, loss_weights: Optional[torch.Tensor] = None,
                     attention_mask: Optional[torch.Tensor] = None, ignore_index: int = -100) -> Dict[str, torch.Tensor]:
        """Training objective with the output head fused into the loss."""
        x, aux_losses = self.hidden_states(input_ids, attention_mask)
        loss, raw, nvalid, acc = ops.linear_cross_entropy(x, self.lm_head, labels, loss_weights, ignore_index)
        total_aux = torch.stack(aux_losses).sum() if aux_losses else loss.new_zeros(())
        return {"loss": loss + total_aux.to(loss.dtype), "lm_loss": loss, "raw_loss": raw, "aux_loss": total_aux.detach(),
                "valid_tokens": nvalid, "accuracy": acc}

    # -- statistics (reference core/model.py:1975-2264) -----------------------------------------------------
    def get_moe_layers(self) -> List[MoEFFNLayer]:
        return [b.ffn for b in self.layers if b.ffn_kind == "moe"]

    def get_mod_layers(self) -> List[MoDFFN]:
        return [b.ffn for b in self.layers if b.ffn_kind == "mod"]

    def get_routing_statistics(self, reset: bool = False) -> Dict[str, Any]:
        return {f"layer_{b.layer_idx}": b.ffn.get_routing_stats(reset) for b in self.layers if b.ffn_kind == "moe"}

    def get_mod_statistics(self) -> Dict[str, Any]:
        return {f"layer_{b.layer_idx}": b.ffn.router.get_stats() for b in self.layers if b.ffn_kind == "mod"}

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    def get_memory_footprint(self) -> Dict[str, float]:
        pbytes = sum(p.numel() * p.element_size() for p in self.parameters())
        return {"parameters_mb": pbytes / 2 ** 20, "total_parameters": float(self.num_parameters())}

    def make_cache(self, batch: int, max_len: int, dtype=None, device=None) -> KVCache:
        p = self.embed_tokens.weight
        n_kv = self.layers[0].self_attn.n_kv if len(self.layers) else self.config.num_kv_heads  # this rank's KV heads (tensor parallelism)
        return KVCache(self.config.num_layers, batch, max_len, n_kv, self.config.head_dim, dtype or p.dtype, device or p.device)


# ----------------------------------------------------------------------------------------------------------
# state-dict name translation (fused storage <-> reference checkpoint names)
# ----------------------------------------------------------------------------------------------------------
def _export_reference_names(module: DeepSeekTransformer, state: Dict[str, torch.Tensor], prefix: str, _meta) -> None:
    cfg = module.config
    for i, blk in enumerate(module.layers):
        base = f"{prefix}layers.{i}."
        nq, nk = blk.self_attn.n_q * cfg.head_dim, blk.self_attn.n_kv * cfg.head_dim  # this rank's heads under tensor parallelism
        qkv = state.pop(base + "self_attn.qkv_proj")
        state[base + "self_attn.q_proj.weight"] = qkv[:nq]
        state[base + "self_attn.k_proj.weight"] = qkv[nq:nq + nk]
        state[base + "self_attn.v_proj.weight"] = qkv[nq + nk:]
        state[base + "self_attn.o_proj.weight"] = state.pop(base + "self_attn.o_proj")
        if blk.ffn_kind == "moe":
            w1 = state.pop(base + "ffn.experts_w1")
            w2 = state.pop(base + "ffn.experts_w2")
            first = blk.ffn.ep_rank * w1.shape[0]
            for j in range(w1.shape[0]):
                state[f"{base}ffn.experts.{first + j}.gate_up_proj.weight"] = w1[j]
                state[f"{base}ffn.experts.{first + j}.down_proj.weight"] = w2[j]
        else:
            state[base + "ffn.gate_up_proj.weight"] = state.pop(base + "ffn.gate_up_proj")
            state[base + "ffn.down_proj.weight"] = state.pop(base + "ffn.down_proj")
    if module.lm_head_weight is not None:
        state[prefix + "lm_head.weight"] = state.pop(prefix + "lm_head_weight")
    else:
        state[prefix + "lm_head.weight"] = state[prefix + "embed_tokens.weight"]


def _import_reference_names(module: DeepSeekTransformer, state: Dict[str, torch.Tensor], prefix: str, *args) -> None:
    cfg = module.config
    for i, blk in enumerate(module.layers):
        base = f"{prefix}layers.{i}."
        att = blk.self_attn
        tpw, tpr = getattr(att, "tp_size", 1), getattr(att, "tp_rank", 0)

        def rows(t, full_rows):  # a full tensor loaded into a tensor-parallel model: keep this rank's rows / columns
            return t[tpr * (full_rows // tpw):(tpr + 1) * (full_rows // tpw)] if (tpw > 1 and t.shape[0] == full_rows) else t

        def cols(t, full_cols):
            return t[:, tpr * (full_cols // tpw):(tpr + 1) * (full_cols // tpw)] if (tpw > 1 and t.shape[1] == full_cols) else t
        if base + "self_attn.q_proj.weight" in state:
            q = rows(state.pop(base + "self_attn.q_proj.weight"), cfg.num_heads * cfg.head_dim)
            k = rows(state.pop(base + "self_attn.k_proj.weight"), cfg.num_kv_heads * cfg.head_dim)
            v = rows(state.pop(base + "self_attn.v_proj.weight"), cfg.num_kv_heads * cfg.head_dim)
            state[base + "self_attn.qkv_proj"] = torch.cat([q, k, v], dim=0)
        if base + "self_attn.o_proj.weight" in state:
            state[base + "self_attn.o_proj"] = cols(state.pop(base + "self_attn.o_proj.weight"), cfg.num_heads * cfg.head_dim)
        if blk.ffn_kind == "moe":
            e_local = blk.ffn.experts_w1.shape[0]
            first = blk.ffn.ep_rank * e_local
            if all(f"{base}ffn.experts.{first + j}.gate_up_proj.weight" in state for j in range(e_local)):
                state[base + "ffn.experts_w1"] = torch.stack(
                    [state[f"{base}ffn.experts.{first + j}.gate_up_proj.weight"] for j in range(e_local)])
                state[base + "ffn.experts_w2"] = torch.stack(
                    [state[f"{base}ffn.experts.{first + j}.down_proj.weight"] for j in range(e_local)])
            for key in [k_ for k_ in state if k_.startswith(base + "ffn.experts.")]:
                state.pop(key)
        else:
            if base + "ffn.gate_up_proj.weight" in state:
                gu, dn = state.pop(base + "ffn.gate_up_proj.weight"), state.pop(base + "ffn.down_proj.weight")
                ftp, ftr = getattr(blk.ffn, "tp_size", 1), getattr(blk.ffn, "tp_rank", 0)
                if ftp > 1 and gu.shape[0] == 2 * cfg.intermediate_size:
                    half, n = cfg.intermediate_size, cfg.intermediate_size // ftp
                    gu = torch.cat([gu[ftr * n:(ftr + 1) * n], gu[half + ftr * n:half + (ftr + 1) * n]], dim=0)
                    dn = dn[:, ftr * n:(ftr + 1) * n]
                state[base + "ffn.gate_up_proj"] = gu
                state[base + "ffn.down_proj"] = dn
    if prefix + "lm_head.weight" in state:
        w = state.pop(prefix + "lm_head.weight")
        if module.lm_head_weight is not None:
            state[prefix + "lm_head_weight"] = w


def estimate_parameters(cfg: ModelConfig) -> int:
    return cfg.num_parameters()

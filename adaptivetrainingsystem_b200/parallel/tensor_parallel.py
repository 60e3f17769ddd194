"""Tensor parallelism (1-D, Megatron style) with its sequence-parallel variant, and vocabulary-parallel embedding / loss.

Mechanics of the reference's vendored shardformer (``colossalai/shardformer/layer/linear.py:190-442``,
``layer/_operation.py:95-570``, ``layer/embedding.py:381-395``, ``layer/loss.py:17-131``): column-parallel linear
(identity forward / all-reduce of the input gradient), row-parallel linear (all-reduce of the output, or
reduce-scatter along the sequence with ``sequence_parallel``), all-gather of sequence shards before the column
linear; vocabulary-parallel embedding masks foreign ids and all-reduces; vocabulary-parallel cross-entropy needs three
all-reduces of ``[tokens]`` vectors (row max, target logit, sum of exponentials)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops


def _size(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


class _CopyToRegion(torch.autograd.Function):
    """identity forward, all-reduce backward"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _size(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRegion(torch.autograd.Function):
    """all-reduce forward, identity backward"""

    @staticmethod
    def forward(ctx, x, group):
        if _size(group) > 1:
            x = x.contiguous()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherSeq(torch.autograd.Function):
    """all-gather along the sequence dim forward, reduce-scatter backward (sequence-parallel entry of a column linear)"""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        w = _size(group)
        if w == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(w)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    @staticmethod
    def backward(ctx, g):
        w = _size(ctx.group)
        if w == 1:
            return g, None, None
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g.chunk(w, dim=ctx.dim)[_rank(ctx.group)].contiguous(), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    """reduce-scatter along the sequence dim forward, all-gather backward (sequence-parallel exit of a row linear)"""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        w = _size(group)
        if w == 1:
            return x
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x.chunk(w, dim=dim)[_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, g):
        w = _size(ctx.group)
        if w == 1:
            return g, None, None
        parts = [torch.empty_like(g) for _ in range(w)]
        dist.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=ctx.dim), None, None


class ColumnParallelLinear(nn.Module):
    """y_local = x @ W_local^T with W split along the output dimension."""

    def __init__(self, in_features: int, out_features: int, group=None, sequence_parallel: bool = False, gather_output: bool = False):
        super().__init__()
        self.group, self.sp, self.gather_output = group, sequence_parallel, gather_output
        w = _size(group)
        assert out_features % w == 0
        self.weight = nn.Parameter(torch.empty(out_features // w, in_features))
        nn.init.normal_(self.weight, std=0.02)

    @classmethod
    def from_full(cls, full_weight: torch.Tensor, group=None, **kw) -> "ColumnParallelLinear":
        m = cls(full_weight.shape[1], full_weight.shape[0], group, **kw)
        m.weight.data.copy_(full_weight.chunk(_size(group), dim=0)[_rank(group)])
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = _GatherSeq.apply(x, self.group, 1) if self.sp else _CopyToRegion.apply(x, self.group)
        y = ops.linear(x, self.weight)
        if self.gather_output and _size(self.group) > 1:
            parts = [torch.empty_like(y) for _ in range(_size(self.group))]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            parts[_rank(self.group)] = y
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    """y = sum over ranks of x_local @ W_local^T with W split along the input dimension."""

    def __init__(self, in_features: int, out_features: int, group=None, sequence_parallel: bool = False):
        super().__init__()
        self.group, self.sp = group, sequence_parallel
        w = _size(group)
        assert in_features % w == 0
        self.weight = nn.Parameter(torch.empty(out_features, in_features // w))
        nn.init.normal_(self.weight, std=0.02)

    @classmethod
    def from_full(cls, full_weight: torch.Tensor, group=None, **kw) -> "RowParallelLinear":
        m = cls(full_weight.shape[1], full_weight.shape[0], group, **kw)
        m.weight.data.copy_(full_weight.chunk(_size(group), dim=1)[_rank(group)])
        return m

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        y = ops.linear(x_local, self.weight)
        return _ReduceScatterSeq.apply(y, self.group, 1) if self.sp else _ReduceFromRegion.apply(y, self.group)


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab: int, hidden: int, group=None):
        super().__init__()
        self.group = group
        w, r = _size(group), _rank(group)
        assert vocab % w == 0
        self.per = vocab // w
        self.lo = r * self.per
        self.weight = nn.Parameter(torch.empty(self.per, hidden))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        local = ids - self.lo
        mine = (local >= 0) & (local < self.per)
        out = torch.nn.functional.embedding(local.clamp(0, self.per - 1), self.weight) * mine.unsqueeze(-1).to(self.weight.dtype)
        return _ReduceFromRegion.apply(out, self.group)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_local, labels, group, ignore_index):
        w, r = _size(group), _rank(group)
        per = logits_local.shape[-1]
        lg = logits_local.float()
        mx = lg.max(-1).values
        if w > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        lg = lg - mx.unsqueeze(-1)
        local = labels - r * per
        mine = (local >= 0) & (local < per)
        tgt = torch.gather(lg, -1, local.clamp(0, per - 1).unsqueeze(-1)).squeeze(-1) * mine
        se = lg.exp().sum(-1)
        if w > 1:
            dist.all_reduce(tgt, group=group)
            dist.all_reduce(se, group=group)
        valid = labels != ignore_index
        loss_tok = (se.log() - tgt) * valid
        n = valid.sum().clamp(min=1)
        ctx.save_for_backward(lg.exp() / se.unsqueeze(-1), local, mine & valid, valid, n)
        return loss_tok.sum() / n

    @staticmethod
    def backward(ctx, g):
        sm, local, hit, valid, n = ctx.saved_tensors
        grad = sm * valid.unsqueeze(-1)
        idx = local.clamp(0, sm.shape[-1] - 1).unsqueeze(-1)
        grad.scatter_add_(-1, idx, -hit.unsqueeze(-1).to(grad.dtype))
        return (grad * (g / n)).to(sm.dtype), None, None, None


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, labels: torch.Tensor, group=None, ignore_index: int = -100) -> torch.Tensor:
    """Mean next-token loss when the vocabulary dimension of ``logits_local`` is split over ``group``."""
    return _VocabParallelCE.apply(logits_local.reshape(-1, logits_local.shape[-1]), labels.reshape(-1), group, ignore_index)

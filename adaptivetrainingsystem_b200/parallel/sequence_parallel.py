"""Sequence (context) parallelism by head scatter: every rank holds ``L / W`` tokens of each sequence; before attention an
all-to-all turns ``[B, L/W, H, D]`` into ``[B, L, H/W, D]`` (all tokens, a slice of the heads) and the inverse follows
(the "all_to_all" / DeepSpeed-Ulysses mode of the reference's vendored tree, ``colossalai/shardformer/layer/_operation.py:778-935``,
``shardformer/modeling/llama.py:503-540``).  On NVSwitch an all-to-all costs the same to every peer, so this is the
long-context option; ring attention is not needed for the sequence lengths of the benchmark configs."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    w = dist.get_world_size(group) if dist.is_initialized() else 1
    if w == 1:
        return x
    send = torch.stack([t.contiguous() for t in x.chunk(w, dim=scatter_dim)])  # [W, ...]: slice i goes to rank i
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return torch.cat(list(recv.unbind(0)), dim=gather_dim)


class _SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group):
        ctx.dims, ctx.group = (scatter_dim, gather_dim), group
        return _a2a(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        s, ga = ctx.dims
        return _a2a(g, ga, s, ctx.group), None, None, None


def scatter_heads_gather_sequence(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, L/W, H, D] -> [B, L, H/W, D]"""
    return _SeqAllToAll.apply(x, 2, 1, group)


def scatter_sequence_gather_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, L, H/W, D] -> [B, L/W, H, D]"""
    return _SeqAllToAll.apply(x, 1, 2, group)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None) -> torch.Tensor:
    """Causal attention over a sequence split across ``group``; q [B, L/W, Hq, D], k/v [B, L/W, Hkv, D]
    (Hq and Hkv divisible by W)."""
    from .. import ops
    qf, kf, vf = (scatter_heads_gather_sequence(t, group) for t in (q, k, v))
    o = ops.attention(qf, kf, vf, causal=True)
    return scatter_sequence_gather_heads(o, group)

"""Ring-decomposed sequence / context parallelism: collectives cut into ``world - 1`` neighbour exchanges so that the
partial result of the chunk already present is computed while the next chunk is in flight.

* :func:`ring_allgather_linear` / :func:`linear_ring_reducescatter`: the "ring" sequence-parallel mode of the reference's
  vendored tree (``colossalai/shardformer/layer/_operation.py:170-221`` ring as all-gather in front of a column-parallel
  linear, ``:404-459`` ring as reduce-scatter behind a row-parallel linear).
* :func:`ring_attention`: context-parallel causal attention, K / V shards circulating around the ring (vendored legacy
  ``colossalai/legacy/nn/layer/parallel_sequence/_operation.py:15-160`` ``RingQK`` / ``RingAV``).  Unlike that code it never
  materialises the ``[L/p, L]`` score rows: every step produces an (output, log-sum-exp) pair for one K / V chunk and the
  pairs are merged online; chunks that lie entirely in the causal future are skipped.

Each step posts its send and receive as one grouped exchange (``batch_isend_irecv``), computes, then waits.  On NVSwitch
a ring has no bandwidth advantage over an all-to-all; these paths exist for feature parity and for topologies without a
switch, the head-scatter form in ``sequence_parallel.py`` is the default for long context.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def _info(group) -> Tuple[int, int, List[int]]:
    if not dist.is_initialized():
        return 1, 0, [0]
    return dist.get_world_size(group), dist.get_rank(group), dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))


def _exchange(send: torch.Tensor, recv: torch.Tensor, dst: int, src: int, group):
    ops_ = [dist.P2POp(dist.isend, send, dst, group), dist.P2POp(dist.irecv, recv, src, group)]
    return dist.batch_isend_irecv(ops_)


# ------------------------------------------------------------------------------------------------------- linear layers
class _RingAllGatherLinear(torch.autograd.Function):
    """y = allgather_seq(x) @ w^T, x [L/p, K] per rank -> y [L, N_local]."""

    @staticmethod
    def forward(ctx, x, w, group):
        W, r, ranks = _info(group)
        Lc = x.shape[0]
        y = x.new_empty(Lc * W, w.shape[0])
        cur = x.contiguous()
        ctx.save_for_backward(x, w)
        ctx.group = group
        for s in range(W):
            owner = (r - s) % W  # whose chunk `cur` is
            reqs = None
            if s + 1 < W:
                nxt = torch.empty_like(cur)
                reqs = _exchange(cur, nxt, ranks[(r + 1) % W], ranks[(r - 1) % W], group)
            y[owner * Lc:(owner + 1) * Lc] = cur @ w.t()  # overlaps the transfer of the next chunk
            if reqs is not None:
                for q in reqs:
                    q.wait()
                cur = nxt
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group = ctx.group
        W, r, ranks = _info(group)
        Lc = x.shape[0]
        # dx = reduce_scatter_seq(dy @ w): partial sums travel around the ring, each rank adds its contribution to the chunk
        # that is passing through; dw needs the gathered x again (second ring pass, overlapped the same way)
        acc = None
        for s in range(W):
            chunk = (r - s - 1) % W
            part = dy[chunk * Lc:(chunk + 1) * Lc] @ w
            acc = part if acc is None else acc + part
            if s + 1 < W:
                nxt = torch.empty_like(acc)
                for q in _exchange(acc.contiguous(), nxt, ranks[(r + 1) % W], ranks[(r - 1) % W], group):
                    q.wait()
                acc = nxt
        dx = acc
        dw = torch.zeros_like(w)
        cur = x.contiguous()
        for s in range(W):
            owner = (r - s) % W
            reqs = None
            if s + 1 < W:
                nxt = torch.empty_like(cur)
                reqs = _exchange(cur, nxt, ranks[(r + 1) % W], ranks[(r - 1) % W], group)
            dw += dy[owner * Lc:(owner + 1) * Lc].t() @ cur
            if reqs is not None:
                for q in reqs:
                    q.wait()
                cur = nxt
        return dx, dw, None


def ring_allgather_linear(x: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    """Column-parallel linear on a sequence-sharded input: x [L/p, K], w [N_local, K] -> [L, N_local]."""
    return _RingAllGatherLinear.apply(x, w, group)


class _LinearRingReduceScatter(torch.autograd.Function):
    """y = reduce_scatter_seq(x @ w^T), x [L, K_local] per rank -> y [L/p, N]."""

    @staticmethod
    def forward(ctx, x, w, group):
        W, r, ranks = _info(group)
        Lc = x.shape[0] // W
        ctx.save_for_backward(x, w)
        ctx.group = group
        acc = None
        for s in range(W):
            chunk = (r - s - 1) % W
            part = x[chunk * Lc:(chunk + 1) * Lc] @ w.t()
            acc = part if acc is None else acc + part
            if s + 1 < W:
                nxt = torch.empty_like(acc)
                for q in _exchange(acc.contiguous(), nxt, ranks[(r + 1) % W], ranks[(r - 1) % W], group):
                    q.wait()
                acc = nxt
        return acc

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group = ctx.group
        W, r, ranks = _info(group)
        Lc = dy.shape[0]
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w)
        cur = dy.contiguous()
        for s in range(W):
            owner = (r - s) % W
            reqs = None
            if s + 1 < W:
                nxt = torch.empty_like(cur)
                reqs = _exchange(cur, nxt, ranks[(r + 1) % W], ranks[(r - 1) % W], group)
            dx[owner * Lc:(owner + 1) * Lc] = cur @ w
            dw += cur.t() @ x[owner * Lc:(owner + 1) * Lc]
            if reqs is not None:
                for q in reqs:
                    q.wait()
                cur = nxt
        return dx, dw, None


def linear_ring_reducescatter(x: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    """Row-parallel linear whose output goes back to sequence shards: x [L, K_local], w [N, K_local] -> [L/p, N]."""
    return _LinearRingReduceScatter.apply(x, w, group)


# ------------------------------------------------------------------------------------------------------- ring attention
def _block_attention(q, k, v, causal: bool):
    """q [B, Lq, Hq, D], k / v [B, Lk, Hkv, D] -> (out fp32 [B, Lq, Hq, D], lse fp32 [B, Hq, Lq]); causal = same-offset diagonal."""
    B, Lq, Hq, D = q.shape
    Lk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3).reshape(B, Hkv, rep, Lq, D)
    kf, vf = k.float().permute(0, 2, 1, 3), v.float().permute(0, 2, 1, 3)
    s = torch.einsum("bgrqd,bgkd->bgrqk", qf, kf) / math.sqrt(D)
    if causal:
        mask = torch.arange(Lk, device=q.device)[None, :] > torch.arange(Lq, device=q.device)[:, None]
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bgrqk,bgkd->bgrqd", torch.exp(s - lse.unsqueeze(-1)), vf)
    return o.reshape(B, Hq, Lq, D).permute(0, 2, 1, 3), lse.reshape(B, Hq, Lq)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None) -> torch.Tensor:
    """Causal attention over a sequence split in contiguous chunks across ``group`` (rank r holds chunk r):
    q [B, L/p, Hq, D], k / v [B, L/p, Hkv, D] -> [B, L/p, Hq, D].  Differentiable (the exchange is replayed in reverse by
    autograd through the send / receive pair below)."""
    W, r, ranks = _info(group)
    if W == 1:
        o, _ = _block_attention(q, k, v, True)
        return o.to(q.dtype)
    out = None
    lse = None
    kv = torch.stack([k, v]).contiguous()
    for s in range(W):
        owner = (r - s) % W
        nxt = _RingShift.apply(kv, group) if s + 1 < W else None  # posts the exchange; autograd routes the gradient back
        if owner <= r:  # chunks from the causal future contribute nothing
            o_s, l_s = _block_attention(q, kv[0], kv[1], causal=(owner == r))
            if out is None:
                out, lse = o_s, l_s
            else:
                new = torch.logaddexp(lse, l_s)
                out = out * torch.exp(lse - new).permute(0, 2, 1).unsqueeze(-1) + o_s * torch.exp(l_s - new).permute(0, 2, 1).unsqueeze(-1)
                lse = new
        elif out is not None:
            # a chunk from the causal future is not used, but every rank must replay every exchange in the backward pass:
            # tie the unused chunk into the graph with a zero gradient
            out = _Tie.apply(out, kv)
        if nxt is not None:
            kv = nxt
    return out.to(q.dtype)


class _Tie(torch.autograd.Function):
    """Identity on ``x`` that makes ``other`` part of the autograd graph (its gradient is zero)."""

    @staticmethod
    def forward(ctx, x, other):
        ctx.shape, ctx.dtype = other.shape, other.dtype
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g, torch.zeros(ctx.shape, dtype=ctx.dtype, device=g.device)


class _RingShift(torch.autograd.Function):
    """Send a tensor to the next rank of the ring and return what the previous rank sent; the gradient goes the other way."""

    @staticmethod
    def forward(ctx, x, group):
        W, r, ranks = _info(group)
        ctx.group = group
        recv = torch.empty_like(x)
        for q in _exchange(x.contiguous(), recv, ranks[(r + 1) % W], ranks[(r - 1) % W], group):
            q.wait()
        return recv

    @staticmethod
    def backward(ctx, g):
        W, r, ranks = _info(ctx.group)
        recv = torch.empty_like(g)
        for q in _exchange(g.contiguous(), recv, ranks[(r - 1) % W], ranks[(r + 1) % W], ctx.group):
            q.wait()
        return recv, None

"""Pipeline parallelism: stage partition of the decoder, fixed-shape activation send/recv on NCCL (or Gloo) p2p and the
1F1B schedule.

What the reference's vendored tree does (``colossalai/pipeline/schedule/one_f_one_b.py:28-453``, ``pipeline/p2p.py:208-688``)
with pickled metadata per message is done here with a fixed wire format: every message between adjacent stages is one
``[micro_batch, seq, hidden]`` tensor in the compute dtype, so nothing is pickled on the hot path.  Schedule:
``warmup = stages - stage - 1`` forwards, then steady 1F1B, then ``warmup`` cooldown backwards; the last stage scales
the loss by ``1 / num_microbatches``; in the steady state a stage posts "send activation" and "receive gradient" as one
grouped exchange so neighbours never wait on each other.  ``InterleavedSchedule`` runs several model chunks per rank in the
interleaved 1F1B order.  A stage frees the weights of every other stage (``free_foreign_parameters``).
Pipeline send/recv stays on the collective library by design (compute and transfer overlap through the schedule).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def free_foreign_parameters(model, keep_layers, keep_embedding: bool, keep_head: bool) -> int:
    """A pipeline stage holds only what it runs: the weights of every other stage are released (their tensors become empty and
    stop requiring gradients), so the memory of a stage is its share of the model.  Returns the number of elements released."""
    freed = 0
    dev = next(model.parameters()).device

    def drop(p):
        nonlocal freed
        freed += p.numel()
        p.requires_grad_(False)
        p.data = torch.empty(0, dtype=p.dtype, device=dev)
    for i, blk in enumerate(model.layers):
        if i not in keep_layers:
            for p in blk.parameters():
                drop(p)
    tied = model.lm_head_weight is None
    if not keep_embedding and not (tied and keep_head):
        drop(model.embed_tokens.weight)
    if not keep_head:
        drop(model.norm.weight)
        if model.lm_head_weight is not None:
            drop(model.lm_head_weight)
    return freed


def partition_layers(num_layers: int, num_stages: int) -> List[Tuple[int, int]]:
    """Contiguous [start, end) ranges, remainders given to the earliest stages."""
    base, rem = divmod(num_layers, num_stages)
    out, s = [], 0
    for i in range(num_stages):
        n = base + (1 if i < rem else 0)
        out.append((s, s + n))
        s += n
    return out


class PipelineStage(nn.Module):
    """The slice of a ``DeepSeekTransformer`` owned by one stage: embedding on the first, final norm + head on the last."""

    def __init__(self, model, stage: int, num_stages: int):
        super().__init__()
        self.stage, self.num_stages = stage, num_stages
        self.start, self.end = partition_layers(len(model.layers), num_stages)[stage]
        self.model = model
        self.is_first, self.is_last = stage == 0, stage == num_stages - 1
        # parameters of foreign stages neither train nor live here
        self.freed = free_foreign_parameters(model, set(range(self.start, self.end)), self.is_first, self.is_last)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: token ids on the first stage, hidden states otherwise -> (hidden or final hidden, aux loss)."""
        m = self.model
        if self.is_first:
            import math
            from .. import ops
            x = ops.embedding(x, m.embed_tokens.weight, math.sqrt(m.config.hidden_size) if m.config.use_stable_embedding else 1.0)
        aux = x.new_zeros((), dtype=torch.float32)
        for blk in m.layers[self.start:self.end]:
            x, a = blk(x, m.rope)
            aux = aux + a.float().clamp(max=1.0)
        if self.is_last:
            x = m.norm(x)
        return x, aux

    def loss(self, hidden: torch.Tensor, labels: torch.Tensor, weights=None):
        from .. import ops
        return ops.linear_cross_entropy(hidden, self.model.lm_head, labels, weights)[0]


class OneFOneBSchedule:
    def __init__(self, stage_module: PipelineStage, group, num_microbatches: int, act_shape: Tuple[int, int, int],
                 dtype: torch.dtype, device: torch.device):
        self.m, self.group, self.n = stage_module, group, num_microbatches
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if num_microbatches < self.world:
            raise ValueError("1F1B needs num_microbatches >= pipeline stages")
        self.shape, self.dtype, self.device = act_shape, dtype, device
        self.ranks = dist.get_process_group_ranks(group)

    def _peer(self, delta: int) -> int:
        return self.ranks[self.rank + delta]

    def _send(self, t: torch.Tensor, delta: int) -> None:
        dist.send(t.contiguous(), self._peer(delta), group=self.group)

    def _recv(self, delta: int) -> torch.Tensor:
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        dist.recv(buf, self._peer(delta), group=self.group)
        return buf

    def run(self, microbatches: List[Dict[str, torch.Tensor]]) -> Optional[torch.Tensor]:
        """One optimiser step's worth of micro-batches; gradients accumulate in the stage's parameters.
        Returns the mean loss on the last stage, ``None`` elsewhere."""
        m, n, s, S = self.m, self.n, self.rank, self.world
        warmup = min(S - s - 1, n)
        inputs: List[Optional[torch.Tensor]] = []
        outputs: List[torch.Tensor] = []
        losses: List[torch.Tensor] = []
        fwd_i = bwd_i = 0

        def forward_one(fused_exchange: bool) -> Optional[torch.Tensor]:
            """Forward of the next micro-batch.  In the steady state the activation send to the next stage and the
            receive of the gradient the next backward needs are posted as ONE grouped exchange: two neighbours that
            each sent first would otherwise wait on each other forever."""
            nonlocal fwd_i
            mb = microbatches[fwd_i]
            grad_in = None
            if m.is_first:
                x_in = None
                out, aux = m(mb["input_ids"])
            else:
                x_in = self._recv(-1).requires_grad_()
                out, aux = m(x_in)
            if m.is_last:
                loss = (m.loss(out, mb["labels"], mb.get("loss_weights")) + aux) / n
                losses.append(loss.detach())
                out = loss
            elif fused_exchange:
                grad_in = torch.empty(self.shape, dtype=self.dtype, device=self.device)
                ops_ = [dist.P2POp(dist.isend, out.detach().contiguous(), self._peer(+1), self.group),
                        dist.P2POp(dist.irecv, grad_in, self._peer(+1), self.group)]
                for r in dist.batch_isend_irecv(ops_):
                    r.wait()
            else:
                self._send(out.detach(), +1)
            inputs.append(x_in)
            outputs.append((out, aux))
            fwd_i += 1
            return grad_in

        def backward_one(grad_in: Optional[torch.Tensor] = None):
            nonlocal bwd_i
            out, aux = outputs[bwd_i]
            x_in = inputs[bwd_i]
            if m.is_last:
                out.backward()
            else:
                g = grad_in if grad_in is not None else self._recv(+1)
                if aux.requires_grad:  # MoE / MoD stages add their own auxiliary loss
                    torch.autograd.backward([out, aux / n], [g, torch.ones_like(aux)])
                else:
                    out.backward(g)
            if not m.is_first:
                self._send(x_in.grad, -1)
            outputs[bwd_i] = None
            inputs[bwd_i] = None
            bwd_i += 1

        for _ in range(warmup):
            forward_one(False)
        for _ in range(n - warmup):
            backward_one(forward_one(True))
        for _ in range(warmup):
            backward_one()
        if m.is_last:
            return torch.stack(losses).sum()
        return None


class InterleavedStages(nn.Module):
    """``chunks`` model chunks per rank: virtual stage ``k = c * stages + rank`` owns a contiguous slice of the decoder
    (virtual pipeline of ``stages * chunks`` stages, the placement of the reference's vendored interleaved schedule,
    ``colossalai/pipeline/schedule/interleaved_pp.py``)."""

    def __init__(self, model, rank: int, num_stages: int, chunks: int):
        super().__init__()
        self.model, self.rank, self.num_stages, self.chunks = model, rank, num_stages, chunks
        total = num_stages * chunks
        parts = partition_layers(len(model.layers), total)
        self.ranges = [parts[c * num_stages + rank] for c in range(chunks)]
        self.virtual = [c * num_stages + rank for c in range(chunks)]
        self.total = total
        keep = {i for (a, b) in self.ranges for i in range(a, b)}
        self.freed = free_foreign_parameters(model, keep, 0 in self.virtual, total - 1 in self.virtual)

    def forward_chunk(self, c: int, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        m = self.model
        k = self.virtual[c]
        if k == 0:
            import math
            from .. import ops
            x = ops.embedding(x, m.embed_tokens.weight, math.sqrt(m.config.hidden_size) if m.config.use_stable_embedding else 1.0)
        aux = x.new_zeros((), dtype=torch.float32)
        a, b = self.ranges[c]
        for blk in m.layers[a:b]:
            x, al = blk(x, m.rope)
            aux = aux + al.float().clamp(max=1.0)
        if k == self.total - 1:
            x = m.norm(x)
        return x, aux

    def loss(self, hidden: torch.Tensor, labels: torch.Tensor, weights=None):
        from .. import ops
        return ops.linear_cross_entropy(hidden, self.model.lm_head, labels, weights)[0]


def interleaved_order(stage: int, num_stages: int, chunks: int, num_microbatches: int) -> List[Tuple[str, int, int]]:
    """The interleaved 1F1B order of one rank: a list of ``("F" | "B", chunk, micro-batch)``.

    Work comes in groups of ``stages`` micro-batches per chunk (so ``num_microbatches`` must be a multiple of ``stages``):
    forward operation ``k`` runs chunk ``(k // stages) % chunks`` on micro-batch ``(k // (stages * chunks)) * stages + k % stages``;
    backward operations walk the chunks in reverse.  A rank starts with
    ``2 * (stages - stage - 1) + (chunks - 1) * stages`` forwards, then alternates one forward with one backward, then
    drains the remaining backwards (reference: ``colossalai/pipeline/schedule/interleaved_pp.py:406-470``)."""
    S, C, n = num_stages, chunks, num_microbatches
    if n % S:
        raise ValueError("interleaved 1F1B needs num_microbatches to be a multiple of the pipeline stages")
    total = n * C

    def fwd(k):
        return ("F", (k // S) % C, (k // (S * C)) * S + k % S)

    def bwd(k):
        return ("B", C - 1 - (k // S) % C, (k // (S * C)) * S + k % S)
    warm = min(2 * (S - stage - 1) + (C - 1) * S, total)
    order = [fwd(k) for k in range(warm)]
    for i in range(total - warm):
        order.append(fwd(warm + i))
        order.append(bwd(i))
    order += [bwd(k) for k in range(total - warm, total)]
    return order


class InterleavedSchedule:
    """Interleaved 1F1B over the virtual pipeline of :class:`InterleavedStages`.

    Every directed link between neighbouring ranks (forward activations ``r -> r + 1``, gradients ``r + 1 -> r``, both around
    the ring) gets a communicator of its own, so traffic on one link never queues behind traffic on another.  On every link the
    sender's production order equals the receiver's consumption order (both follow :func:`interleaved_order`), sends are
    posted asynchronously and a receive is posted right before the operation that needs it; with ``stages`` ranks at most
    ``warm-up`` activations per chunk are alive on a rank, not all ``num_microbatches``."""

    def __init__(self, stages: InterleavedStages, group, num_microbatches: int, act_shape: Tuple[int, int, int], dtype, device):
        self.m, self.group, self.n = stages, group, num_microbatches
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.ranks = dist.get_process_group_ranks(group)
        self.shape, self.dtype, self.device = act_shape, dtype, device
        self.order = interleaved_order(self.rank, self.world, stages.chunks, num_microbatches)
        # one communicator per directed link and kind of traffic (created in the same order on every rank of the pipeline group)
        self.link: Dict[Tuple[int, int, str], object] = {}
        S = self.world
        for src in range(S):
            for dst, kind in (((src + 1) % S, "act"), ((src - 1) % S, "grad")):
                if src != dst:
                    self.link[(src, dst, kind)] = dist.new_group([self.ranks[src], self.ranks[dst]])

    def _isend(self, t: torch.Tensor, dst: int, kind: str):
        return dist.isend(t, self.ranks[dst], group=self.link[(self.rank, dst, kind)])

    def _recv(self, src: int, kind: str) -> torch.Tensor:
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        dist.recv(buf, self.ranks[src], group=self.link[(src, self.rank, kind)])
        return buf

    def run(self, microbatches: List[Dict[str, torch.Tensor]]) -> Optional[torch.Tensor]:
        m, n, S, r = self.m, self.n, self.world, self.rank
        nxt, prv = (r + 1) % S, (r - 1) % S
        saved: Dict[Tuple[int, int], Tuple[Optional[torch.Tensor], torch.Tensor, torch.Tensor]] = {}
        losses: List[torch.Tensor] = []
        pending, keep_alive = [], []
        self.max_alive = 0
        for kind, c, i in self.order:
            k = m.virtual[c]
            mb = microbatches[i]
            if kind == "F":
                if k == 0:
                    x_in = None
                    out, aux = m.forward_chunk(c, mb["input_ids"])
                else:
                    x_in = self._recv(prv, "act").requires_grad_()
                    out, aux = m.forward_chunk(c, x_in)
                if k == m.total - 1:
                    loss = (m.loss(out, mb["labels"], mb.get("loss_weights")) + aux) / n
                    losses.append(loss.detach())
                    out = loss
                else:
                    act = out.detach().contiguous()
                    keep_alive.append(act)
                    pending.append(self._isend(act, nxt, "act"))
                saved[(c, i)] = (x_in, out, aux)
                self.max_alive = max(self.max_alive, len(saved))
            else:
                x_in, out, aux = saved.pop((c, i))
                if k == m.total - 1:
                    out.backward()
                else:
                    g = self._recv(nxt, "grad")
                    if aux.requires_grad:
                        torch.autograd.backward([out, aux / n], [g, torch.ones_like(aux)])
                    else:
                        out.backward(g)
                if k != 0:
                    gin = x_in.grad.contiguous()
                    keep_alive.append(gin)
                    pending.append(self._isend(gin, prv, "grad"))
        for h in pending:
            h.wait()
        if m.total - 1 in m.virtual:
            return torch.stack(losses).sum()
        return None

"""Pipeline parallelism: stage partition of the decoder, fixed-shape activation send/recv on NCCL (or Gloo) p2p and the
1F1B schedule.

What the reference's vendored tree does (``colossalai/pipeline/schedule/one_f_one_b.py:28-453``, ``pipeline/p2p.py:208-688``)
with pickled metadata per message is done here with a fixed wire format: every message between adjacent stages is one
``[micro_batch, seq, hidden]`` tensor in the compute dtype, so nothing is pickled on the hot path.  Schedule:
``warmup = stages - stage - 1`` forwards, then steady 1F1B, then ``warmup`` cooldown backwards; the last stage scales
the loss by ``1 / num_microbatches``; in the steady state a stage posts "send activation" and "receive gradient" as one
grouped exchange so neighbours never wait on each other.
Pipeline send/recv stays on the collective library by design (compute and transfer overlap through the schedule).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


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
        keep = set(range(self.start, self.end))
        for i, blk in enumerate(model.layers):  # parameters of foreign stages do not train here
            if i not in keep:
                for p in blk.parameters():
                    p.requires_grad_(False)
        if not self.is_first:
            model.embed_tokens.weight.requires_grad_(False)
        if not self.is_last:
            model.norm.weight.requires_grad_(False)
            if model.lm_head_weight is not None:
                model.lm_head_weight.requires_grad_(False)

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

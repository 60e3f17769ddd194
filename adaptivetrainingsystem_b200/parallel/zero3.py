"""ZeRO stage 3: parameters, gradients and optimiser state are all partitioned; a transformer block's parameters exist in
full only while that block runs.

Each block is one *unit* (the FSDP wrapping unit / Gemini chunk of the reference's backends, ``backend/backend_fsdp.py:151-198``,
``colossalai/zero/gemini/chunk/chunk.py:58-650``): its parameters are packed into one flat range of which every rank keeps
a ``1/W`` shard (bf16 shard + fp32 master / moments).  Hooks gather the unit's flat buffer right before its forward and
again before its backward (the next unit is prefetched on a side stream), point the parameters into it, and release it
afterwards; the unit's gradient buffer is reduce-scattered into the gradient shard as soon as its backward finishes,
overlapping with the backward of the unit below.  Embedding, final norm and head form a root unit that stays gathered
(like FSDP's root).  The optimiser step touches shards only; no all-gather follows it.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from .bootstrap import ProcessMesh
from .zero import NO_DECAY_KEYS, _pad_to


class Unit:
    def __init__(self, name: str, module: Optional[nn.Module], params: List[Tuple[str, nn.Parameter]], group, W: int, r: int,
                 dtype, device, resident: bool):
        self.name, self.module, self.group, self.W, self.r, self.resident = name, module, group, W, r, resident
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.shapes = [p.shape for p in self.params]
        self.decay_mask_needed = True
        offs, total = [], 0
        for p in self.params:
            offs.append(total)
            total += _pad_to(p.numel(), 8)
        self.offsets, self.padded = offs, _pad_to(max(total, 8), W * 8)
        self.shard = self.padded // W
        full = torch.zeros(self.padded, dtype=dtype, device=device)
        for p, o in zip(self.params, offs):
            full[o:o + p.numel()].copy_(p.data.reshape(-1))
        lo, hi = r * self.shard, (r + 1) * self.shard
        self.param_shard = full[lo:hi].clone()
        self.grad_shard = torch.zeros_like(self.param_shard)
        self.master = self.param_shard.float()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        # per-element weight-decay multiplier of the owned slice (units mix decayed and non-decayed parameters)
        wd = torch.zeros(self.padded, dtype=torch.float32, device=device)
        for n, p, o in zip(self.names, self.params, offs):
            if not (p.ndim < 2 or any(k in n.lower() for k in NO_DECAY_KEYS)):
                wd[o:o + p.numel()] = 1.0
        self.wd_mask = wd[lo:hi].clone()
        self.full: Optional[torch.Tensor] = None
        self.full_grad: Optional[torch.Tensor] = None
        self.grad_fresh = True
        self.dtype, self.device = dtype, device
        if resident:
            self._attach(full)
        else:
            self._detach()

    def _attach(self, full: torch.Tensor) -> None:
        self.full = full
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            p.data = full[o:o + shp.numel()].view(shp)

    def _detach(self) -> None:
        self.full = None
        for p in self.params:
            p.data = torch.empty(0, dtype=self.dtype, device=self.device)

    def gather(self) -> None:
        if self.full is not None:
            return
        full = torch.empty(self.padded, dtype=self.dtype, device=self.device)
        if self.W == 1 or not dist.is_initialized():
            full.copy_(self.param_shard)
        elif dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(self.param_shard) for _ in range(self.W)]
            dist.all_gather(parts, self.param_shard, group=self.group)
            torch.cat(parts, out=full)
        else:
            dist.all_gather_into_tensor(full, self.param_shard, group=self.group)
        self._attach(full)

    def release(self) -> None:
        if not self.resident and self.full is not None:
            self._detach()

    def open_grads(self) -> None:
        """Full-size gradient buffer for this unit's backward; weight-gradient kernels write straight into it."""
        if self.full_grad is None:
            self.full_grad = torch.zeros(self.padded, dtype=self.dtype, device=self.device)
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            p._ats_grad = self.full_grad[o:o + shp.numel()]
            p._ats_grad_fresh = True
            p.grad = None

    def reduce_grads(self) -> None:
        """Fold autograd-delivered gradients in, reduce-scatter, accumulate into the gradient shard, drop the buffer."""
        if self.full_grad is None:
            return
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            sink = self.full_grad[o:o + shp.numel()]
            if p.grad is not None:
                if getattr(p, "_ats_grad_fresh", True):
                    sink.copy_(p.grad.reshape(-1))
                else:
                    sink.add_(p.grad.reshape(-1).to(sink.dtype))
                p.grad = None
        lo, hi = self.r * self.shard, (self.r + 1) * self.shard
        if self.W > 1 and dist.is_initialized():
            if dist.get_backend(self.group) == "gloo":
                dist.all_reduce(self.full_grad, group=self.group)
                red = self.full_grad[lo:hi]
            else:
                red = torch.empty_like(self.grad_shard)
                dist.reduce_scatter_tensor(red, self.full_grad, group=self.group)
        else:
            red = self.full_grad[lo:hi]
        if self.grad_fresh:
            self.grad_shard.copy_(red)
            self.grad_fresh = False
        else:
            self.grad_shard.add_(red)
        if not self.resident:
            self.full_grad = None
        else:
            self.full_grad.zero_()


class ZeRO3Engine:
    """Same surface as :class:`~adaptivetrainingsystem_b200.parallel.zero.ShardedEngine` (``step``, ``zero_grad``,
    ``set_lr`` ...), for dense models split into block units."""

    def __init__(self, model: nn.Module, lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, mesh: Optional[ProcessMesh] = None, grad_accumulation_steps: int = 1, prefetch: bool = True,
                 fused_comm=None):
        self.model = model
        self.mesh = mesh or ProcessMesh(create_groups=False)
        self.zero_stage = 3
        self.max_grad_norm, self.grad_accumulation_steps = max_grad_norm, max(grad_accumulation_steps, 1)
        p0 = next(model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        group, W, r = self.mesh.group("dp"), self.mesh.size("dp"), self.mesh.index("dp")
        self.units: List[Unit] = []
        in_block = set()
        for i, blk in enumerate(model.layers):
            ps = [(f"layers.{i}.{n}", p) for n, p in blk.named_parameters() if p.requires_grad]
            in_block.update(id(p) for _, p in ps)
            self.units.append(Unit(f"layers.{i}", blk, ps, group, W, r, self.dtype, self.device, resident=False))
        root = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in in_block]
        self.root = Unit("root", None, root, group, W, r, self.dtype, self.device, resident=True)
        self.root.open_grads()
        self.hyper = torch.tensor([lr, betas[0], betas[1], eps, weight_decay, 0.0], dtype=torch.float32, device=self.device)
        self._hyper_host = [lr, betas[0], betas[1], eps, weight_decay, 0.0]
        self.clip_state = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step_count = 0
        self.last_grad_norm = None
        self.prefetch = prefetch and self.device.type == "cuda"
        self._pending: List[int] = []
        self._install_hooks()

    # -- hooks ----------------------------------------------------------------------------------------------
    def _install_hooks(self) -> None:
        n = len(self.units)
        for i, u in enumerate(self.units):
            def pre_fwd(mod, args, i=i):
                self.units[i].gather()
                if self.prefetch and i + 1 < n:
                    self.units[i + 1].gather()

            def post_fwd(mod, args, out, i=i):
                self.units[i].release()

            def pre_bwd(mod, gout, i=i):
                # the unit above has finished its backward: every one of its parameter gradients has been delivered,
                # so its reduce-scatter can go out now and overlap with this unit's backward
                self._flush_pending()
                self.units[i].gather()
                self.units[i].open_grads()
                if self.prefetch and i - 1 >= 0:
                    self.units[i - 1].gather()

            def post_bwd(mod, gin, gout, i=i):
                self._pending.append(i)

            u.module.register_forward_pre_hook(pre_fwd)
            u.module.register_forward_hook(post_fwd)
            u.module.register_full_backward_pre_hook(pre_bwd)
            u.module.register_full_backward_hook(post_bwd)

    def _flush_pending(self) -> None:
        for i in self._pending:
            self.units[i].reduce_grads()
            self.units[i].release()
        self._pending = []

    # -- optimiser API ----------------------------------------------------------------------------------------
    def set_lr(self, lr: float) -> None:
        self._hyper_host[0] = float(lr)
        self.hyper[0] = float(lr)

    def get_lr(self) -> float:
        return self._hyper_host[0]

    def set_weight_decay(self, wd: float) -> None:
        self._hyper_host[4] = float(wd)
        self.hyper[4] = float(wd)

    def zero_grad(self) -> None:
        for u in self.units + [self.root]:
            u.grad_fresh = True
        self.root.open_grads()

    def step(self) -> Dict[str, Any]:
        self.step_count += 1
        self._hyper_host[5] = float(self.step_count)
        self.hyper[5] = float(self.step_count)
        ops.fp8.weights_changed()  # cached quantised weights are stale after this step
        self._flush_pending()
        self.root.reduce_grads()
        units = self.units + [self.root]
        for k, u in enumerate(units):
            if u.grad_fresh:  # the unit took no part in this step
                u.grad_shard.zero_()
            ops.sumsq(u.grad_shard, self.sumsq, accumulate=k > 0)
        if dist.is_initialized() and self.mesh.world > 1:
            dist.all_reduce(self.sumsq)
        scale = 1.0 / (self.mesh.dp_size * self.grad_accumulation_steps)
        ops.clip_coef(self.sumsq, self.clip_state, scale, self.max_grad_norm)
        for u in units:
            self._adamw_masked(u)
        if self.root.full is not None:  # the resident unit needs its full copy refreshed
            self.root.full = None
            self.root.gather()
        self.zero_grad()
        self.last_grad_norm = self.clip_state[1]
        return {"grad_norm": self.clip_state[1], "skipped": self.clip_state[2]}

    def _adamw_masked(self, u: Unit) -> None:
        """AdamW on a shard whose elements carry different weight-decay multipliers: decayed and non-decayed elements
        are updated by two passes of the same kernel over masked gradients would double-apply moments, so the decay is
        applied separately and the kernel runs with decay off."""
        lr, wd = self._hyper_host[0], self._hyper_host[4]
        skip = self.clip_state[2]
        if wd != 0.0:
            u.master.mul_(1.0 - (lr * wd) * u.wd_mask * (1.0 - skip))
        ops.adamw_step(u.master, u.exp_avg, u.exp_avg_sq, u.grad_shard, u.param_shard, self.hyper, self.clip_state, 0.0)

    def get_global_grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    def gather_full_parameters(self) -> None:
        """Materialise every unit (checkpoint save / evaluation without hooks)."""
        for u in self.units:
            u.gather()

    def release_parameters(self) -> None:
        for u in self.units:
            u.release()

    def memory_bytes(self) -> Dict[str, int]:
        units = self.units + [self.root]
        return {"params": sum(u.param_shard.numel() for u in units) * units[0].param_shard.element_size(),
                "grads": sum(u.grad_shard.numel() for u in units) * units[0].grad_shard.element_size(),
                "optimizer": sum(3 * u.master.numel() * 4 for u in units)}

    # -- state (same schema as ShardedEngine.state_dict: full shapes keyed by parameter name) ---------------------
    def _gather_vec(self, u: Unit, t: torch.Tensor) -> torch.Tensor:
        if u.W == 1 or not dist.is_initialized():
            return t
        parts = [torch.empty_like(t) for _ in range(u.W)]
        dist.all_gather(parts, t.contiguous(), group=u.group)
        return torch.cat(parts)

    def state_dict(self) -> Dict[str, Any]:
        state: Dict[str, Any] = {}
        for u in self.units + [self.root]:
            full = {k: self._gather_vec(u, getattr(u, k)) for k in ("master", "exp_avg", "exp_avg_sq")}
            for name, shp, o in zip(u.names, u.shapes, u.offsets):
                state[name] = {k: v[o:o + shp.numel()].view(shp).cpu() for k, v in full.items()}
        return {"state": state, "step": self.step_count, "hyper": list(self._hyper_host), "zero_stage": 3}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = int(sd.get("step", 0))
        if sd.get("hyper"):
            self._hyper_host = list(sd["hyper"])
            self.hyper.copy_(torch.tensor(self._hyper_host, dtype=torch.float32))
        for u in self.units + [self.root]:
            lo, hi = u.r * u.shard, (u.r + 1) * u.shard
            for name, shp, o in zip(u.names, u.shapes, u.offsets):
                st = sd["state"].get(name)
                if st is None:
                    continue
                a, e = max(o, lo), min(o + shp.numel(), hi)
                if a >= e:
                    continue
                for k in ("master", "exp_avg", "exp_avg_sq"):
                    getattr(u, k)[a - lo:e - lo].copy_(st[k].reshape(-1)[a - o:e - o].to(self.device))
            u.param_shard.copy_(u.master.to(u.dtype))
        self.root.full = None
        self.root.gather()

    def owned_pieces(self, unique: bool = True) -> List[Dict[str, Any]]:
        """Same contract as :meth:`ShardedEngine.owned_pieces`: every stretch of a parameter whose state this rank holds."""
        out = []
        for u in self.units + [self.root]:
            lo, hi = u.r * u.shard, (u.r + 1) * u.shard
            for name, o, shp in zip(u.names, u.offsets, u.shapes):
                a, e = max(o, lo), min(o + shp.numel(), hi)
                if e > a:
                    out.append({"name": name, "shape": tuple(shp), "expert": False, "start": a - o, "length": e - a,
                                "tensors": {k: getattr(u, k)[a - lo:e - lo] for k in ("master", "exp_avg", "exp_avg_sq")}})
        return out

    def load_pieces(self, fetch, step: Optional[int] = None, hyper: Optional[List[float]] = None) -> int:
        if step is not None:
            self.step_count = int(step)
        if hyper:
            self._hyper_host = list(hyper)
            self.hyper.copy_(torch.tensor(self._hyper_host, dtype=torch.float32))
        n = 0
        for piece in self.owned_pieces():
            got = fetch(piece)
            if got is None:
                continue
            for k, t in piece["tensors"].items():
                t.copy_(got[k].reshape(-1).to(t.device, t.dtype))
            n += 1
        for u in self.units + [self.root]:
            u.param_shard.copy_(u.master.to(u.dtype))
        self.root.full = None
        self.root.gather()
        return n

    def resync_master_from_params(self) -> None:
        """Parameters were overwritten while gathered (checkpoint load): refresh shards and masters from them."""
        for u in self.units + [self.root]:
            if u.full is None:
                continue
            lo, hi = u.r * u.shard, (u.r + 1) * u.shard
            flat = torch.zeros(u.padded, dtype=u.dtype, device=u.device)
            for p, o, shp in zip(u.params, u.offsets, u.shapes):
                flat[o:o + shp.numel()].copy_(p.data.reshape(-1))
            u.param_shard.copy_(flat[lo:hi])
            u.master.copy_(u.param_shard.float())
            u._attach(flat)
        self.release_parameters()

    @property
    def param_groups(self) -> List[Dict[str, Any]]:
        return [{"lr": self._hyper_host[0], "weight_decay": self._hyper_host[4], "name": u.name, "params": u.params}
                for u in self.units + [self.root]]

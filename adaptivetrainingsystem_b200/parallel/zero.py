"""Sharded data-parallel training engine (ZeRO stages 0-3) on flat buckets.

Layout.  Parameters are packed, in model order, into flat *buckets* (dense+decay, dense+no-decay, expert); each
bucket owns a flat parameter buffer and a flat gradient buffer in the compute dtype, and every parameter (and its
gradient sink) is a view into them.  Each bucket is padded so that it splits into ``W`` equal shards; rank ``r``
owns ``[r*S, (r+1)*S)`` and keeps the fp32 master copy, ``exp_avg`` and ``exp_avg_sq`` only for that slice
(stage >= 1).  This is the chunk/shard pairing of the reference's vendored Gemini and LowLevelZero engines
(``colossalai/zero/gemini/chunk/chunk.py:58-650``, ``zero/low_level/low_level_optim.py:242-449``) without the
CPU placement machinery.

Step (stage >= 1): reduce-scatter of the gradient bucket -> local sum of squares -> one scalar all-reduce ->
clip coefficient on the device -> AdamW on the owned shard, writing the bf16 parameter shard -> all-gather of the
parameter bucket.  The un-scaling (1/W), the clip coefficient and the update are one kernel; nothing reads the
gradient twice.  With ``fused_comm`` and a peer-memory communicator the reduce-scatter and the all-gather are
done by the kernels themselves over NVLink (``parallel/fused.py``); the NCCL/Gloo path below is the baseline
and the CPU path.

Stage 3 additionally keeps only the owned parameter shard between steps and gathers a block's bucket right
before its forward and backward (``ZeRO3Hooks``).
"""
from __future__ import annotations

import contextlib
import math
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from .bootstrap import ProcessMesh

NO_DECAY_KEYS = ("bias", "norm", "embed")


def _pad_to(n: int, m: int) -> int:
    return ((n + m - 1) // m) * m


class Bucket:
    """A flat group of parameters that share a data-parallel group and a weight-decay setting."""

    def __init__(self, name: str, params: List[Tuple[str, nn.Parameter]], group, group_size: int, group_rank: int,
                 decay: bool, shard_states: bool, dtype: torch.dtype, device: torch.device, allocator=None):
        self.name, self.group, self.W, self.r = name, group, max(group_size, 1), group_rank
        self.decay, self.shard_states = decay, shard_states
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        offs, total = [], 0
        for p in self.params:
            offs.append(total)
            total += _pad_to(p.numel(), 8)  # keep every parameter 16-byte aligned inside the bucket
        self.offsets = offs
        self.numel = total
        self.padded = _pad_to(max(total, 8), self.W * 8)
        self.shard = self.padded // self.W
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat_param = alloc(self.padded, dtype)
        self.flat_grad = alloc(self.padded, dtype)
        for p, o in zip(self.params, offs):
            self.flat_param[o:o + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.flat_param[o:o + p.numel()].view(p.shape)
            p._ats_grad = self.flat_grad[o:o + p.numel()]
            p._ats_grad_fresh = True
            ops.functional.register_grad_sink(p)
            p.grad = None
        lo, hi = self.owned_range()
        self.master = self.flat_param[lo:hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)

    def owned_range(self) -> Tuple[int, int]:
        if self.shard_states:
            return self.r * self.shard, (self.r + 1) * self.shard
        return 0, self.padded

    def norm_range(self) -> Tuple[int, int]:
        """Slice whose squared norm this rank contributes to the global norm (a partition of the bucket)."""
        return self.r * self.shard, (self.r + 1) * self.shard

    def mark_fresh(self) -> None:
        for p in self.params:
            p._ats_grad_fresh = True

    def segments_in(self, lo: int, hi: int) -> List[Tuple[int, int, int]]:
        """(start relative to lo, length, parameter index) of every parameter's part inside [lo, hi) (per-tensor optimisers)."""
        out = []
        for i, (p, o) in enumerate(zip(self.params, self.offsets)):
            a, b = max(o, lo), min(o + p.numel(), hi)
            if b > a:
                out.append((a - lo, b - a, i))
        return out

    def collect_autograd_grads(self) -> None:
        """Gradients that arrived through plain autograd (``p.grad``) are folded into the flat buffer; parameters
        that received nothing this step are zeroed."""
        for p, o in zip(self.params, self.offsets):
            sink = self.flat_grad[o:o + p.numel()]
            if p.grad is not None:
                if p._ats_grad_fresh:
                    sink.copy_(p.grad.reshape(-1))
                else:
                    sink.add_(p.grad.reshape(-1).to(sink.dtype))
                p.grad = None
                p._ats_grad_fresh = False
            elif p._ats_grad_fresh:
                sink.zero_()


class ShardedEngine:
    """Owns the buckets, the optimiser state and the step.  ``hyper`` is a device tensor
    ``[lr, beta1, beta2, eps, weight_decay, step]`` so hyper-parameter changes never rebuild anything."""

    def __init__(self, model: nn.Module, lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: float = 1.0, zero_stage: int = 1,
                 mesh: Optional[ProcessMesh] = None, fused_comm=None, grad_accumulation_steps: int = 1,
                 optimizer: str = "adamw", optimizer_kwargs: Optional[Dict[str, Any]] = None):
        self.model = model
        # "adamw" runs the built-in (and peer-memory fused) path; "lamb", "sgd" and "adamw_host" (optimiser state offloaded
        # to pinned host memory) go through an update rule of the optim package
        self.optimizer_name = optimizer.lower()
        self.rule = None
        if self.optimizer_name != "adamw":
            from ..optim import make_rule
            self.rule = make_rule(self.optimizer_name, **(optimizer_kwargs or {}))
        self.mesh = mesh or ProcessMesh(create_groups=False)
        self.zero_stage = zero_stage
        self.max_grad_norm = max_grad_norm
        self.fused = fused_comm
        self.grad_accumulation_steps = max(grad_accumulation_steps, 1)
        p0 = next(model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        self.hyper = torch.tensor([lr, betas[0], betas[1], eps, weight_decay, 0.0], dtype=torch.float32, device=self.device)
        self._hyper_host = [lr, betas[0], betas[1], eps, weight_decay, 0.0]
        self.clip_state = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._scratch = torch.zeros(1024, dtype=torch.float32, device=self.device) if self.device.type == "cuda" else None
        self.step_count = 0
        self.comm_timer = None      # a ``utils.profiler.PhaseTimer`` when the collectives of the step are to be timed
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.buckets: List[Bucket] = []
        self._build_buckets()

    # -- construction ------------------------------------------------------------------------------------
    def _build_buckets(self) -> None:
        dense_d, dense_n, expert = [], [], []
        seen = set()
        for name, p in self.model.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            if getattr(p, "_ats_expert", False):
                expert.append((name, p))
            elif p.ndim < 2 or any(k in name.lower() for k in NO_DECAY_KEYS):
                dense_n.append((name, p))
            else:
                dense_d.append((name, p))
        m = self.mesh
        shard = self.zero_stage >= 1
        alloc = self.fused.allocator() if self.fused is not None else None
        spec = [("dense_decay", dense_d, "dp", True), ("dense_no_decay", dense_n, "dp", False), ("expert", expert, "edp", True)]
        tp = getattr(m, "tp_size", 1)
        if tp > 1:
            # parameters that tensor parallelism splits differ from rank to rank of a tp group; all others are replicated there and
            # must count ONCE in the global gradient norm (reference: colossalai/booster/plugin/hybrid_parallel_plugin.py:342-418)
            split = []
            for name, plist, axis, decay in spec:
                split.append((name + "_tp", [(n, p) for n, p in plist if getattr(p, "_ats_tp", None) is not None], axis, decay))
                split.append((name, [(n, p) for n, p in plist if getattr(p, "_ats_tp", None) is None], axis, decay))
            spec = split
        for name, plist, axis, decay in spec:
            if not plist:
                continue
            b = Bucket(name, plist, m.group(axis), m.size(axis), m.index(axis), decay, shard, self.dtype, self.device, alloc)
            b.norm_weight = 1.0 if (tp == 1 or name.endswith("_tp")) else 1.0 / tp
            self.buckets.append(b)

    # -- hyper-parameters -----------------------------------------------------------------------------------
    def set_lr(self, lr: float) -> None:
        self._hyper_host[0] = float(lr)
        self.hyper[0] = float(lr)

    def get_lr(self) -> float:
        return self._hyper_host[0]

    def set_weight_decay(self, wd: float) -> None:
        self._hyper_host[4] = float(wd)
        self.hyper[4] = float(wd)

    @property
    def param_groups(self) -> List[Dict[str, Any]]:
        """torch.optim-style read-only view for schedulers and reports."""
        return [{"lr": self._hyper_host[0], "weight_decay": self._hyper_host[4] if b.decay else 0.0,
                 "name": b.name, "params": b.params} for b in self.buckets]

    # -- step -----------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        for b in self.buckets:
            b.mark_fresh()
            for p in b.params:
                p.grad = None

    def _comm(self, name: str):
        return self.comm_timer.phase(name) if self.comm_timer is not None else contextlib.nullcontext()

    def _reduce(self, b: Bucket) -> torch.Tensor:
        """Returns the (summed over the group) gradient slice this rank updates."""
        lo, hi = b.owned_range()
        if b.W == 1 or b.group is None and not dist.is_initialized():
            return b.flat_grad[lo:hi]
        with self._comm("grad_reduce"):
            if b.shard_states:
                out = b.flat_grad[lo:hi]
                if dist.get_backend(b.group) == "gloo":
                    dist.all_reduce(b.flat_grad, group=b.group)
                else:
                    dist.reduce_scatter_tensor(out, b.flat_grad, group=b.group)
                return out
            dist.all_reduce(b.flat_grad, group=b.group)
            return b.flat_grad

    def _gather(self, b: Bucket) -> None:
        if b.W == 1 or not b.shard_states or not dist.is_initialized():
            return
        lo, hi = b.owned_range()
        with self._comm("param_gather"):
            if dist.get_backend(b.group) == "gloo":
                parts = [torch.empty_like(b.flat_param[lo:hi]) for _ in range(b.W)]
                dist.all_gather(parts, b.flat_param[lo:hi].clone(), group=b.group)
                for i, t in enumerate(parts):
                    b.flat_param[i * b.shard:(i + 1) * b.shard].copy_(t)
            else:
                dist.all_gather_into_tensor(b.flat_param, b.flat_param[lo:hi], group=b.group)

    def step(self) -> Dict[str, Any]:
        """Reduce gradients, clip by global norm, AdamW on the owned shards, re-assemble parameters.
        Returns device tensors (no host synchronisation): ``grad_norm``, ``skipped``."""
        self.step_count += 1
        self._hyper_host[5] = float(self.step_count)
        self.hyper[5] = float(self.step_count)
        ops.fp8.weights_changed()  # cached quantised weights are stale after this step
        if self.rule is None and self.fused is not None and self.fused.usable(self):
            # reduce-scatter, norm, AdamW and all-gather done by peer-memory kernels (parallel/fused.py)
            self.fused.step(self)
            self.zero_grad()
            self.last_grad_norm = self.clip_state[1]
            return {"grad_norm": self.clip_state[1], "skipped": self.clip_state[2]}
        reduced = []
        first = True
        for b in self.buckets:
            b.collect_autograd_grads()
            g = self._reduce(b)
            reduced.append(g)
            lo, hi = b.owned_range()
            nlo, nhi = b.norm_range()
            if getattr(b, "norm_weight", 1.0) == 1.0:
                ops.sumsq(g[nlo - lo:nhi - lo], self.sumsq, accumulate=not first, scratch=self._scratch)
            else:  # replicated inside a tensor-parallel group: every rank of the group adds 1 / tp of it
                part = torch.zeros_like(self.sumsq)
                ops.sumsq(g[nlo - lo:nhi - lo], part, accumulate=False, scratch=self._scratch)
                if first:
                    self.sumsq.zero_()
                self.sumsq.add_(part * b.norm_weight)
            first = False
        # The objective is the mean over the dp_size data-parallel replicas (and over the accumulated
        # micro-batches); expert gradients already hold the contributions of every expert-parallel peer, so the
        # same 1/dp_size applies to them.  The scale is folded into the AdamW kernel with the clip coefficient.
        scale = 1.0 / (self.mesh.dp_size * self.grad_accumulation_steps)
        if dist.is_initialized() and self.mesh.world > 1:
            dist.all_reduce(self.sumsq)
        ops.clip_coef(self.sumsq, self.clip_state, scale, self.max_grad_norm)
        for b, g in zip(self.buckets, reduced):
            lo, hi = b.owned_range()
            if self.rule is None:
                ops.adamw_step(b.master, b.exp_avg, b.exp_avg_sq, g, b.flat_param[lo:hi], self.hyper, self.clip_state,
                               1.0 if b.decay else 0.0)
            else:
                if getattr(b, "rule_state", None) is None:
                    b.rule_state = self.rule.init_state(b.master)
                    if self.optimizer_name == "adamw_host":  # the device copies of the state are not needed any more
                        b.exp_avg = b.exp_avg_sq = torch.zeros(0, device=self.device)
                kw = {"n_segments": len(b.params)} if self.optimizer_name in ("lamb", "lars") else {}
                self.rule.update(b.rule_state, b.master, g, b.flat_param[lo:hi], self.hyper, self.clip_state, b.decay,
                                 segments=b.segments_in(lo, hi), group=b.group if b.shard_states and b.W > 1 else None, **kw)
            self._gather(b)
        self.zero_grad()
        self.last_grad_norm = self.clip_state[1]
        return {"grad_norm": self.clip_state[1], "skipped": self.clip_state[2]}

    def get_global_grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    # -- state ----------------------------------------------------------------------------------------------
    def _gather_state(self, b: Bucket, t: torch.Tensor) -> torch.Tensor:
        if not b.shard_states or b.W == 1 or not dist.is_initialized():
            return t
        parts = [torch.empty_like(t) for _ in range(b.W)]
        dist.all_gather(parts, t.contiguous(), group=b.group)
        return torch.cat(parts)

    def state_dict(self) -> Dict[str, Any]:
        """Per-parameter optimiser state in full (un-sharded) shapes, keyed by parameter name -- the same on every
        rank of a data-parallel group, so a checkpoint can be re-sharded for any world size."""
        state: Dict[str, Any] = {}
        for b in self.buckets:
            full = {k: self._gather_state(b, getattr(b, k)) for k in ("master", "exp_avg", "exp_avg_sq")}
            for name, p, o in zip(b.names, b.params, b.offsets):
                state[name] = {k: v[o:o + p.numel()].view(p.shape).cpu() for k, v in full.items()}
        return {"state": state, "step": self.step_count, "hyper": list(self._hyper_host), "zero_stage": self.zero_stage}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = int(sd.get("step", 0))
        hyper = sd.get("hyper")
        if hyper:
            self._hyper_host = list(hyper)
            self.hyper.copy_(torch.tensor(hyper, dtype=torch.float32))
        for b in self.buckets:
            lo, hi = b.owned_range()
            for name, p, o in zip(b.names, b.params, b.offsets):
                st = sd["state"].get(name)
                if st is None:
                    continue
                a, e = max(o, lo), min(o + p.numel(), hi)
                if a >= e:
                    continue
                for k in ("master", "exp_avg", "exp_avg_sq"):
                    getattr(b, k)[a - lo:e - lo].copy_(st[k].reshape(-1)[a - o:e - o].to(self.device))

    # -- sharded state: what lives on this rank, piece by piece ---------------------------------------------------
    def owned_pieces(self, unique: bool = True) -> List[Dict[str, Any]]:
        """One entry ``{name, shape, expert, start, length, tensors: {master, exp_avg, exp_avg_sq}}`` for every stretch of a
        parameter (``length`` elements from flat element ``start``) whose optimiser state this rank holds.  With ``unique`` a
        stretch that is replicated over a group (stage 0, or a group of one) is listed by the group's first rank only, so that
        the pieces of all ranks together cover every parameter exactly once."""
        out = []
        for b in self.buckets:
            if unique and not (b.shard_states and b.W > 1) and b.r != 0:
                continue
            lo, hi = b.owned_range()
            for rel, length, i in b.segments_in(lo, hi):
                p = b.params[i]
                out.append({"name": b.names[i], "shape": tuple(p.shape), "expert": bool(getattr(p, "_ats_expert", False)),
                            "start": lo + rel - b.offsets[i], "length": length,
                            "tensors": {k: getattr(b, k)[rel:rel + length] for k in ("master", "exp_avg", "exp_avg_sq")}})
        return out

    def load_pieces(self, fetch: Callable[[Dict[str, Any]], Optional[Dict[str, torch.Tensor]]], step: Optional[int] = None,
                    hyper: Optional[List[float]] = None) -> int:
        """Inverse of :meth:`owned_pieces`: ``fetch(piece)`` returns the three state vectors of that stretch (or ``None`` when
        the checkpoint has nothing for it).  Returns the number of stretches restored."""
        if step is not None:
            self.step_count = int(step)
        if hyper:
            self._hyper_host = list(hyper)
            self.hyper.copy_(torch.tensor(hyper, dtype=torch.float32))
        n = 0
        for piece in self.owned_pieces(unique=False):
            got = fetch(piece)
            if got is None:
                continue
            for k, t in piece["tensors"].items():
                t.copy_(got[k].reshape(-1).to(t.device, t.dtype))
            n += 1
        return n

    # -- row access: moving experts between ranks, permuting router rows -----------------------------------------
    def _locate(self, name: str) -> Tuple[Bucket, int]:
        for b in self.buckets:
            if name in b.names:
                return b, b.names.index(name)
        raise KeyError(name)

    def read_rows(self, name: str, rows: List[int]) -> torch.Tensor:
        """Optimiser state of whole rows (dim 0) of a parameter: ``[3, len(rows), row_numel]`` fp32 (master, exp_avg,
        exp_avg_sq).  Collective over the parameter's group when its state is sharded: every rank of the group gets all of it."""
        b, i = self._locate(name)
        p, o = b.params[i], b.offsets[i]
        rn = p.numel() // p.shape[0]
        lo, hi = b.owned_range()
        out = torch.zeros(3, len(rows), rn, dtype=torch.float32, device=self.device)
        for j, r in enumerate(rows):
            base = o + r * rn
            a, e = max(base, lo), min(base + rn, hi)
            if e > a:
                for k, key in enumerate(("master", "exp_avg", "exp_avg_sq")):
                    out[k, j, a - base:e - base].copy_(getattr(b, key)[a - lo:e - lo])
        if b.shard_states and b.W > 1 and dist.is_initialized():
            dist.all_reduce(out, group=b.group)
        return out

    def write_rows(self, name: str, rows: List[int], state: torch.Tensor) -> None:
        """Inverse of :meth:`read_rows` (local: every rank writes the stretches it owns); the parameter rows are re-derived from
        the master values."""
        b, i = self._locate(name)
        p, o = b.params[i], b.offsets[i]
        rn = p.numel() // p.shape[0]
        lo, hi = b.owned_range()
        for j, r in enumerate(rows):
            base = o + r * rn
            a, e = max(base, lo), min(base + rn, hi)
            if e > a:
                for k, key in enumerate(("master", "exp_avg", "exp_avg_sq")):
                    getattr(b, key)[a - lo:e - lo].copy_(state[k, j, a - base:e - base])
            p.data[r].copy_(state[0, j].view(p.shape[1:]).to(p.dtype))

    def resync_master_from_params(self) -> None:
        """After parameters were overwritten (checkpoint load), refresh the fp32 master slices."""
        for b in self.buckets:
            lo, hi = b.owned_range()
            b.master.copy_(b.flat_param[lo:hi].float())

    def rebuild(self, row_maps: Optional[Dict[str, List[int]]] = None) -> None:
        """Re-pack after the set or shape of parameters changed (expert add / prune).  State of surviving
        parameters is carried over by name.  ``row_maps[name][i] = j`` says that row ``i`` of the new parameter
        continues row ``j`` of the old one (``-1``: a new row, which starts with zero moments and a master copy
        taken from the parameter itself)."""
        old = self.state_dict()
        named = dict(self.model.named_parameters())
        for name, rows in (row_maps or {}).items():
            st = old["state"].get(name)
            if st is None or name not in named:
                continue
            p = named[name]
            idx = torch.tensor([max(j, 0) for j in rows], dtype=torch.long)
            fresh = torch.tensor([j < 0 for j in rows])
            for k in ("master", "exp_avg", "exp_avg_sq"):
                t = st[k].index_select(0, idx).clone()
                if fresh.any():
                    t[fresh] = p.data[fresh.to(p.device)].float().cpu() if k == "master" else 0.0
                st[k] = t
        self.buckets = []
        self._build_buckets()
        named = dict(self.model.named_parameters())
        old["state"] = {k: v for k, v in old["state"].items() if k in named and v["master"].numel() == named[k].numel()}
        self.load_state_dict({**old, "step": self.step_count, "hyper": self._hyper_host})

    def memory_bytes(self) -> Dict[str, int]:
        out = {"params": 0, "grads": 0, "optimizer": 0}
        for b in self.buckets:
            out["params"] += b.flat_param.numel() * b.flat_param.element_size()
            out["grads"] += b.flat_grad.numel() * b.flat_grad.element_size()
            out["optimizer"] += 3 * b.master.numel() * 4
        return out

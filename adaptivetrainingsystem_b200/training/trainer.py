"""Trainer: loss, micro-batch / optimiser steps, evaluation, epochs, schedulers, checkpoints and the runtime
intervention API the orchestrator drives.

Public surface mirrors the reference trainer (reference ``training/trainer.py:985-3643``; README API
``Readme.md:763-857``): ``train``, ``train_with_oom_fallback``, ``train_epoch``, ``train_step``,
``optimizer_step``, ``evaluate``, ``compute_loss``, ``_setup_scheduler`` and the interventions
``add_expert / prune_expert / adjust_capacity_factor / adjust_routing_temperature / enable_expert_dropout /
get_expert_statistics / adjust_mod_capacity / get_mod_statistics / adjust_batch_size / emergency_lr_reduction /
rollback_steps / adjust_weight_decay / adjust_learning_rate / get_current_metrics``.

Design differences:

* one engine (``parallel.zero.ShardedEngine``) does DDP / ZeRO-1/2/3 / expert-parallel steps -- the trainer
  never branches on a backend;
* no host synchronisation inside a step: loss, gradient norm and skip flag stay on the device and are read
  once per logging interval (the reference synchronises >= 4 times per micro-batch, ``trainer.py:2461-2519``);
* interventions requested from another thread are queued and applied at the next step boundary under a lock
  (the reference mutates optimiser state concurrently with the training thread);
* the metric lists the orchestrator reads are really appended (``train_losses``, ``gradient_norms``,
  ``learning_rates``), and epoch / eval losses are means, with the best value reported separately.
"""
from __future__ import annotations

import gc
import json
import logging
import math
import os
import threading
import contextlib
import time
from collections import deque
from contextlib import nullcontext
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import Config
from ..models.transformer import DeepSeekTransformer, MoEFFNLayer
from ..parallel.bootstrap import ProcessMesh, get_rank, world_size
from ..parallel.zero import ShardedEngine
from .checkpoint import CheckpointManager
from .precision import PrecisionManager, QuantizationManager
from .schedulers import build_scheduler

log = logging.getLogger("ats.trainer")


@dataclass
class TrainingMetrics:
    """Snapshot handed to the orchestrator (reference ``training/orchestrator.py:48-67``)."""
    epoch: int = 0
    step: int = 0
    loss: float = 0.0
    grad_norm: float = 0.0
    learning_rate: float = 0.0
    expert_utilization: Dict[str, float] = field(default_factory=dict)
    memory_usage: Dict[str, float] = field(default_factory=dict)
    throughput: float = 0.0
    semantic_coherence: float = 0.0
    factual_accuracy: float = 0.0
    reasoning_score: float = 0.0
    timestamp: float = field(default_factory=time.time)


class SyntheticOOM(RuntimeError):
    """Raised by host-side fault injection; carries the same text torch uses so recovery paths match."""

    def __init__(self):
        super().__init__("CUDA out of memory. (injected on the host)")


def is_oom_error(e: BaseException) -> bool:
    return isinstance(e, (torch.cuda.OutOfMemoryError, SyntheticOOM)) or "out of memory" in str(e).lower()


class EnhancedConversationTrainer:
    def __init__(self, model: DeepSeekTransformer, tokenizer=None, config: Optional[Config] = None, logger=None,
                 mesh: Optional[ProcessMesh] = None, fused_comm=None):
        self.config = config or Config()
        self.model = model
        self.tokenizer = tokenizer
        self.logger = logger or log
        self.mesh = mesh or ProcessMesh(create_groups=False)
        self.device = next(model.parameters()).device
        # parallel strategies of the run (Config.tensor_parallel_size / sequence_parallel_size / pipeline_parallel_size through
        # ProcessMesh.from_config): the model is converted in place before the engine packs its parameters
        self.pipeline = None
        if self.mesh.tp_size > 1 or self.mesh.sp_size > 1:
            from ..parallel.strategy import apply_sequence_parallel, apply_tensor_parallel
            apply_tensor_parallel(model, self.mesh)
            apply_sequence_parallel(model, self.mesh)
        if self.mesh.pp_size > 1:
            from ..parallel.pipeline import InterleavedStages, PipelineStage
            chunks = int(getattr(self.config, "pipeline_chunks", 1) or 1)
            if chunks > 1:
                self.pipeline = InterleavedStages(model, self.mesh.coord.pp, self.mesh.pp_size, chunks)
            else:
                self.pipeline = PipelineStage(model, self.mesh.coord.pp, self.mesh.pp_size)
            self._pp_batches: List[Dict[str, torch.Tensor]] = []
            self._pp_schedule = None
        self.precision_manager = PrecisionManager(self.config, self.device)
        # fp8 precisions switch the linear layers' forward products to the e4m3 tcgen05 GEMM (process-wide switch)
        from .. import ops as _ops
        _ops.fp8.set_enabled(self.precision_manager.uses_fp8 and self.device.type == "cuda")
        self.quantization_manager = QuantizationManager(self.config)
        self.moe_manager = MoEOptimizationManager(self.config)
        self.pad_token_id = getattr(tokenizer, "pad_token_id", None)
        self.ignore_index = -100

        opt = dict(lr=self.config.learning_rate, betas=(self.config.adam_beta1, self.config.adam_beta2), eps=self.config.adam_eps,
                   weight_decay=self.config.weight_decay, max_grad_norm=getattr(self.config, "max_grad_norm", 1.0), mesh=self.mesh,
                   grad_accumulation_steps=1 if self.pipeline is not None else self.config.gradient_accumulation_steps)
        # (a pipeline schedule already divides the loss by its number of micro-batches)
        if self.config.zero_stage >= 3 and self.mesh.ep_size == 1 and self.mesh.world > 1:
            from ..parallel.zero3 import ZeRO3Engine
            self.engine = ZeRO3Engine(model, fused_comm=fused_comm, **opt)  # per-block gather / release
        else:
            if self.config.zero_stage >= 3 and self.mesh.world > 1:
                self.logger.warning("zero_stage 3 requested with expert parallelism (ep=%d): experts stay partitioned by expert "
                                    "parallelism, the dense part runs stage 2", self.mesh.ep_size)
            # optimiser choice: config.optimizer ("adamw" | "lamb" | "sgd"); the offload flags of the reference's DeepSpeed
            # section (cpu_offload / cpu_offload_optimizer) move the AdamW state to pinned host memory
            name = str(getattr(self.config, "optimizer", "adamw")).lower()
            nvme = bool(getattr(self.config, "nvme_offload_optimizer", False) and getattr(self.config, "nvme_path", None))
            if name == "adamw" and (self.config.cpu_offload or self.config.cpu_offload_optimizer or nvme):
                name = "adamw_host"
            # nvme_offload_optimizer + nvme_path: the host-side state lives in memory-mapped files under that path
            okw = {"spill_dir": os.path.join(self.config.nvme_path, "ats_optimizer_state")} if (nvme and name == "adamw_host") else None
            self.engine = ShardedEngine(model, zero_stage=min(self.config.zero_stage, 2), fused_comm=fused_comm, optimizer=name,
                                        optimizer_kwargs=okw, **opt)
        self.optimizer = self.engine  # reference attribute name
        self.scheduler = None
        self.use_deepspeed = False

        self.global_step = 0
        self.current_epoch = 0
        self.best_eval_loss = float("inf")
        self.patience_counter = 0
        self.should_stop = False
        self.micro_step = 0
        self.metrics: Dict[str, List[Any]] = {k: [] for k in (
            "train_losses", "eval_losses", "learning_rates", "gradient_norms", "throughput", "epoch_times",
            "tokens_per_second", "accuracies")}
        self.checkpoint_history: List[Dict[str, Any]] = []
        exp_dir = os.path.join(getattr(self.config, "output_dir", "experiments"), self.config.experiment_name or "run")
        self.checkpoint_manager = CheckpointManager(self.config, os.path.join(exp_dir, "checkpoints"))
        self._last_backup = time.time()
        # profiling flags of the configuration (declared by the reference, consumed by none of its live code)
        from ..utils.profiler import PhaseTimer
        self.phase_timer = PhaseTimer(self.device) if getattr(self.config, "enable_profiling", False) else None
        if getattr(self.config, "profile_communication", False) and hasattr(self.engine, "comm_timer"):
            self.engine.comm_timer = PhaseTimer(self.device)
        self.peak_memory_gb: List[float] = []
        self.checkpoint_manager.extra_meta = lambda: {"precision_info": self.precision_manager.get_precision_info(),
                                                      "quantization_info": self.quantization_manager.get_quantization_info()}
        self.chinchilla_scaler = None
        self.train_dataset = None
        self.eval_dataset = None
        self._dataloader_factory: Optional[Callable] = None

        # adaptive-LR override bookkeeping (reference trainer.py:1144-1175, 2610-2652)
        self.adaptive_lr_override = False
        self.lr_override_steps_left = 0
        self.lr_override_emergency = False
        self.recent_grad_norms: deque = deque(maxlen=5)

        # step-boundary mailbox for interventions coming from the monitor thread
        self._lock = threading.RLock()
        self._train_thread = threading.current_thread()
        self._pending: List[Callable[[], None]] = []
        self._pending_device: List[Dict[str, torch.Tensor]] = []
        self._tokens_window: deque = deque(maxlen=10)
        self._last_step_time = time.perf_counter()
        self._inject_oom_at: Optional[int] = None

        # failure detection: in-kernel waits on peers give up after comm_timeout_s (status word -> KernelError on the host);
        # a heartbeat through the rendezvous store tells the survivors of a lost rank before they launch the next step
        self.heartbeat = None
        if self.mesh.world > 1:
            import torch.distributed as _dist
            if fused_comm is not None and self.device.type == "cuda":
                from ..parallel.peer import set_wait_budget
                set_wait_budget(float(getattr(self.config, "comm_timeout_s", 1.0) or 1.0))
            hb = float(getattr(self.config, "heartbeat_interval_s", 0.0) or 0.0)
            if hb > 0 and _dist.is_initialized():
                from ..parallel.health import Heartbeat
                self.heartbeat = Heartbeat(interval_s=hb, timeout_s=float(getattr(self.config, "heartbeat_timeout_s", 30.0))).start()

    # ------------------------------------------------------------------------------------------------------
    # loss
    # ------------------------------------------------------------------------------------------------------
    def compute_loss(self, logits: torch.Tensor, labels: torch.Tensor,
                     loss_weights: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """Weighted next-token cross-entropy.  ``labels`` are already aligned with ``logits`` (the dataset shifts
        them); positions equal to ``ignore_index`` -- or to the pad id when the tokenizer defines a non-zero one --
        are excluded.  Returns ``loss`` (weighted mean, differentiable), ``raw_loss`` (unweighted mean, detached),
        ``perplexity = exp(min(raw_loss, 15))`` (``inf`` when nothing is valid), ``valid_tokens``, ``accuracy``."""
        lb = labels
        if self.pad_token_id not in (None, 0):
            lb = torch.where(lb == self.pad_token_id, torch.full_like(lb, self.ignore_index), lb)
        loss, raw, nvalid, acc = ops.cross_entropy(logits, lb, loss_weights, self.ignore_index)
        return self._loss_dict(loss, raw, nvalid, acc)

    @staticmethod
    def _loss_dict(loss, raw, nvalid, acc) -> Dict[str, torch.Tensor]:
        ppl = torch.where(nvalid > 0, torch.exp(torch.clamp(raw.detach().float(), max=15.0)),
                          torch.full_like(raw.detach().float(), float("inf")))
        return {"loss": loss, "raw_loss": raw.detach(), "perplexity": ppl, "valid_tokens": nvalid, "accuracy": acc}

    # ------------------------------------------------------------------------------------------------------
    # steps
    # ------------------------------------------------------------------------------------------------------
    def _to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        """Forward + backward of one micro-batch.  Every returned value is a device tensor (no sync)."""
        if self._inject_oom_at is not None and self.micro_step == self._inject_oom_at:
            self._inject_oom_at = None
            raise SyntheticOOM()
        if self.heartbeat is not None:
            self.heartbeat.check()  # a lost peer surfaces here, on the host, before any kernel waits for it
        self.model.train()
        with self._phase("to_device"):
            batch = self._to_device(batch)
        if self.mesh.sp_size > 1:
            from ..parallel.strategy import shard_sequence
            batch = shard_sequence(batch, self.mesh)  # this rank's L / W tokens of every sequence
        if self.pipeline is not None:
            return self._pipeline_collect(batch)
        labels = batch["labels"]
        if self.pad_token_id not in (None, 0):
            labels = torch.where(labels == self.pad_token_id, torch.full_like(labels, self.ignore_index), labels)
        mask = batch.get("attention_mask")
        if mask is not None and bool(getattr(self.config, "assume_full_attention_mask", True)):
            mask = None  # packed / synthetic batches are dense; padding is handled by the label mask
        with self._phase("forward"), self.precision_manager.autocast():
            out = self.model.forward_loss(batch["input_ids"], labels, batch.get("loss_weights"), mask, self.ignore_index)
        with self._phase("backward"):
            out["loss"].backward()
        self.micro_step += 1
        res = self._loss_dict(out["loss"].detach(), out["raw_loss"], out["valid_tokens"], out["accuracy"])
        res["aux_loss"] = out["aux_loss"]
        res["tokens"] = batch["input_ids"].numel()
        self._pending_device.append(res)
        return res

    # -- pipeline parallelism: micro-batches are collected and run through the schedule at the optimiser step -------------------
    def _pipeline_collect(self, batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        labels = batch["labels"]
        if self.pad_token_id not in (None, 0):
            labels = torch.where(labels == self.pad_token_id, torch.full_like(labels, self.ignore_index), labels)
        self._pp_batches.append({"input_ids": batch["input_ids"], "labels": labels, "loss_weights": batch.get("loss_weights")})
        self.micro_step += 1
        zero = torch.zeros((), device=self.device)
        res = {"loss": zero, "raw_loss": zero, "perplexity": zero, "valid_tokens": zero, "accuracy": zero, "aux_loss": zero,
               "tokens": batch["input_ids"].numel(), "pipeline_pending": True}
        return res

    def _pipeline_run(self) -> None:
        """All collected micro-batches through the 1F1B (or interleaved 1F1B) schedule; the loss of the last stage is shared
        with the other stages for logging."""
        from ..parallel.pipeline import InterleavedSchedule, InterleavedStages, OneFOneBSchedule
        import torch.distributed as dist
        mbs, self._pp_batches = self._pp_batches, []
        if not mbs:
            return
        group = self.mesh.group("pp")
        B, L = mbs[0]["input_ids"].shape
        shape = (B, L, self.model.config.hidden_size)
        dtype = next(p for p in self.model.parameters() if p.numel() > 0).dtype
        key = (len(mbs), shape)
        if self._pp_schedule is None or self._pp_schedule[0] != key:
            cls = InterleavedSchedule if isinstance(self.pipeline, InterleavedStages) else OneFOneBSchedule
            self._pp_schedule = (key, cls(self.pipeline, group, len(mbs), shape, dtype, self.device))
        loss = self._pp_schedule[1].run(mbs)
        last = self.mesh.ranks_along("pp")[-1]
        t = loss.detach().float().reshape(1) if loss is not None else torch.zeros(1, device=self.device)
        dist.broadcast(t, last, group=group)
        tokens = sum(m["input_ids"].numel() for m in mbs)
        self._pending_device.append({"loss": t[0], "raw_loss": t[0], "accuracy": torch.zeros((), device=self.device), "tokens": tokens})

    def _phase(self, name: str):
        return self.phase_timer.phase(name) if self.phase_timer is not None else contextlib.nullcontext()

    def profiling_summary(self) -> Dict[str, Any]:
        """What the profiling flags collected: ``enable_profiling`` -> mean device (CUDA events) or host milliseconds per
        phase of a micro-step; ``profile_communication`` -> the same for the engine's collectives (the fused peer-memory step
        has no separate collectives to time); ``profile_memory`` -> peak allocated GB per epoch."""
        out: Dict[str, Any] = {}
        if self.phase_timer is not None:
            out["phase_ms"] = self.phase_timer.summary()
        timer = getattr(self.engine, "comm_timer", None)
        if timer is not None:
            out["communication_ms"] = timer.summary()
        if getattr(self.config, "profile_memory", False):
            out["peak_memory_gb_per_epoch"] = list(self.peak_memory_gb)
        return out

    def optimizer_step(self) -> Dict[str, Any]:
        if self.pipeline is not None:
            self._pipeline_run()
        with self._lock:
            with self._phase("optimizer"):
                stats = self.engine.step()
            self.global_step += 1
            self._advance_scheduler(stats)
            pending, self._pending = self._pending, []
        for fn in pending:  # interventions queued by other threads, applied between steps
            fn()
        return stats

    def _advance_scheduler(self, stats: Dict[str, Any]) -> None:
        if self.adaptive_lr_override:
            if self.lr_override_emergency:
                # released once the last five gradient norms are all below 10 (one host read, emergency only)
                self.recent_grad_norms.append(float(stats["grad_norm"]))
                if len(self.recent_grad_norms) == self.recent_grad_norms.maxlen and max(self.recent_grad_norms) < 10.0:
                    self.adaptive_lr_override = False
                    self.lr_override_emergency = False
            else:
                self.lr_override_steps_left -= 1
                if self.lr_override_steps_left <= 0:
                    self.adaptive_lr_override = False
            return
        if self.scheduler is not None and getattr(self.config, "use_lr_scheduler", True):
            self.engine.set_lr(self.scheduler.step())

    def _flush_metrics(self) -> Optional[Dict[str, float]]:
        """One host read for everything accumulated since the last flush."""
        if not self._pending_device:
            return None
        items, self._pending_device = self._pending_device, []
        loss = torch.stack([i["loss"].float() for i in items]).mean()
        raw = torch.stack([i["raw_loss"].float() for i in items]).mean()
        acc = torch.stack([i["accuracy"].float() for i in items]).mean()
        gn = self.engine.last_grad_norm if self.engine.last_grad_norm is not None else loss.new_zeros(())
        vals = torch.stack([loss, raw, acc, gn.float().reshape(())]).tolist()
        tokens = sum(i["tokens"] for i in items)
        now = time.perf_counter()
        dt = max(now - self._last_step_time, 1e-9)
        self._last_step_time = now
        tps = tokens * world_size() / dt
        self._tokens_window.append(tps)
        self.metrics["train_losses"].append(vals[0])
        self.metrics["gradient_norms"].append(vals[3])
        self.metrics["learning_rates"].append(self.engine.get_lr())
        self.metrics["tokens_per_second"].append(tps)
        self.metrics["accuracies"].append(vals[2])
        return {"loss": vals[0], "raw_loss": vals[1], "accuracy": vals[2], "grad_norm": vals[3], "tokens_per_second": tps,
                "perplexity": math.exp(min(vals[1], 15.0)), "lr": self.engine.get_lr()}

    # ------------------------------------------------------------------------------------------------------
    # evaluation
    # ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self, eval_dataset=None, max_batches: int = 100) -> Dict[str, float]:
        ds = eval_dataset if eval_dataset is not None else self.eval_dataset
        if ds is None:
            return {}
        self.model.eval()
        loader = self._make_loader(ds, shuffle=False)
        losses, accs, toks = [], [], 0
        for i, batch in enumerate(loader):
            if i >= max_batches:
                break
            batch = self._to_device(batch)
            with self.precision_manager.autocast():
                out = self.model.forward_loss(batch["input_ids"], batch["labels"], batch.get("loss_weights"), None, self.ignore_index)
            losses.append(out["raw_loss"].float())
            accs.append(out["accuracy"].float())
            toks += batch["input_ids"].numel()
        self.model.train()
        if not losses:
            return {}
        lv = torch.stack(losses)
        mean, best = float(lv.mean()), float(lv.min())
        res = {"eval_loss": mean, "eval_best_batch_loss": best, "eval_perplexity": math.exp(min(mean, 15.0)),
               "eval_accuracy": float(torch.stack(accs).mean()), "eval_tokens": toks}
        self.metrics["eval_losses"].append(mean)
        return res

    # ------------------------------------------------------------------------------------------------------
    # epochs
    # ------------------------------------------------------------------------------------------------------
    def _make_loader(self, dataset, shuffle: bool):
        if self._dataloader_factory is not None:
            return self._dataloader_factory(dataset, self.config, shuffle)
        from ..data.dataset import create_dataloader
        return create_dataloader(dataset, self.config, shuffle=shuffle)

    def _recreate_dataloader(self, dataset, shuffle: bool = True):
        return self._make_loader(dataset, shuffle)

    def _setup_scheduler(self, total_steps: int) -> None:
        self.scheduler = build_scheduler(self.config, total_steps)
        if getattr(self.config, "use_lr_scheduler", True):
            self.engine.set_lr(self.scheduler.current_lr())

    def train_epoch(self, loader, epoch: int) -> Dict[str, float]:
        accum = max(self.config.gradient_accumulation_steps, 1)
        t0 = time.perf_counter()
        sum_loss, n_flush, best = 0.0, 0, float("inf")
        log_every = max(int(getattr(self.config, "log_every_n_steps", 50)), 1)
        for i, batch in enumerate(loader):
            if self.should_stop:
                break
            self.train_step(batch)
            if (i + 1) % accum:
                continue
            self.optimizer_step()
            if self.global_step % log_every == 0:
                m = self._flush_metrics()
                if m:
                    sum_loss += m["loss"]
                    n_flush += 1
                    best = min(best, m["loss"])
                    self._log_step(epoch, m)
                    if not math.isfinite(m["loss"]):
                        self.logger.warning("non-finite loss at step %d", self.global_step)
                    if self.chinchilla_scaler is not None:
                        self.chinchilla_scaler.update_metrics(self.global_step, m["loss"], m["tokens_per_second"], m["grad_norm"])
                        if self.global_step % 100 == 0 and self.chinchilla_scaler.should_stop_early():
                            self.should_stop = True
                try:
                    ops.check_status()
                except ops.KernelError:
                    raise
            rebalance = int(getattr(self.config, "expert_rebalance_interval", 0) or 0)
            if rebalance and self.global_step % rebalance == 0:
                self.rebalance_experts()
            every = getattr(self.config, "save_every_n_batches", 0)
            if every and self.global_step % every == 0:
                self.save_checkpoint(epoch, tag=f"step_{self.global_step}")
            self._maybe_backup(epoch)
        m = self._flush_metrics()
        if m:
            sum_loss += m["loss"]
            n_flush += 1
            best = min(best, m["loss"])
        dt = time.perf_counter() - t0
        self.metrics["epoch_times"].append(dt)
        return {"avg_loss": sum_loss / max(n_flush, 1), "best_loss": best, "epoch_time": dt, "steps": self.global_step}

    def _log_step(self, epoch: int, m: Dict[str, float]) -> None:
        if get_rank() != 0:
            return
        mem = torch.cuda.max_memory_allocated() / 2 ** 30 if self.device.type == "cuda" else 0.0
        rate = "%.0f tok/s | " % m["tokens_per_second"] if getattr(self.config, "log_throughput", True) else ""
        self.logger.info("epoch %d step %d | loss %.4f ppl %.2f acc %.3f | lr %.3e | gnorm %.3f | %s%s | %.1f GB",
                         epoch, self.global_step, m["loss"], m["perplexity"], m["accuracy"], m["lr"], m["grad_norm"],
                         rate, self.config.precision, mem)

    def train(self, train_dataset, eval_dataset=None) -> Dict[str, Any]:
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        loader = self._make_loader(train_dataset, shuffle=True)
        accum = max(self.config.gradient_accumulation_steps, 1)
        try:
            steps_per_epoch = max(len(loader) // accum, 1)
        except TypeError:
            steps_per_epoch = 1000
        if self.scheduler is None:
            self._setup_scheduler(steps_per_epoch * self.config.num_epochs)
        summary: Dict[str, Any] = {"epochs": []}
        try:
            for epoch in range(self.current_epoch, self.config.num_epochs):
                self.current_epoch = epoch
                ep = self.train_epoch(loader, epoch)
                if eval_dataset is not None:
                    ev = self.evaluate(eval_dataset)
                    ep.update(ev)
                    if ev and ev["eval_loss"] < self.best_eval_loss:
                        self.best_eval_loss = ev["eval_loss"]
                        self.patience_counter = 0
                    else:
                        self.patience_counter += 1
                    pat = self.config.early_stopping_patience
                    if pat and self.patience_counter >= pat:
                        self.should_stop = True
                if getattr(self.config, "profile_memory", False):
                    if self.device.type == "cuda":
                        self.peak_memory_gb.append(torch.cuda.max_memory_allocated(self.device) / 2 ** 30)
                        torch.cuda.reset_peak_memory_stats(self.device)
                    else:
                        import resource
                        self.peak_memory_gb.append(resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 2 ** 20)
                path = self.save_checkpoint(epoch)
                self.checkpoint_history.append({"epoch": epoch, "global_step": self.global_step, "path": path})
                self.checkpoint_history = self.checkpoint_history[-10:]
                summary["epochs"].append(ep)
                if self.should_stop:
                    break
                loader = self._make_loader(train_dataset, shuffle=True)
        finally:
            try:
                prof = self.profiling_summary()
                if prof:
                    summary["profiling"] = prof
                    if get_rank() == 0:
                        self.logger.info("profiling: %s", prof)
                summary["final_checkpoint"] = self.save_checkpoint(self.current_epoch, tag="final")
            except Exception as e:  # never mask the original error
                self.logger.warning("final checkpoint failed: %s", e)
        summary["global_step"] = self.global_step
        summary["best_eval_loss"] = self.best_eval_loss
        return summary

    def _maybe_backup(self, epoch: int) -> None:
        """``backup_every_n_hours``: a rolling ``checkpoint_backup.pt`` on a wall-clock period, independent of the step- and
        epoch-based saves (the reference reads the flag only in a loop it never imports, ``training_loop.py``).  The clock is
        rank 0's, broadcast when several ranks train, so that every rank enters the collective save together."""
        hours = float(getattr(self.config, "backup_every_n_hours", 0) or 0)
        if hours <= 0:
            return
        import torch.distributed as dist
        due = time.time() - self._last_backup >= hours * 3600.0
        if dist.is_initialized() and dist.get_world_size() > 1:
            flag = torch.tensor([int(due)], device=self.device if self.device.type == "cuda" else "cpu")
            dist.broadcast(flag, 0)
            due = bool(flag.item())
        if due:
            self._last_backup = time.time()
            self.save_checkpoint(epoch, tag="backup")

    def train_with_oom_fallback(self, train_dataset, eval_dataset=None, max_attempts: Optional[int] = None) -> Dict[str, Any]:
        """Retry with half the micro-batch and twice the accumulation after an out-of-memory error
        (reference ``trainer.py:1836-1955``); the working pair is written to ``optimal_batch_config.json``.  ``max_attempts``
        defaults to the configuration's ``max_retries`` (10 when that is unset)."""
        if max_attempts is None:
            max_attempts = int(getattr(self.config, "max_retries", 10) or 10)
        attempts = 0
        while True:
            try:
                res = self.train(train_dataset, eval_dataset)
                self._write_batch_config()
                return res
            except Exception as e:
                if not is_oom_error(e) or attempts >= max_attempts:
                    raise
                attempts += 1
                old = self.config.micro_batch_size or self.config.batch_size
                if old <= 1 and self.config.gradient_accumulation_steps >= 32:
                    raise
                self.engine.zero_grad()
                self._pending_device.clear()
                gc.collect()
                if self.device.type == "cuda":
                    torch.cuda.empty_cache()
                new = max(old // 2, 1)
                self.config.micro_batch_size = new
                self.config.batch_size = new
                self.config.gradient_accumulation_steps = min(self.config.gradient_accumulation_steps * 2, 32)
                self.engine.grad_accumulation_steps = self.config.gradient_accumulation_steps
                self.logger.warning("OOM: retry %d with micro-batch %d, accumulation %d", attempts, new,
                                    self.config.gradient_accumulation_steps)

    def _write_batch_config(self) -> None:
        try:
            os.makedirs(self.checkpoint_manager.directory, exist_ok=True)
            with open(os.path.join(self.checkpoint_manager.directory, "optimal_batch_config.json"), "w") as f:
                json.dump({"micro_batch_size": self.config.micro_batch_size,
                           "gradient_accumulation_steps": self.config.gradient_accumulation_steps}, f)
        except OSError:
            pass

    def shutdown(self, leaving: bool = False) -> None:
        """Stop the heartbeat thread.  ``leaving=True`` announces an orderly departure to the peers (only between steps)."""
        if self.heartbeat is not None:
            (self.heartbeat.leave if leaving else self.heartbeat.stop)()
            self.heartbeat = None

    def inject_oom(self, at_micro_step: Optional[int] = None) -> None:
        """Host-side fault injection: the next (or the given) micro-step raises a synthetic OOM."""
        self._inject_oom_at = self.micro_step if at_micro_step is None else at_micro_step

    # ------------------------------------------------------------------------------------------------------
    # checkpoints
    # ------------------------------------------------------------------------------------------------------
    def save_checkpoint(self, epoch: int, tag: Optional[str] = None) -> Optional[str]:
        if self.device.type == "cuda":
            ops.check_status()  # never write a state that a timed-out kernel wait may have left half-updated
        return self.checkpoint_manager.save_checkpoint(
            self.model, self.engine, self.scheduler, self.global_step, epoch, self.metrics, tag, mesh=self.mesh)

    def load_checkpoint(self, path: str = "latest", strict: bool = True) -> Dict[str, Any]:
        info = self.checkpoint_manager.load_checkpoint(path, self.model, self.engine, self.scheduler, strict=strict)
        self.global_step = info.get("global_step", 0)
        self.current_epoch = info.get("epoch", 0)
        return info

    def rollback_steps(self, n: int = 100) -> bool:
        """Reload the history checkpoint closest to ``global_step - n`` (reference ``trainer.py:1727-1786``)."""
        if not self.checkpoint_history:
            return False
        target = self.global_step - n
        entry = min(self.checkpoint_history, key=lambda e: abs(e["global_step"] - target))
        if not entry.get("path") or not os.path.exists(entry["path"]):
            return False
        try:
            self.load_checkpoint(entry["path"])
        except Exception as e:  # e.g. the architecture changed since that checkpoint (expert add / prune)
            self.logger.warning("rollback to %s failed: %s", entry["path"], e)
            return False
        for k in ("train_losses", "gradient_norms", "learning_rates", "tokens_per_second", "accuracies"):
            keep = max(len(self.metrics[k]) - n, 0)
            self.metrics[k] = self.metrics[k][:keep]
        self.engine.zero_grad()
        return True

    # ------------------------------------------------------------------------------------------------------
    # interventions
    # ------------------------------------------------------------------------------------------------------
    def _at_step_boundary(self, fn: Callable[[], None]) -> None:
        """Run now when called from the training thread, otherwise at the next step boundary."""
        if threading.current_thread() is self._train_thread:
            fn()
        else:
            with self._lock:
                self._pending.append(fn)

    def adjust_learning_rate(self, new_lr: float, grace_period: int = 10, emergency: bool = False) -> None:
        def apply():
            self.engine.set_lr(new_lr)
            self.config.learning_rate = new_lr
            self.adaptive_lr_override = True
            self.lr_override_steps_left = grace_period
            self.lr_override_emergency = emergency
            self.recent_grad_norms.clear()
        self._at_step_boundary(apply)

    def emergency_lr_reduction(self, reduction_factor: float = 10.0) -> float:
        new_lr = self.engine.get_lr() / reduction_factor
        self.config.learning_rate = self.config.learning_rate / reduction_factor

        def apply():
            self.engine.set_lr(new_lr)
            if self.scheduler is not None:
                self.scheduler.scale_base(1.0 / reduction_factor)
        self._at_step_boundary(apply)
        return new_lr

    def adjust_weight_decay(self, value: float) -> None:
        self.config.weight_decay = value
        self._at_step_boundary(lambda: self.engine.set_weight_decay(value))

    def _update_optimizer_param_groups(self, name: str, value: float) -> None:
        if name == "lr":
            self.engine.set_lr(value)
        elif name == "weight_decay":
            self.engine.set_weight_decay(value)
        else:
            raise KeyError(name)

    def adjust_batch_size(self, new_batch_size: int) -> None:
        """Keeps the effective batch: accumulation = max(1, old_effective // new)."""
        old_eff = (self.config.micro_batch_size or self.config.batch_size) * self.config.gradient_accumulation_steps
        self.config.batch_size = new_batch_size
        self.config.micro_batch_size = new_batch_size
        self.config.gradient_accumulation_steps = max(1, old_eff // new_batch_size)
        self.engine.grad_accumulation_steps = self.config.gradient_accumulation_steps

    # -- MoE ----------------------------------------------------------------------------------------------
    def _moe_layers(self, layer_idx: Optional[int] = None) -> List[MoEFFNLayer]:
        layers = self.model.get_moe_layers()
        if layer_idx is None:
            return layers
        return [l for l in layers if l.layer_idx == layer_idx]

    @torch.no_grad()
    def add_expert(self, layer_idx: Optional[int] = None) -> int:
        """Append one expert to the targeted MoE layers: weights = mean of the existing experts + N(0, 0.01) noise,
        new gate row N(0, 0.01); optimiser state of surviving parameters is kept (reference ``trainer.py:1270-1376``).

        Under expert parallelism every rank appends one expert to ITS experts (mean of its local experts), so the layer
        grows by ``ep_size`` experts and stays evenly divided; global expert ids are re-planned as rank-major blocks
        (rank r owns ids ``r * E_local .. (r + 1) * E_local - 1``) and the replicated gate matrix gets its new rows at the
        end of every rank's block, drawn from a generator seeded identically on all ranks.  Returns the number of layers
        changed."""
        changed = 0
        maps: Dict[str, List[int]] = {}
        for layer in self._moe_layers(layer_idx):
            W = layer.ep_size
            e_local = layer.num_experts // W
            local_rows = list(range(e_local)) + [-1]
            gate_rows: List[int] = []
            for r in range(W):
                gate_rows += [r * e_local + j for j in range(e_local)] + [-1]
            prefix = f"layers.{layer.layer_idx}.ffn."
            maps[prefix + "experts_w1"] = local_rows
            maps[prefix + "experts_w2"] = local_rows
            maps[prefix + "gate.weight"] = gate_rows
            for attr in ("experts_w1", "experts_w2"):
                w = getattr(layer, attr)
                new = w.data.float().mean(0, keepdim=True) + 0.01 * torch.randn_like(w.data[:1].float())
                p = nn.Parameter(torch.cat([w.data, new.to(w.dtype)], dim=0))
                p._ats_expert = True
                setattr(layer, attr, p)
            g = layer.gate.weight
            gen = torch.Generator().manual_seed(7919 * (layer.layer_idx + 1) + layer.num_experts)  # same rows on every rank
            fresh = (0.01 * torch.randn(W, g.shape[1], generator=gen)).to(device=g.device, dtype=g.dtype)
            blocks = []
            for r in range(W):
                blocks += [g.data[r * e_local:(r + 1) * e_local], fresh[r:r + 1]]
            layer.gate.weight = nn.Parameter(torch.cat(blocks, dim=0))
            layer.gate.out_features += W
            layer.num_experts += W
            if layer.ep is not None:
                layer.ep.num_experts = layer.num_experts
            layer.expert_demand = torch.zeros(layer.num_experts, dtype=torch.float64, device=g.device)
            changed += 1
        if changed:
            self.model.config.num_experts = max(l.num_experts for l in self.model.get_moe_layers())
            self.config.num_experts = self.model.config.num_experts
            self.engine.rebuild(maps)
        return changed

    @torch.no_grad()
    def prune_expert(self, layer_idx: int, expert_idx: int) -> bool:
        """Remove one expert and its gate row; its optimiser state is dropped with it (the reference leaves the
        dead parameters in the optimiser, ``trainer.py:1408-1426``).

        Under expert parallelism the layer must stay evenly divided, so the expert at the same LOCAL position as
        ``expert_idx`` is removed on every rank (``ep_size`` experts in all, the named one among them) and the remaining
        experts keep their order inside every rank's block of ids."""
        done = False
        maps: Dict[str, List[int]] = {}
        for layer in self._moe_layers(layer_idx):
            W = layer.ep_size
            e_local = layer.num_experts // W
            if not 0 <= expert_idx < layer.num_experts or e_local < 2 or layer.num_experts - W < max(layer.top_k, 2):
                return False
            slot = expert_idx % e_local
            keep_local = [i for i in range(e_local) if i != slot]
            keep_gate = [r * e_local + i for r in range(W) for i in keep_local]
            prefix = f"layers.{layer.layer_idx}.ffn."
            maps[prefix + "experts_w1"] = keep_local
            maps[prefix + "experts_w2"] = keep_local
            maps[prefix + "gate.weight"] = keep_gate
            for attr in ("experts_w1", "experts_w2"):
                w = getattr(layer, attr)
                p = nn.Parameter(w.data[keep_local].clone())
                p._ats_expert = True
                setattr(layer, attr, p)
            g = layer.gate.weight
            layer.gate.weight = nn.Parameter(g.data[keep_gate].clone())
            layer.gate.out_features -= W
            layer.num_experts -= W
            if layer.ep is not None:
                layer.ep.num_experts = layer.num_experts
            layer.expert_demand = torch.zeros(layer.num_experts, dtype=torch.float64, device=g.device)
            done = True
        if done:
            self.model.config.num_experts = max(l.num_experts for l in self.model.get_moe_layers())
            self.config.num_experts = self.model.config.num_experts
            self.engine.rebuild(maps)
        return done

    def adjust_capacity_factor(self, factor: float) -> None:
        self.config.capacity_factor = factor
        self.model.config.capacity_factor = factor
        for l in self.model.get_moe_layers():
            l.capacity_factor = factor

    def adjust_routing_temperature(self, temperature: float) -> None:
        self.config.routing_temperature = temperature
        self.model.config.routing_temperature = temperature
        for l in self.model.get_moe_layers():
            l.routing_temperature = temperature

    def enable_expert_dropout(self, p: float) -> None:
        """Randomly drops non-primary routed experts of a token during training (the reference attaches an
        ``nn.Dropout`` no forward uses, ``trainer.py:1510-1514``)."""
        for l in self.model.get_moe_layers():
            l.expert_dropout = float(p)

    def rebalance_experts(self) -> Optional[Dict[str, Any]]:
        """Exchange hot experts between expert-parallel ranks (``parallel/load_balance.py``); collective, between steps.
        Returns the balancer's report, or ``None`` when the layout leaves nothing to move."""
        mesh = self.mesh
        if mesh is None or mesh.ep_size < 2 or not self.model.get_moe_layers():
            return None
        if self.model.get_moe_layers()[0].num_experts // mesh.ep_size < 2:
            return None  # one expert per rank: every placement loads the ranks alike
        from ..parallel.load_balance import ExpertLoadBalancer
        # built per call: experts may have been added or pruned since the last one
        balancer = ExpertLoadBalancer(self.model, mesh, self.engine if hasattr(self.engine, "read_rows") else None,
                                      tolerance=float(getattr(self.config, "expert_rebalance_tolerance", 0.1)))
        report = balancer.balance()
        if report["swaps"] and self.logger is not None:
            worst = max(r["before"] for r in report["layers"])
            after = max(r["after"] for r in report["layers"])
            self.logger.info("expert rebalance at step %d: %d exchanges, heaviest rank / mean %.2f -> %.2f", self.global_step,
                             report["swaps"], worst, after)
        return report

    def get_expert_statistics(self) -> Dict[str, Any]:
        per_layer = self.model.get_routing_statistics()
        imb = [v["imbalance_ratio"] for v in per_layer.values()]
        return {"layers": per_layer, "avg_imbalance": sum(imb) / len(imb) if imb else 1.0,
                "max_imbalance": max(imb) if imb else 1.0}

    def adjust_mod_capacity(self, capacity: float) -> None:
        self.config.mod_capacity_factor = capacity
        self.model.config.mod_capacity_factor = capacity
        for l in self.model.get_mod_layers():
            l.router.capacity_factor = capacity

    def get_mod_statistics(self) -> Dict[str, Any]:
        per_layer = self.model.get_mod_statistics()
        ratios = [v["selected_ratio"] for v in per_layer.values()]
        avg = sum(ratios) / len(ratios) if ratios else 1.0
        return {"layers": per_layer, "avg_selected_ratio": avg, "total_compute_savings": 1.0 - avg}

    # -- metrics --------------------------------------------------------------------------------------------
    def _extract_moe_routing_stats(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for name, st in self.model.get_routing_statistics().items():
            for j, u in enumerate(st["expert_usage"]):
                out[f"{name}_expert_{j}"] = 100.0 * u
        return out

    def _calculate_throughput(self) -> float:
        w = list(self._tokens_window)
        return sum(w) / len(w) if w else 0.0

    def _get_memory_usage(self) -> Dict[str, float]:
        if self.device.type == "cuda":
            return {"gpu_allocated_gb": torch.cuda.memory_allocated() / 2 ** 30,
                    "gpu_reserved_gb": torch.cuda.memory_reserved() / 2 ** 30,
                    "gpu_peak_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
        try:
            import psutil
            return {"cpu_rss_gb": psutil.Process().memory_info().rss / 2 ** 30}
        except Exception:
            return {}

    def get_current_metrics(self) -> TrainingMetrics:
        self._flush_metrics()
        tl, gn = self.metrics["train_losses"], self.metrics["gradient_norms"]
        return TrainingMetrics(epoch=self.current_epoch, step=self.global_step, loss=tl[-1] if tl else 0.0,
                               grad_norm=gn[-1] if gn else 0.0, learning_rate=self.engine.get_lr(),
                               expert_utilization=self._extract_moe_routing_stats() if self.model.config.use_moe else {},
                               memory_usage=self._get_memory_usage(), throughput=self._calculate_throughput())

    def get_quantization_status(self) -> Dict[str, Any]:
        return self.quantization_manager.status()


class MoEOptimizationManager:
    """Expert-parallel sizing and routing-balance diagnostics (reference ``trainer.py:804-982``)."""

    def __init__(self, config: Config):
        self.config = config
        self.routing_history: deque = deque(maxlen=100)

    def calculate_optimal_expert_parallel_size(self, world: int, balance: float = 1.0) -> int:
        """Largest divisor of both the world size and the expert count, scored by
        ``min(experts_per_rank / 4, 1) * balance / ep`` ... with NVSwitch all-to-all cost is flat, so the widest
        legal EP (fewest experts per rank, least weight memory) wins unless balance is poor."""
        e = self.config.num_experts
        cands = [d for d in range(1, world + 1) if world % d == 0 and e % d == 0]
        if balance < 0.5:
            return cands[len(cands) // 2]
        return cands[-1]

    def monitor_routing_balance(self, usage: List[float]) -> Dict[str, float]:
        if not usage:
            return {"balance": 1.0, "collapsed": 0.0}
        mean = sum(usage) / len(usage)
        dev = sum(abs(u - mean) for u in usage) / (2 * max(mean * len(usage), 1e-9))
        self.routing_history.append(1.0 - dev)
        collapsed = float(min(usage) < 0.01 * mean * len(usage) / len(usage) and max(usage) > 0.5)
        return {"balance": 1.0 - dev, "collapsed": collapsed}

    def deepspeed_moe_block(self) -> Dict[str, Any]:
        c = self.config
        return {"enabled": c.use_moe, "num_experts": c.num_experts, "top_k": c.moe_top_k,
                "capacity_factor": c.capacity_factor, "expert_parallel_size": c.expert_parallel_size or 1,
                "min_capacity": 4, "drop_tokens": bool(getattr(c, "drop_tokens", True))}


def profile_training_loop_overhead(trainer: EnhancedConversationTrainer, dataloader: Iterable, n: int = 10) -> Dict[str, float]:
    """Per-phase device time with CUDA events (host time on CPU): to_device / forward+backward / optimizer
    (reference ``trainer.py:3821-3978`` uses wall clock with synchronize fences)."""
    from ..utils.profiler import PhaseTimer
    timer = PhaseTimer(trainer.device)
    it = iter(dataloader)
    for _ in range(n):
        try:
            batch = next(it)
        except StopIteration:
            break
        with timer.phase("to_device"):
            batch = trainer._to_device(batch)
        with timer.phase("forward_backward"):
            trainer.train_step(batch)
        with timer.phase("optimizer"):
            trainer.optimizer_step()
    return timer.summary()

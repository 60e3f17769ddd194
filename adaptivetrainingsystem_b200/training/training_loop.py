"""Stand-alone training loop with health monitoring, periodic evaluation and checkpoint retention.

The reference ships an older loop beside its trainer (reference ``training/training_loop.py:1-446``) that fills a
``metrics`` dictionary, consults a health monitor, evaluates and saves on fixed step intervals -- and installs itself by
monkey-patching the trainer class on import (``:432-447``).  The behaviour is kept, the patching is not: ``TrainingLoop``
wraps any trainer that offers ``train_step`` / ``optimizer_step`` / ``evaluate`` and leaves the class untouched.
"""
from __future__ import annotations

import math
import time
from typing import Any, Dict, Iterable, List, Optional

import torch

from ..monitoring.logger import TrainingHealthMonitor
from .checkpoint import CheckpointManager


class TrainingLoop:
    def __init__(self, trainer, checkpoint_manager: Optional[CheckpointManager] = None,
                 health_monitor: Optional[TrainingHealthMonitor] = None, eval_every_n_steps: int = 0, save_every_n_steps: int = 0,
                 log_every_n_steps: int = 50, max_steps: Optional[int] = None, early_stopping_patience: int = 0):
        self.trainer = trainer
        self.config = trainer.config
        self.checkpoints = checkpoint_manager
        self.health = health_monitor or TrainingHealthMonitor()
        self.eval_every = eval_every_n_steps or int(getattr(self.config, "eval_every_n_batches", 0) or 0)
        self.save_every = save_every_n_steps or int(getattr(self.config, "save_every_n_batches", 0) or 0)
        self.log_every = log_every_n_steps
        self.max_steps = max_steps
        self.patience = early_stopping_patience or int(getattr(self.config, "early_stopping_patience", 0) or 0)
        self.metrics: Dict[str, List[float]] = {k: [] for k in ("train_losses", "eval_losses", "learning_rates", "gradient_norms",
                                                               "throughput", "epoch_times")}
        self.global_step = 0
        self.best_eval = math.inf
        self._bad_evals = 0
        self.should_stop = False

    # -- one epoch ------------------------------------------------------------------------------------------------
    def train_epoch(self, loader: Iterable[Dict[str, torch.Tensor]], epoch: int, eval_dataset=None) -> Dict[str, float]:
        accum = max(int(self.config.gradient_accumulation_steps), 1)
        t0 = time.time()
        tokens = 0
        losses: List[float] = []
        micro = 0
        for batch in loader:
            out = self.trainer.train_step(batch)
            micro += 1
            tokens += int(batch["input_ids"].numel())
            if micro % accum:
                continue
            stats = self.trainer.optimizer_step()
            self.global_step += 1
            loss = float(out["loss"])
            gnorm = float(stats.get("grad_norm", 0.0))
            lr = float(self.trainer.engine.get_lr()) if hasattr(self.trainer, "engine") else float(stats.get("lr", 0.0))
            losses.append(loss)
            self.metrics["train_losses"].append(loss)
            self.metrics["gradient_norms"].append(gnorm)
            self.metrics["learning_rates"].append(lr)
            elapsed = max(time.time() - t0, 1e-9)
            self.metrics["throughput"].append(tokens / elapsed)
            self.health.update(self.global_step, loss, grad_norm=gnorm, learning_rate=lr, throughput=tokens / elapsed)
            if not math.isfinite(loss):
                self.should_stop = True
                break
            if self.eval_every and eval_dataset is not None and self.global_step % self.eval_every == 0:
                self._evaluate(eval_dataset, epoch)
            if self.save_every and self.global_step % self.save_every == 0:
                self._save(epoch, {"loss": loss})
            if self.max_steps and self.global_step >= self.max_steps:
                self.should_stop = True
            if self.should_stop:
                break
        dt = time.time() - t0
        self.metrics["epoch_times"].append(dt)
        return {"avg_loss": sum(losses) / max(len(losses), 1), "steps": len(losses), "tokens": tokens, "seconds": dt,
                "tokens_per_sec": tokens / max(dt, 1e-9)}

    def _evaluate(self, eval_dataset, epoch: int) -> Dict[str, float]:
        res = self.trainer.evaluate(eval_dataset)
        ev = float(res.get("eval_loss", res.get("loss", math.nan)))
        self.metrics["eval_losses"].append(ev)
        if ev < self.best_eval - 1e-6:
            self.best_eval = ev
            self._bad_evals = 0
            self._save(epoch, {"eval_loss": ev}, is_best=True)
        else:
            self._bad_evals += 1
            if self.patience and self._bad_evals >= self.patience:
                self.should_stop = True
        return res

    def _save(self, epoch: int, metrics: Dict[str, float], is_best: bool = False) -> Optional[str]:
        if self.checkpoints is None:
            return self.trainer.save_checkpoint(epoch) if hasattr(self.trainer, "save_checkpoint") else None
        return self.checkpoints.save_checkpoint(self.trainer.model, getattr(self.trainer, "engine", None), getattr(self.trainer, "scheduler", None),
                                                self.global_step, epoch, self.metrics, is_best=is_best, eval_loss=metrics.get("eval_loss"))

    # -- whole run ------------------------------------------------------------------------------------------------
    def train(self, train_dataset, eval_dataset=None, num_epochs: Optional[int] = None) -> Dict[str, Any]:
        epochs = int(num_epochs or self.config.num_epochs)
        history = []
        for epoch in range(epochs):
            loader = self.trainer._make_loader(train_dataset, shuffle=True)
            stats = self.train_epoch(loader, epoch, eval_dataset)
            if eval_dataset is not None and not self.eval_every:
                stats.update(self._evaluate(eval_dataset, epoch))
            history.append(stats)
            if self.should_stop:
                break
        return {"epochs": history, "global_step": self.global_step, "best_eval_loss": self.best_eval, "metrics": self.metrics,
                "health": self.health.get_report()}

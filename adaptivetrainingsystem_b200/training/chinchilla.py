"""Chinchilla-style epoch planner with convergence detection, compute-efficiency tracking and an adaptive curriculum.

API of the reference (``training/chinchilla_scaler.py``): ``EnhancedChinchillaScaler(config, model, dataset)`` with
``get_optimal_epochs``, ``update_metrics``, ``should_stop_early``, ``get_status_report``, ``save_state``; helper classes
``ConvergenceDetector`` (``:38-106``), ``ComputeEfficiencyTracker`` (``:117-118``: 6 N FLOPs per token),
``AdaptiveCurriculumManager`` (``:155-174``).  Rule (``:237-242``): epochs = ceil(multiplier * N / dataset_tokens)
clamped to ``[min_auto_epochs, max_auto_epochs]``, re-planned every 500 steps.  For sparse models ``N`` is the ACTIVE
parameter count (what each token trains), which the reference does not distinguish.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import time
from collections import deque
from typing import Any, Deque, Dict, List, Optional


class ConvergenceDetector:
    """Plateau / divergence / oscillation classification over a sliding window of losses."""

    def __init__(self, window: int = 100, plateau_threshold: float = 1e-3, patience: int = 5):
        self.losses: Deque[float] = deque(maxlen=10 * window)
        self.window, self.plateau_threshold, self.patience = window, plateau_threshold, patience
        self.plateau_count = 0
        self.best = float("inf")

    def update(self, loss: float) -> Dict[str, Any]:
        if math.isfinite(loss):
            self.losses.append(loss)
            self.best = min(self.best, loss)
        return self.status()

    def status(self) -> Dict[str, Any]:
        n = len(self.losses)
        if n < 2 * self.window:
            return {"state": "warming_up", "score": 0.0, "improvement": float("nan")}
        l = list(self.losses)
        prev = statistics.fmean(l[-2 * self.window:-self.window])
        cur = statistics.fmean(l[-self.window:])
        imp = (prev - cur) / max(abs(prev), 1e-12)
        sd = statistics.pstdev(l[-self.window:])
        if imp < -0.05:
            state = "diverging"
        elif abs(imp) < self.plateau_threshold:
            self.plateau_count += 1
            state = "plateau" if self.plateau_count >= self.patience else "slowing"
        elif sd > 0.25 * max(abs(cur), 1e-12):
            state = "oscillating"
        else:
            self.plateau_count = 0
            state = "improving"
        score = max(0.0, min(1.0, 1.0 - abs(imp) / max(10 * self.plateau_threshold, 1e-12)))
        return {"state": state, "score": score, "improvement": imp, "best": self.best}


class ComputeEfficiencyTracker:
    """Loss reduction per PFLOP spent; ``flops_per_token = 6 * N_active`` (forward + backward)."""

    def __init__(self, active_params: int):
        self.flops_per_token = 6.0 * active_params
        self.samples: List[Dict[str, float]] = []
        self.total_tokens = 0.0

    def update(self, step: int, loss: float, tokens: float) -> None:
        self.total_tokens += tokens
        self.samples.append({"step": step, "loss": loss, "pflops": self.total_tokens * self.flops_per_token / 1e15})

    def efficiency(self, window: int = 50) -> float:
        if len(self.samples) < 2 * window:
            return float("nan")
        a, b = self.samples[-2 * window], self.samples[-1]
        dp = b["pflops"] - a["pflops"]
        return (a["loss"] - b["loss"]) / dp if dp > 0 else float("nan")

    def efficiency_decline(self, window: int = 50) -> float:
        """1 - recent efficiency / peak efficiency (0 = still at peak, 1 = no more progress per FLOP)."""
        if len(self.samples) < 4 * window:
            return 0.0
        effs = []
        for i in range(2 * window, len(self.samples), window):
            a, b = self.samples[i - 2 * window], self.samples[i]
            dp = b["pflops"] - a["pflops"]
            if dp > 0:
                effs.append((a["loss"] - b["loss"]) / dp)
        if not effs or max(effs) <= 0:
            return 0.0
        return max(0.0, 1.0 - effs[-1] / max(effs))


class AdaptiveCurriculumManager:
    """Difficulty in [0, 1] that grows while the model keeps improving (sequence-length / MoD-capacity curricula read it)."""

    def __init__(self, start: float = 0.3, step: float = 0.05):
        self.difficulty, self.step = start, step

    def update(self, convergence_state: str) -> float:
        if convergence_state in ("improving", "slowing"):
            self.difficulty = min(1.0, self.difficulty + self.step)
        elif convergence_state == "diverging":
            self.difficulty = max(0.1, self.difficulty - 2 * self.step)
        return self.difficulty

    def mod_capacity(self, start: float = 0.7, mid: float = 0.5, end: float = 0.3) -> float:
        """MoD capacity curriculum 0.7 -> 0.5 -> 0.3 (reference ``Main.py:1583-1586``)."""
        d = self.difficulty
        return start + (mid - start) * min(d / 0.5, 1.0) if d < 0.5 else mid + (end - mid) * ((d - 0.5) / 0.5)


class EnhancedChinchillaScaler:
    def __init__(self, config, model=None, dataset=None, dataset_tokens: Optional[int] = None):
        self.config = config
        mc = model.config if model is not None and hasattr(model, "config") else config.to_model_config()
        self.total_params = mc.num_parameters()
        self.active_params = mc.num_parameters(active_only=True)
        if dataset_tokens is None and dataset is not None:
            if hasattr(dataset, "total_tokens"):
                dataset_tokens = int(dataset.total_tokens())
            else:
                try:
                    dataset_tokens = len(dataset) * config.seq_length
                except TypeError:
                    dataset_tokens = 0
        self.dataset_tokens = int(dataset_tokens or 0)
        self.multiplier = float(getattr(config, "chinchilla_multiplier", 20.0))
        self.min_epochs = int(getattr(config, "min_auto_epochs", 1))
        self.max_epochs = int(getattr(config, "max_auto_epochs", 50))
        self.convergence = ConvergenceDetector(patience=int(getattr(config, "plateau_patience", 5)))
        self.efficiency = ComputeEfficiencyTracker(self.active_params)
        self.curriculum = AdaptiveCurriculumManager()
        self.replan_every = 500
        self.history: List[Dict[str, Any]] = []
        self.current_plan = self.get_optimal_epochs()
        self.stop_reason: Optional[str] = None

    @property
    def optimal_tokens(self) -> float:
        return self.multiplier * self.active_params

    def get_optimal_epochs(self) -> int:
        if self.dataset_tokens <= 0:
            return max(self.min_epochs, min(getattr(self.config, "num_epochs", 1), self.max_epochs))
        e = math.ceil(self.optimal_tokens / self.dataset_tokens)
        return int(max(self.min_epochs, min(e, self.max_epochs)))

    def update_metrics(self, step: int, loss: float, tokens_per_second: float = 0.0, grad_norm: float = 0.0,
                       tokens: Optional[float] = None) -> Dict[str, Any]:
        tok = tokens if tokens is not None else float(getattr(self.config, "effective_batch_size", 1) * self.config.seq_length)
        conv = self.convergence.update(loss)
        self.efficiency.update(step, loss, tok)
        if getattr(self.config, "enable_adaptive_curriculum", True):
            self.curriculum.update(conv["state"])
        if step and step % self.replan_every == 0:
            self._replan(conv)
        rec = {"step": step, "loss": loss, "state": conv["state"], "tps": tokens_per_second, "grad_norm": grad_norm}
        self.history.append(rec)
        return rec

    def _replan(self, conv: Dict[str, Any]) -> None:
        base = self.get_optimal_epochs()
        if conv["state"] == "plateau":
            base = max(self.min_epochs, math.ceil(base * 0.8))
        elif conv["state"] == "improving" and self.efficiency.efficiency_decline() < 0.1:
            base = min(self.max_epochs, math.ceil(base * 1.1))
        self.current_plan = base

    def should_stop_early(self) -> bool:
        if not getattr(self.config, "enable_early_stopping", True):
            return False
        st = self.convergence.status()
        if st["state"] == "diverging" and len(self.convergence.losses) > 4 * self.convergence.window:
            self.stop_reason = "loss diverging"
            return True
        if st["state"] == "plateau" and st["score"] >= float(getattr(self.config, "convergence_threshold", 0.85)):
            self.stop_reason = "converged (plateau)"
            return True
        if getattr(self.config, "enable_compute_efficiency", True) and \
                self.efficiency.efficiency_decline() > 1.0 - float(getattr(self.config, "efficiency_decline_threshold", 0.3)) and \
                self.efficiency.total_tokens > self.optimal_tokens:
            self.stop_reason = "compute efficiency collapsed past the Chinchilla budget"
            return True
        return False

    def get_status_report(self) -> Dict[str, Any]:
        return {"total_params": self.total_params, "active_params": self.active_params, "dataset_tokens": self.dataset_tokens,
                "optimal_tokens": self.optimal_tokens, "planned_epochs": self.current_plan,
                "tokens_seen": self.efficiency.total_tokens,
                "budget_fraction": self.efficiency.total_tokens / max(self.optimal_tokens, 1.0),
                "convergence": self.convergence.status(), "efficiency": self.efficiency.efficiency(),
                "efficiency_decline": self.efficiency.efficiency_decline(), "curriculum_difficulty": self.curriculum.difficulty,
                "stop_reason": self.stop_reason}

    def save_state(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump({"report": self.get_status_report(), "history": self.history[-2000:], "saved_at": time.time()}, f, indent=2,
                      default=lambda o: None if isinstance(o, float) and not math.isfinite(o) else str(o))


def auto_adjust_epochs_chinchilla(config, model, dataset) -> EnhancedChinchillaScaler:
    """Entry-script helper (reference ``Main.py:1404``): plans ``config.num_epochs`` and returns the scaler."""
    scaler = EnhancedChinchillaScaler(config, model, dataset)
    if getattr(config, "auto_epoch_scaling", True):
        config.num_epochs = scaler.get_optimal_epochs()
    return scaler

"""Training observability: windowed metric history with alert thresholds, trend and health score, phase detection and a
JSON health report; plus the ``ProductionLogger`` the orchestrator expects.

Follows the reference ``monitoring/logger.py`` (``TrainingAlert``, ``MetricsCollector`` ``:29-273`` with thresholds
``:39-46``, least-squares trend ``:223-244``, health score ``:246-273``; ``TrainingHealthMonitor`` ``:276-532`` with phase
detection ``:340-374`` and checks every 50 steps).  ``ProductionLogger`` is referenced by the reference orchestrator
(``orchestrator.py:683``) but absent from its tree; it exists here.
"""
from __future__ import annotations

import json
import logging
import math
import os
import statistics
import time
from collections import defaultdict, deque
from dataclasses import asdict, dataclass, field
from typing import Any, Deque, Dict, List, Optional


@dataclass
class TrainingAlert:
    level: str          # info | warning | critical
    metric: str
    value: float
    threshold: float
    message: str
    step: int = 0
    timestamp: float = field(default_factory=time.time)


class MetricsCollector:
    DEFAULT_THRESHOLDS = {"loss_spike_ratio": 2.0, "grad_norm_max": 100.0, "grad_norm_min": 1e-7, "lr_min": 1e-9,
                          "throughput_drop": 0.5, "memory_fraction": 0.95, "loss_max": 50.0}

    def __init__(self, window: int = 1000, thresholds: Optional[Dict[str, float]] = None):
        self.window = window
        self.history: Dict[str, Deque[float]] = defaultdict(lambda: deque(maxlen=window))
        self.steps: Dict[str, Deque[int]] = defaultdict(lambda: deque(maxlen=window))
        self.thresholds = {**self.DEFAULT_THRESHOLDS, **(thresholds or {})}
        self.alerts: List[TrainingAlert] = []

    def add(self, name: str, value: float, step: int = 0) -> List[TrainingAlert]:
        self.history[name].append(float(value))
        self.steps[name].append(step)
        new = self._check(name, float(value), step)
        self.alerts.extend(new)
        return new

    def add_many(self, metrics: Dict[str, float], step: int = 0) -> List[TrainingAlert]:
        out: List[TrainingAlert] = []
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                out.extend(self.add(k, v, step))
        return out

    def _check(self, name: str, v: float, step: int) -> List[TrainingAlert]:
        t, out = self.thresholds, []
        h = list(self.history[name])
        if not math.isfinite(v):
            return [TrainingAlert("critical", name, v, 0.0, f"{name} is not finite", step)]
        if name == "loss":
            if v > t["loss_max"]:
                out.append(TrainingAlert("critical", name, v, t["loss_max"], "loss above hard limit", step))
            if len(h) >= 20:
                base = statistics.fmean(h[-20:-1])
                if v > t["loss_spike_ratio"] * base:
                    out.append(TrainingAlert("warning", name, v, t["loss_spike_ratio"] * base, "loss spike", step))
        elif name == "grad_norm":
            if v > t["grad_norm_max"]:
                out.append(TrainingAlert("critical", name, v, t["grad_norm_max"], "gradient explosion", step))
            elif 0 <= v < t["grad_norm_min"]:
                out.append(TrainingAlert("warning", name, v, t["grad_norm_min"], "vanishing gradients", step))
        elif name == "throughput" and len(h) >= 20:
            base = statistics.fmean(h[-20:-1])
            if base > 0 and v < t["throughput_drop"] * base:
                out.append(TrainingAlert("warning", name, v, t["throughput_drop"] * base, "throughput dropped", step))
        elif name == "memory_fraction" and v > t["memory_fraction"]:
            out.append(TrainingAlert("warning", name, v, t["memory_fraction"], "device memory nearly full", step))
        return out

    def get(self, name: str, n: Optional[int] = None) -> List[float]:
        h = list(self.history.get(name, []))
        return h if n is None else h[-n:]

    def mean(self, name: str, n: int = 100) -> float:
        h = self.get(name, n)
        return statistics.fmean(h) if h else float("nan")

    def trend(self, name: str, n: int = 100) -> float:
        """Least-squares slope of the last n values per step."""
        ys = self.get(name, n)
        if len(ys) < 2:
            return 0.0
        xs = list(range(len(ys)))
        mx, my = statistics.fmean(xs), statistics.fmean(ys)
        den = sum((x - mx) ** 2 for x in xs) or 1e-12
        return sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den

    def health_score(self) -> float:
        """0..1: starts at 1, loses for non-improving loss, unstable gradients and recent alerts."""
        score = 1.0
        if len(self.get("loss")) >= 20 and self.trend("loss") > 0:
            score -= 0.3
        g = self.get("grad_norm", 50)
        if len(g) >= 10:
            m = statistics.fmean(g)
            if m > 0 and statistics.pstdev(g) / m > 1.0:
                score -= 0.2
        recent = [a for a in self.alerts[-20:] if time.time() - a.timestamp < 600]
        score -= 0.1 * sum(a.level == "warning" for a in recent) + 0.25 * sum(a.level == "critical" for a in recent)
        return max(0.0, min(1.0, score))

    def summary(self) -> Dict[str, Any]:
        return {k: {"last": v[-1], "mean": statistics.fmean(v), "min": min(v), "max": max(v), "n": len(v)}
                for k, v in ((k, list(d)) for k, d in self.history.items()) if v}


class TrainingHealthMonitor:
    def __init__(self, config=None, check_interval: int = 50, log_dir: Optional[str] = None):
        self.collector = MetricsCollector()
        self.check_interval = int(getattr(config, "health_check_interval", check_interval) or check_interval) if config else check_interval
        self.log_dir = log_dir
        self.phase = "warmup"
        self.start_time = time.time()
        self.last_check_step = 0
        self.reports: List[Dict[str, Any]] = []

    def update(self, step: int, loss: float, grad_norm: float = 0.0, learning_rate: float = 0.0, throughput: float = 0.0,
               **extra: float) -> List[TrainingAlert]:
        alerts = self.collector.add_many({"loss": loss, "grad_norm": grad_norm, "learning_rate": learning_rate,
                                          "throughput": throughput, **extra}, step)
        if step - self.last_check_step >= self.check_interval:
            self.last_check_step = step
            self.phase = self.detect_phase()
            self.reports.append(self.health_check(step))
        return alerts

    def detect_phase(self) -> str:
        loss = self.collector.get("loss")
        lr = self.collector.get("learning_rate", 50)
        if len(loss) < 50:
            return "warmup"
        if len(lr) >= 2 and lr[-1] > lr[0] * 1.05:
            return "warmup"
        slope = self.collector.trend("loss", 200)
        scale = max(abs(statistics.fmean(loss[-200:])), 1e-8)
        rel = slope / scale
        if rel < -1e-3:
            return "rapid_learning"
        if rel < -1e-5:
            return "steady_learning"
        if rel > 1e-4:
            return "diverging"
        return "plateau"

    def health_check(self, step: int) -> Dict[str, Any]:
        return {"step": step, "phase": self.phase, "health_score": self.collector.health_score(),
                "loss_trend": self.collector.trend("loss"), "alerts": len(self.collector.alerts),
                "elapsed_s": time.time() - self.start_time}

    def get_report(self) -> Dict[str, Any]:
        return {"phase": self.phase, "health_score": self.collector.health_score(), "metrics": self.collector.summary(),
                "alerts": [asdict(a) for a in self.collector.alerts[-50:]], "checks": self.reports[-20:]}

    def save_report(self, path: Optional[str] = None) -> str:
        path = path or os.path.join(self.log_dir or ".", "health_report.json")
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(self.get_report(), f, indent=2, default=str)
        return path


class ProductionLogger:
    """Rank-aware logger: console + ``training_<timestamp>.log`` file, structured metric lines as JSONL."""

    def __init__(self, log_level: str = "INFO", experiment_name: Optional[str] = None, log_dir: str = "logs", rank: int = 0):
        self.rank = rank
        self.logger = logging.getLogger(f"ats.{experiment_name or 'run'}")
        self.logger.setLevel(getattr(logging, str(log_level).upper(), logging.INFO))
        self.metrics_path = None
        if rank == 0 and not self.logger.handlers:
            fmt = logging.Formatter("%(asctime)s %(levelname)s %(message)s")
            sh = logging.StreamHandler()
            sh.setFormatter(fmt)
            self.logger.addHandler(sh)
            try:
                os.makedirs(log_dir, exist_ok=True)
                fh = logging.FileHandler(os.path.join(log_dir, time.strftime("training_%Y%m%d_%H%M%S.log")))
                fh.setFormatter(fmt)
                self.logger.addHandler(fh)
                self.metrics_path = os.path.join(log_dir, "metrics.jsonl")
            except OSError:
                pass

    def log_metrics(self, step: int, metrics: Dict[str, Any]) -> None:
        if self.rank != 0 or not self.metrics_path:
            return
        with open(self.metrics_path, "a") as f:
            f.write(json.dumps({"step": step, "time": time.time(), **{k: v for k, v in metrics.items() if isinstance(v, (int, float, str))}}) + "\n")

    def __getattr__(self, name):  # info / warning / error / debug pass through
        return getattr(self.logger, name)

"""Adaptive training orchestrator: watches the metric stream of a trainer, detects anomalies, and answers with
interventions (LR changes, rollback, expert add / prune, capacity / temperature tuning, OOM recovery).

API follows the reference (reference ``training/orchestrator.py:673-2160``): ``AdaptiveTrainingOrchestrator(config)``
with ``initialize_training``, ``run_adaptive_training``, ``get_adaptive_status``, ``cleanup``; data classes
``TrainingMetrics`` / ``AdaptiveDecision``; helpers ``MetaLearningEngine``, ``AdaptiveHyperparameterOptimizer``,
``ArchitectureEvolution``, ``RealTimeAnalytics``, ``ProductionMonitoring``.  Decision vocabulary (``:1040-1131``):
``learning_rate_adjustment, corrective_lr_reduction, optimization_lr_increase, emergency_lr_reduction,
plateau_intervention, divergence_prevention, checkpoint_rollback, add_expert, prune_expert, loss_spike_response``.

What is different: the monitor thread never touches optimiser state -- it posts decisions that the trainer applies at
the next step boundary; every decision type has a handler (the reference has none for ``loss_spike_response``);
``ProductionMonitoring`` reports measured values (the reference returns random numbers, ``:638-671``); the model the
orchestrator trains can be supplied by the caller (the reference silently builds a second one, ``:1155-1170``).
"""
from __future__ import annotations

import json
import logging
import math
import os
import pickle
import queue
import signal
import statistics
import threading
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Tuple

import torch

from .trainer import EnhancedConversationTrainer, TrainingMetrics, is_oom_error

log = logging.getLogger("ats.orchestrator")

CONFIDENCE_LADDER = {"soft": 0.70, "medium": 0.80, "hard": 0.90, "critical": 0.0}


@dataclass
class AdaptiveDecision:
    decision_type: str
    parameters: Dict[str, Any]
    confidence: float
    reasoning: str
    expected_improvement: float = 0.0
    timestamp: float = field(default_factory=time.time)
    applied: bool = False


class MetaLearningEngine:
    """Remembers past runs (config summary -> outcome) and suggests hyper-parameters for a new one."""

    def __init__(self, state_path: Optional[str] = None):
        self.state_path = state_path
        self.training_history: List[Dict[str, Any]] = []
        self.successful_strategies: List[Dict[str, Any]] = []
        self.failure_patterns: List[Dict[str, Any]] = []
        if state_path and os.path.exists(state_path):
            self.load(state_path)

    def record_run(self, config_summary: Dict[str, Any], final_loss: float, converged: bool, notes: str = "") -> None:
        rec = {"config": config_summary, "final_loss": final_loss, "converged": converged, "notes": notes, "time": time.time()}
        self.training_history.append(rec)
        (self.successful_strategies if converged else self.failure_patterns).append(rec)

    def suggest_hyperparameters(self, config_summary: Dict[str, Any]) -> Dict[str, float]:
        """Nearest successful run in (log params, log batch) space; falls back to a scaling rule lr ~ N^-0.25."""
        n = float(config_summary.get("parameters", 1e8))
        best, dist_best = None, float("inf")
        for r in self.successful_strategies:
            m = float(r["config"].get("parameters", 1e8))
            d = abs(math.log(max(m, 1.0)) - math.log(max(n, 1.0)))
            if d < dist_best:
                best, dist_best = r, d
        if best is not None and "learning_rate" in best["config"]:
            return {"learning_rate": float(best["config"]["learning_rate"]), "source_distance": dist_best}
        return {"learning_rate": float(min(6e-4, 3e-4 * (1.3e9 / max(n, 1.0)) ** 0.25)), "source_distance": float("inf")}

    def predict_training_trajectory(self, losses: List[float], horizon: int = 100) -> Dict[str, float]:
        """Power-law extrapolation loss ~ a * step^-b fitted on the recent history."""
        if len(losses) < 10:
            return {"predicted_loss": losses[-1] if losses else float("nan"), "slope": 0.0}
        xs = [math.log(i + 1) for i in range(len(losses))]
        ys = [math.log(max(l, 1e-8)) for l in losses]
        mx, my = statistics.fmean(xs), statistics.fmean(ys)
        den = sum((x - mx) ** 2 for x in xs) or 1e-12
        b = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den
        a = my - b * mx
        return {"predicted_loss": math.exp(a + b * math.log(len(losses) + horizon)), "slope": b}

    def save(self, path: Optional[str] = None) -> None:
        path = path or self.state_path
        if not path:
            return
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "wb") as f:
            pickle.dump({"history": self.training_history, "ok": self.successful_strategies, "bad": self.failure_patterns}, f)

    def load(self, path: str) -> None:
        try:
            with open(path, "rb") as f:
                d = pickle.load(f)
            self.training_history, self.successful_strategies, self.failure_patterns = d["history"], d["ok"], d["bad"]
        except Exception as e:  # a corrupt state file must not stop training
            log.warning("meta-learning state %s unreadable: %s", path, e)


class AdaptiveHyperparameterOptimizer:
    """Bounded multiplicative LR search driven by loss improvement per step."""

    def __init__(self, min_lr: float = 1e-7, max_lr: float = 1e-2):
        self.min_lr, self.max_lr = min_lr, max_lr
        self.trials: List[Tuple[float, float]] = []

    def observe(self, lr: float, improvement: float) -> None:
        self.trials.append((lr, improvement))

    def suggest(self, current_lr: float) -> float:
        if len(self.trials) < 4:
            return current_lr
        recent = self.trials[-4:]
        better = [lr for lr, imp in recent if imp > 0]
        if not better:
            return max(current_lr * 0.5, self.min_lr)
        if all(imp > 0 for _, imp in recent) and recent[-1][1] < 0.25 * recent[0][1]:
            return min(current_lr * 1.25, self.max_lr)
        return current_lr


class ArchitectureEvolution:
    """Expert-count policy: grow a layer whose busiest expert is over ``grow_at`` utilisation of capacity, prune an
    expert under ``prune_at`` of the uniform share; 4..16 experts per layer (reference ``Main.py:1576-1580``)."""

    def __init__(self, grow_at: float = 0.85, prune_at: float = 0.15, min_experts: int = 4, max_experts: int = 16):
        self.grow_at, self.prune_at, self.min_experts, self.max_experts = grow_at, prune_at, min_experts, max_experts

    def propose(self, layer_stats: Dict[str, Dict[str, Any]]) -> List[Dict[str, Any]]:
        out = []
        for name, st in layer_stats.items():
            usage = st.get("expert_usage") or []
            n = len(usage)
            if not n:
                continue
            layer_idx = int(name.split("_")[-1])
            uniform = 1.0 / n
            if max(usage) > self.grow_at and n < self.max_experts:
                out.append({"action": "add_expert", "layer_idx": layer_idx, "reason": f"expert holds {max(usage):.0%} of the traffic"})
            elif min(usage) < self.prune_at * uniform and n > self.min_experts:
                out.append({"action": "prune_expert", "layer_idx": layer_idx, "expert_idx": usage.index(min(usage)),
                            "reason": f"expert receives {min(usage):.2%} of the traffic"})
        return out


class RealTimeAnalytics:
    """Windowed anomaly detection (reference thresholds ``orchestrator.py:460-467, 555-628``)."""

    def __init__(self, window: int = 1000, min_samples: int = 50):
        self.history: Deque[TrainingMetrics] = deque(maxlen=window)
        self.min_samples = min_samples
        self.thresholds = {"loss_spike_sigma": 2.0, "loss_spike_abs": 0.1, "grad_explosion_abs": 100.0,
                           "grad_explosion_rel": 10.0, "expert_min_pct": 1.0, "expert_max_pct": 50.0,
                           "plateau_window": 200, "plateau_rel": 1e-3}

    def add(self, m: TrainingMetrics) -> None:
        self.history.append(m)

    def detect_training_anomalies(self, m: Optional[TrainingMetrics] = None) -> List[Dict[str, Any]]:
        if m is not None:
            self.add(m)
        out: List[Dict[str, Any]] = []
        h = list(self.history)
        if not h:
            return out
        cur = h[-1]
        if not math.isfinite(cur.loss):
            out.append({"type": "divergence", "severity": "critical", "detail": "non-finite loss"})
            return out
        if cur.grad_norm > self.thresholds["grad_explosion_abs"]:
            out.append({"type": "gradient_explosion", "severity": "critical", "detail": f"grad norm {cur.grad_norm:.1f}"})
        if len(h) >= self.min_samples:
            losses = [x.loss for x in h[:-10] if math.isfinite(x.loss)]
            recent = [x.loss for x in h[-10:] if math.isfinite(x.loss)]
            if len(losses) >= 10 and recent:
                mu, sd = statistics.fmean(losses[-100:]), statistics.pstdev(losses[-100:])
                rm = statistics.fmean(recent)
                if rm > mu + self.thresholds["loss_spike_sigma"] * sd and rm > mu + self.thresholds["loss_spike_abs"]:
                    out.append({"type": "loss_spike", "severity": "hard", "detail": f"recent {rm:.3f} vs {mu:.3f}+-{sd:.3f}"})
            gns = [x.grad_norm for x in h[:-1] if x.grad_norm > 0]
            if gns and cur.grad_norm > self.thresholds["grad_explosion_rel"] * statistics.fmean(gns[-100:]) and cur.grad_norm > 1.0:
                out.append({"type": "gradient_explosion", "severity": "hard", "detail": "grad norm 10x its running mean"})
            w = self.thresholds["plateau_window"]
            if len(h) >= 2 * w:
                a = statistics.fmean(x.loss for x in h[-2 * w:-w])
                b = statistics.fmean(x.loss for x in h[-w:])
                if abs(a - b) < self.thresholds["plateau_rel"] * max(abs(a), 1e-8):
                    out.append({"type": "plateau", "severity": "soft", "detail": f"loss flat over {2 * w} samples"})
        if cur.expert_utilization:
            vals = list(cur.expert_utilization.values())
            if min(vals) < self.thresholds["expert_min_pct"] and max(vals) > self.thresholds["expert_max_pct"]:
                out.append({"type": "expert_collapse", "severity": "medium", "detail": f"min {min(vals):.2f}% max {max(vals):.1f}%"})
        return out

    def trend(self, key: str = "loss", n: int = 100) -> float:
        vals = [getattr(x, key) for x in list(self.history)[-n:]]
        if len(vals) < 2:
            return 0.0
        xs = list(range(len(vals)))
        mx, my = statistics.fmean(xs), statistics.fmean(vals)
        den = sum((x - mx) ** 2 for x in xs) or 1e-12
        return sum((x - mx) * (y - my) for x, y in zip(xs, vals)) / den


class ProductionMonitoring:
    """Measured process / device health."""

    def snapshot(self) -> Dict[str, float]:
        out: Dict[str, float] = {"time": time.time()}
        try:
            import psutil
            p = psutil.Process()
            out["cpu_percent"] = psutil.cpu_percent(interval=None)
            out["rss_gb"] = p.memory_info().rss / 2 ** 30
            out["host_mem_percent"] = psutil.virtual_memory().percent
        except Exception:
            pass
        if torch.cuda.is_available():
            out["gpu_allocated_gb"] = torch.cuda.memory_allocated() / 2 ** 30
            out["gpu_reserved_gb"] = torch.cuda.memory_reserved() / 2 ** 30
            free, total = torch.cuda.mem_get_info()
            out["gpu_used_fraction"] = 1.0 - free / total
        return out


class AdaptiveTrainingOrchestrator:
    def __init__(self, config, model=None, tokenizer=None, trainer: Optional[EnhancedConversationTrainer] = None,
                 mesh=None, install_signal_handlers: bool = False):
        self.config = config
        self.model, self.tokenizer, self.trainer, self.mesh = model, tokenizer, trainer, mesh
        self.logger = log
        exp = os.path.join(getattr(config, "output_dir", "experiments"), config.experiment_name or "run")
        self.experiment_dir = exp
        self.meta_learning = MetaLearningEngine(os.path.join(exp, "meta_learning_state.pkl"))
        self.hyperopt = AdaptiveHyperparameterOptimizer(min_lr=getattr(config, "min_lr", 1e-7))
        self.architecture = ArchitectureEvolution()
        self.analytics = RealTimeAnalytics()
        self.monitoring = ProductionMonitoring()
        self.decisions: List[AdaptiveDecision] = []
        self.metrics_queue: "queue.Queue[TrainingMetrics]" = queue.Queue(maxsize=1000)
        self.is_training = False
        self.should_stop = False
        self.monitor_thread: Optional[threading.Thread] = None
        self.consecutive_errors = 0
        self.max_consecutive_errors = 10
        self.last_lr_change_step = -10 ** 9
        self.lr_cooldown_steps = 20
        self.enable_architecture_evolution = bool(getattr(config, "enable_architecture_evolution", False))
        self.train_dataset = None
        self.eval_dataset = None
        if install_signal_handlers and threading.current_thread() is threading.main_thread():
            for sig in (signal.SIGINT, signal.SIGTERM):
                signal.signal(sig, self._on_signal)
            if hasattr(signal, "SIGUSR1"):
                signal.signal(signal.SIGUSR1, self._on_save_signal)

    # -- signals --------------------------------------------------------------------------------------------
    def _on_signal(self, signum, frame) -> None:
        self.logger.warning("signal %s: saving state and stopping", signum)
        self.should_stop = True
        if self.trainer is not None:
            self.trainer.should_stop = True
        self.meta_learning.save()

    def _on_save_signal(self, signum, frame) -> None:
        if self.trainer is not None:
            self.trainer._at_step_boundary(lambda: self.trainer.save_checkpoint(self.trainer.current_epoch, tag=f"signal_{int(time.time())}"))

    # -- set-up ---------------------------------------------------------------------------------------------
    def initialize_training(self, train_dataset=None, eval_dataset=None) -> EnhancedConversationTrainer:
        if self.trainer is None:
            if self.model is None:
                from ..models.transformer import DeepSeekTransformer
                dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
                dtype = torch.bfloat16 if dev.type == "cuda" and "fp32" not in self.config.precision else torch.float32
                self.model = DeepSeekTransformer(self.config.to_model_config()).to(dev, dtype)
            self.trainer = EnhancedConversationTrainer(self.model, self.tokenizer, self.config, mesh=self.mesh)
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self._enhance_trainer_with_adaptive_features()
        hint = self.meta_learning.suggest_hyperparameters({"parameters": self.trainer.model.num_parameters()})
        self.logger.info("meta-learning LR hint %.2e (distance %.2f)", hint["learning_rate"], hint["source_distance"])
        return self.trainer

    def _enhance_trainer_with_adaptive_features(self) -> None:
        """Subscribe to the trainer's metric flushes (the reference monkey-patches train_step / optimizer_step,
        ``orchestrator.py:1265-1456``); inline guards run on the training thread."""
        tr = self.trainer
        if getattr(tr, "_orchestrated", False):
            return
        flush = tr._flush_metrics

        def flush_and_publish():
            m = flush()
            if m is not None:
                tm = TrainingMetrics(epoch=tr.current_epoch, step=tr.global_step, loss=m["loss"], grad_norm=m["grad_norm"],
                                     learning_rate=m["lr"], throughput=m["tokens_per_second"],
                                     expert_utilization=tr._extract_moe_routing_stats() if tr.model.config.use_moe and tr.global_step % 50 == 0 else {})
                self._inline_guards(tm)
                try:
                    self.metrics_queue.put_nowait(tm)
                except queue.Full:
                    pass
            return m
        tr._flush_metrics = flush_and_publish
        tr._orchestrated = True

    def _inline_guards(self, m: TrainingMetrics) -> None:
        """Cheap checks on the training thread (reference ``orchestrator.py:1359-1406``)."""
        tl = self.trainer.metrics["train_losses"]
        if not math.isfinite(m.loss):
            self._decide("divergence_prevention", {"rollback_steps": 100, "lr_factor": 0.1}, 1.0, "non-finite loss")
            return
        if m.grad_norm > 100.0:
            self._decide("emergency_lr_reduction", {"factor": 10.0}, 0.95, f"grad norm {m.grad_norm:.1f} > 100")
        elif len(tl) >= 20:
            base = statistics.fmean(tl[-20:-1])
            if m.loss > 2.0 * base:
                self._decide("loss_spike_response", {"lr_factor": 0.5, "grace_period": 20}, 0.85, f"loss {m.loss:.3f} > 2x mean {base:.3f}")

    # -- monitor thread ---------------------------------------------------------------------------------------
    def start_real_time_monitoring(self) -> None:
        if self.monitor_thread is not None and self.monitor_thread.is_alive():
            return
        self.is_training = True
        self.monitor_thread = threading.Thread(target=self._monitoring_loop, name="ats-monitor", daemon=True)
        self.monitor_thread.start()

    def _monitoring_loop(self) -> None:
        while self.is_training and not self.should_stop:
            try:
                m = self.metrics_queue.get(timeout=0.2)
            except queue.Empty:
                continue
            try:
                self._process_real_time_metrics(m)
                self.consecutive_errors = 0
            except Exception as e:
                self.consecutive_errors += 1
                self.logger.warning("monitor error %d/%d: %s", self.consecutive_errors, self.max_consecutive_errors, e)
                if self.consecutive_errors >= self.max_consecutive_errors:
                    self.logger.error("monitor disabled after repeated errors")
                    return

    def _process_real_time_metrics(self, m: TrainingMetrics) -> None:
        for a in self.analytics.detect_training_anomalies(m):
            self._handle_training_anomaly(a, m)
        if self.enable_architecture_evolution and m.expert_utilization and self.trainer is not None:
            for prop in self.architecture.propose(self.trainer.model.get_routing_statistics()):
                if prop["action"] == "add_expert":
                    self._decide("add_expert", {"layer_idx": prop["layer_idx"]}, 0.8, prop["reason"])
                else:
                    self._decide("prune_expert", {"layer_idx": prop["layer_idx"], "expert_idx": prop["expert_idx"]}, 0.8, prop["reason"])

    def _handle_training_anomaly(self, a: Dict[str, Any], m: TrainingMetrics) -> None:
        kind = a["type"]
        if kind == "divergence":
            self._decide("divergence_prevention", {"rollback_steps": 100, "lr_factor": 0.1}, 1.0, a["detail"])
        elif kind == "gradient_explosion":
            f = 10.0 if a["severity"] == "critical" else 2.0
            self._decide("emergency_lr_reduction" if f >= 10 else "corrective_lr_reduction", {"factor": f}, 0.92, a["detail"])
        elif kind == "loss_spike":
            self._decide("loss_spike_response", {"lr_factor": 0.5, "grace_period": 20}, 0.85, a["detail"])
        elif kind == "plateau":
            self._decide("plateau_intervention", {"lr_factor": 1.25, "grace_period": 10}, 0.72, a["detail"])
        elif kind == "expert_collapse":
            self._decide("expert_rebalance", {"temperature_factor": 1.2, "capacity_factor": 1.1}, 0.8, a["detail"])

    # -- decisions --------------------------------------------------------------------------------------------
    def _decide(self, kind: str, params: Dict[str, Any], confidence: float, why: str) -> AdaptiveDecision:
        d = AdaptiveDecision(kind, params, confidence, why)
        self.decisions.append(d)
        if getattr(self.config, "log_lr_decisions", True):
            self.logger.info("decision %s (confidence %.2f): %s", kind, confidence, why)
        self._execute_decision(d)
        return d

    def _lr_allowed(self, emergency: bool) -> bool:
        if not getattr(self.config, "enable_adaptive_lr", True):
            return emergency and getattr(self.config, "emergency_override_enabled", True)
        if emergency:
            return True
        step = self.trainer.global_step if self.trainer else 0
        return step - self.last_lr_change_step >= self.lr_cooldown_steps

    def _apply_learning_rate_adjustment(self, factor: float, grace_period: int = 10, emergency: bool = False) -> bool:
        tr = self.trainer
        if tr is None or not self._lr_allowed(emergency):
            return False
        if not emergency and abs(factor - 1.0) < getattr(self.config, "min_override_threshold", 0.2):
            return False
        new_lr = max(tr.engine.get_lr() * factor, 1e-8)
        tr.adjust_learning_rate(new_lr, grace_period=grace_period, emergency=emergency)
        self.last_lr_change_step = tr.global_step
        return True

    def _execute_decision(self, d: AdaptiveDecision) -> None:
        tr = self.trainer
        if tr is None:
            return
        k, p = d.decision_type, d.parameters
        if k in ("learning_rate_adjustment", "optimization_lr_increase", "plateau_intervention"):
            d.applied = self._apply_learning_rate_adjustment(p.get("lr_factor", p.get("factor", 1.0)), p.get("grace_period", 10))
        elif k in ("corrective_lr_reduction", "loss_spike_response"):
            f = p.get("lr_factor", 1.0 / p.get("factor", 2.0))
            d.applied = self._apply_learning_rate_adjustment(f, p.get("grace_period", 20))
        elif k == "emergency_lr_reduction":
            if self._lr_allowed(True):
                tr.emergency_lr_reduction(p.get("factor", 10.0))
                tr.adjust_learning_rate(tr.engine.get_lr() / p.get("factor", 10.0) if threading.current_thread() is not tr._train_thread
                                        else tr.engine.get_lr(), grace_period=20, emergency=True)
                self.last_lr_change_step = tr.global_step
                d.applied = True
        elif k in ("divergence_prevention", "checkpoint_rollback"):
            n = int(p.get("rollback_steps", 100))
            tr._at_step_boundary(lambda: tr.rollback_steps(n))
            self._apply_learning_rate_adjustment(p.get("lr_factor", 0.1), 20, emergency=True)
            d.applied = True
        elif k == "add_expert":
            tr._at_step_boundary(lambda: tr.add_expert(p.get("layer_idx")))
            d.applied = True
        elif k == "prune_expert":
            tr._at_step_boundary(lambda: tr.prune_expert(p["layer_idx"], p["expert_idx"]))
            d.applied = True
        elif k == "expert_rebalance":
            t = tr.model.config.routing_temperature * p.get("temperature_factor", 1.0)
            c = tr.model.config.capacity_factor * p.get("capacity_factor", 1.0)
            tr._at_step_boundary(lambda: (tr.adjust_routing_temperature(min(t, 4.0)), tr.adjust_capacity_factor(min(c, 4.0))))
            d.applied = True

    # documented helpers (docs/adaptive_training.md) -----------------------------------------------------------
    def increase_capacity_factor(self, factor: float = 1.1) -> None:
        self.trainer.adjust_capacity_factor(self.trainer.model.config.capacity_factor * factor)

    def increase_mod_capacity(self, delta: float = 0.1) -> None:
        self.trainer.adjust_mod_capacity(min(1.0, self.trainer.model.config.mod_capacity_factor + delta))

    def decrease_mod_capacity(self, delta: float = 0.1) -> None:
        self.trainer.adjust_mod_capacity(max(0.05, self.trainer.model.config.mod_capacity_factor - delta))

    def add_router_jitter(self, std: float = 0.1) -> None:
        for l in self.trainer.model.get_moe_layers():
            l.routing_noise_std = std

    def suggest_precision_change(self) -> Dict[str, Any]:
        nonfinite = sum(1 for d in self.decisions if d.decision_type == "divergence_prevention")
        return {"current": self.config.precision, "suggested": "mixed_bf16" if nonfinite and "fp8" in self.config.precision else self.config.precision,
                "reason": f"{nonfinite} divergence events"}

    def suggest_quantization_adjustment(self, serving_memory_gb: Optional[float] = None) -> Dict[str, Any]:
        """Which post-training quantisation to serve the current model with: the bf16 weights against the memory of the serving
        GPU (default: this GPU, or 180 GB without one).  fp8 halves the weight bytes of projections and experts; int4 quarters
        the projections (dense models) and wants a GPTQ calibration pass."""
        n = self.trainer.model.config.num_parameters() if self.trainer is not None else self.config.num_parameters()
        if serving_memory_gb is None:
            serving_memory_gb = torch.cuda.get_device_properties(0).total_memory / 2 ** 30 if torch.cuda.is_available() else 180.0
        bf16_gb = 2.0 * n / 2 ** 30
        frac = bf16_gb / serving_memory_gb
        moe = bool(getattr(self.config, "use_moe", False))
        if frac < 0.35:
            pick, why = None, "the bf16 weights leave most of the memory to the KV cache"
        elif frac < 0.7 or moe:
            pick, why = "fp8", "e4m3 weights (experts included) halve the bytes a decode step streams"
        else:
            pick, why = "int4", "4-bit projections (GPTQ) are what fits next to a KV cache"
        return {"current": getattr(self.config, "quantization_method", None), "suggested": pick, "bf16_weight_gb": round(bf16_gb, 2),
                "fraction_of_memory": round(frac, 3), "reason": why}

    def enable_memory_optimizations(self) -> None:
        self.trainer.model.config.gradient_checkpointing = True

    # -- run ------------------------------------------------------------------------------------------------------
    def run_adaptive_training(self, train_dataset=None, eval_dataset=None) -> Dict[str, Any]:
        if self.trainer is None:
            self.initialize_training(train_dataset, eval_dataset)
        train_dataset = train_dataset if train_dataset is not None else self.train_dataset
        eval_dataset = eval_dataset if eval_dataset is not None else self.eval_dataset
        self.start_real_time_monitoring()
        t0 = time.time()
        try:
            summary = self.trainer.train_with_oom_fallback(train_dataset, eval_dataset)
        finally:
            self.is_training = False
            if self.monitor_thread is not None:
                self.monitor_thread.join(timeout=2.0)
        tl = self.trainer.metrics["train_losses"]
        final = tl[-1] if tl else float("nan")
        self.meta_learning.record_run({"parameters": self.trainer.model.num_parameters(), "learning_rate": self.config.learning_rate,
                                       "batch": self.config.effective_batch_size}, final, math.isfinite(final))
        self.meta_learning.save()
        summary["adaptive"] = self.get_adaptive_status()
        summary["wall_time_s"] = time.time() - t0
        self._write_reports(summary)
        return summary

    def get_adaptive_status(self) -> Dict[str, Any]:
        by_type: Dict[str, int] = {}
        for d in self.decisions:
            by_type[d.decision_type] = by_type.get(d.decision_type, 0) + 1
        return {"decisions_total": len(self.decisions), "decisions_applied": sum(d.applied for d in self.decisions),
                "decisions_by_type": by_type, "monitoring_active": bool(self.monitor_thread and self.monitor_thread.is_alive()),
                "loss_trend": self.analytics.trend("loss"), "meta_runs": len(self.meta_learning.training_history),
                "system": self.monitoring.snapshot(),
                "recent_decisions": [asdict(d) for d in self.decisions[-5:]]}

    def _write_reports(self, summary: Dict[str, Any]) -> None:
        try:
            os.makedirs(self.experiment_dir, exist_ok=True)
            with open(os.path.join(self.experiment_dir, "adaptive_learning_summary.json"), "w") as f:
                json.dump(summary.get("adaptive", {}), f, indent=2, default=str)
            with open(os.path.join(self.experiment_dir, "adaptive_insights_report.json"), "w") as f:
                json.dump({"decisions": [asdict(d) for d in self.decisions]}, f, indent=2, default=str)
        except OSError as e:
            self.logger.warning("could not write reports: %s", e)

    def cleanup(self) -> None:
        self.is_training = False
        self.should_stop = True
        if self.monitor_thread is not None:
            self.monitor_thread.join(timeout=2.0)
        self.meta_learning.save()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def wrap_orchestrator_with_oom_protection(make_orchestrator: Callable[[Any], AdaptiveTrainingOrchestrator], config,
                                          train_dataset, eval_dataset=None, max_attempts: int = 10) -> Dict[str, Any]:
    """Outer retry loop of the entry script (reference ``Main.py:292-524``): on an out-of-memory error rebuild the
    whole orchestrator with half the batch and twice the accumulation (capped at 32)."""
    attempt = 0
    while True:
        orch = make_orchestrator(config)
        try:
            return orch.run_adaptive_training(train_dataset, eval_dataset)
        except Exception as e:
            if not is_oom_error(e) or attempt >= max_attempts:
                raise
            attempt += 1
            orch.cleanup()
            config.micro_batch_size = max((config.micro_batch_size or config.batch_size) // 2, 1)
            config.batch_size = config.micro_batch_size
            config.gradient_accumulation_steps = min(config.gradient_accumulation_steps * 2, 32)
            log.warning("OOM at orchestrator level: attempt %d with batch %d", attempt, config.batch_size)

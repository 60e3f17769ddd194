"""Learning-rate schedules as pure functions of the step (cosine / onecycle / constant / linear / warmup-decay, reference
``training/trainer.py:3438-3582``; multistep / polynomial / flat-then-anneal as in the reference's vendored scheduler package,
``colossalai/nn/lr_scheduler/``, each with the same optional linear warm-up).  The scheduler returns a number; the engine
writes it into its device-side hyper-parameter vector, so a schedule step costs no kernel rebuild and no optimizer
param-group walk."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Sequence


class LRSchedule:
    def __init__(self, kind: str, base_lr: float, total_steps: int, warmup_ratio: float = 0.0, min_lr: float = 0.0,
                 milestones: Optional[Sequence[float]] = None, gamma: float = 0.1, power: float = 1.0, flat_fraction: float = 0.72):
        self.kind, self.base_lr, self.total_steps = kind, float(base_lr), max(int(total_steps), 1)
        self.warmup_steps = int(self.total_steps * warmup_ratio)
        self.min_lr = float(min_lr)
        self.last_step = 0
        ms = list(milestones) if milestones else [0.5, 0.75]
        self.milestones = sorted(int(m * self.total_steps) if m <= 1 else int(m) for m in ms)   # fractions of the run or steps
        self.gamma, self.power, self.flat_fraction = float(gamma), float(power), float(flat_fraction)

    def lr_at(self, step: int) -> float:
        b, m, T, W = self.base_lr, self.min_lr, self.total_steps, self.warmup_steps
        if self.kind == "constant":
            return b
        if W > 0 and step < W:
            return b * (step + 1) / W
        prog = min(max((step - W) / max(T - W, 1), 0.0), 1.0)
        if self.kind == "cosine":
            return m + (b - m) * 0.5 * (1.0 + math.cos(math.pi * prog))
        if self.kind in ("linear", "warmup_decay"):
            return m + (b - m) * (1.0 - prog)
        if self.kind == "multistep":
            return max(b * self.gamma ** sum(1 for ms in self.milestones if step >= ms), m)
        if self.kind == "poly":
            return m + (b - m) * (1.0 - prog) ** self.power
        if self.kind == "flat_anneal":
            f = min(max(self.flat_fraction, 0.0), 0.999)
            return b if prog < f else m + (b - m) * 0.5 * (1.0 + math.cos(math.pi * (prog - f) / (1.0 - f)))
        if self.kind == "onecycle":
            peak = 0.3
            p = min(step / T, 1.0)
            if p < peak:
                return b / 25.0 + (b - b / 25.0) * 0.5 * (1 - math.cos(math.pi * p / peak))
            return m + (b - m) * 0.5 * (1 + math.cos(math.pi * (p - peak) / (1 - peak)))
        raise ValueError(f"unknown scheduler {self.kind}")

    def current_lr(self) -> float:
        return self.lr_at(self.last_step)

    def step(self) -> float:
        self.last_step += 1
        return self.lr_at(self.last_step)

    def scale_base(self, factor: float) -> None:
        self.base_lr *= factor
        self.min_lr = min(self.min_lr, self.base_lr)

    @property
    def base_lrs(self):
        return [self.base_lr]

    def state_dict(self) -> Dict[str, Any]:
        return dict(kind=self.kind, base_lr=self.base_lr, total_steps=self.total_steps, warmup_steps=self.warmup_steps,
                    min_lr=self.min_lr, last_step=self.last_step, milestones=list(self.milestones), gamma=self.gamma, power=self.power,
                    flat_fraction=self.flat_fraction)

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        for k, v in sd.items():
            setattr(self, k, v)


def build_scheduler(config, total_steps: int) -> LRSchedule:
    return LRSchedule(getattr(config, "lr_scheduler", "cosine"), config.learning_rate, total_steps,
                      getattr(config, "warmup_ratio", 0.0), getattr(config, "min_lr", 0.0), getattr(config, "lr_milestones", None),
                      getattr(config, "lr_gamma", 0.1), getattr(config, "lr_power", 1.0), getattr(config, "lr_flat_fraction", 0.72))

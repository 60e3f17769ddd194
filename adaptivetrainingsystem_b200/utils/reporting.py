"""Experiment reports: training summary JSON and a dependency-free HTML page (reference ``utils/reporting.py:11-193``)."""
from __future__ import annotations

import html
import json
import os
import time
from typing import Any, Dict, List, Optional


def create_training_summary(trainer, extra: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    m = trainer.metrics
    tl = m.get("train_losses", [])
    out = {"experiment": trainer.config.experiment_name, "global_step": trainer.global_step, "epochs": trainer.current_epoch + 1,
           "final_loss": tl[-1] if tl else None, "best_loss": min(tl) if tl else None, "best_eval_loss": trainer.best_eval_loss,
           "mean_tokens_per_second": (sum(m["tokens_per_second"]) / len(m["tokens_per_second"])) if m.get("tokens_per_second") else None,
           "parameters": trainer.model.num_parameters(), "precision": trainer.config.precision, "created": time.time()}
    out.update(extra or {})
    return out


def _sparkline(values: List[float], width: int = 600, height: int = 120) -> str:
    vals = [v for v in values if v == v]
    if len(vals) < 2:
        return ""
    lo, hi = min(vals), max(vals)
    rng = (hi - lo) or 1.0
    pts = " ".join(f"{i * width / (len(vals) - 1):.1f},{height - (v - lo) / rng * height:.1f}" for i, v in enumerate(vals))
    return f'<svg width="{width}" height="{height}"><polyline fill="none" stroke="#06c" stroke-width="1.5" points="{pts}"/></svg>'


def create_html_report(trainer, path: str, extra: Optional[Dict[str, Any]] = None) -> str:
    s = create_training_summary(trainer, extra)
    rows = "".join(f"<tr><td>{html.escape(str(k))}</td><td>{html.escape(str(v))}</td></tr>" for k, v in s.items())
    body = (f"<html><head><meta charset='utf-8'><title>{html.escape(str(s['experiment']))}</title></head><body>"
            f"<h1>{html.escape(str(s['experiment']))}</h1><table border=1 cellpadding=4>{rows}</table>"
            f"<h2>training loss</h2>{_sparkline(trainer.metrics.get('train_losses', []))}"
            f"<h2>gradient norm</h2>{_sparkline(trainer.metrics.get('gradient_norms', []))}"
            f"<h2>tokens / s</h2>{_sparkline(trainer.metrics.get('tokens_per_second', []))}</body></html>")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(body)
    return path


def save_experiment_metadata(config, directory: str, system_info: Optional[Dict[str, Any]] = None) -> None:
    os.makedirs(directory, exist_ok=True)
    config.save(os.path.join(directory, "config.yaml"))
    config.save(os.path.join(directory, "config.json"))
    with open(os.path.join(directory, "metadata.json"), "w") as f:
        json.dump({"experiment": config.experiment_name, "created": time.time(), "parameters": config.num_parameters(),
                   "active_parameters": config.num_parameters(True)}, f, indent=2)
    if system_info is not None:
        with open(os.path.join(directory, "system_info.json"), "w") as f:
            json.dump(system_info, f, indent=2, default=str)

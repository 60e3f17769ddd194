"""Two small debugging aids the reference carries in its vendored utilities (``colossalai/utils/rank_recorder``,
``colossalai/utils/tensor_detector``), rebuilt without plotting dependencies:

* :class:`RankRecorder` -- named intervals per rank (device-synchronised wall clock), one JSON file per rank, merged into one
  timeline whose times are relative to the earliest event of any rank; :func:`timeline_text` renders it as rows of text.
* :class:`TensorDetector` -- the live tensors of a process between two calls: what appeared, what vanished, what changed
  device or shape, and the bytes held per device.
"""
from __future__ import annotations

import contextlib
import gc
import json
import os
import time
from typing import Any, Dict, List, Optional, Tuple

import torch


class RankRecorder:
    def __init__(self, rank: Optional[int] = None, directory: str = "record.log"):
        import torch.distributed as dist
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
        self.directory = directory
        self.events: List[Dict[str, Any]] = []

    @staticmethod
    def _now() -> float:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.time()

    @contextlib.contextmanager
    def record(self, name: str):
        t0 = self._now()
        try:
            yield
        finally:
            self.events.append({"name": name, "rank": self.rank, "start": t0, "end": self._now()})

    def export(self) -> str:
        os.makedirs(self.directory, exist_ok=True)
        path = os.path.join(self.directory, f"rank_{self.rank}.json")
        with open(path, "w") as f:
            json.dump(self.events, f)
        return path

    @staticmethod
    def merge(directory: str = "record.log") -> List[Dict[str, Any]]:
        """All ranks' files of ``directory`` as one list sorted by start time, times relative to the earliest start."""
        events: List[Dict[str, Any]] = []
        for name in sorted(os.listdir(directory)):
            if name.startswith("rank_") and name.endswith(".json"):
                with open(os.path.join(directory, name)) as f:
                    events += json.load(f)
        if not events:
            return []
        base = min(e["start"] for e in events)
        for e in events:
            e["start"], e["end"] = e["start"] - base, e["end"] - base
        events.sort(key=lambda e: (e["start"], e["rank"]))
        with open(os.path.join(directory, "timeline.json"), "w") as f:
            json.dump(events, f, indent=1)
        return events


def timeline_text(events: List[Dict[str, Any]], width: int = 80) -> str:
    """One row per rank, one letter per event name, ``width`` columns for the whole span."""
    if not events:
        return ""
    span = max(e["end"] for e in events) or 1e-9
    names = sorted({e["name"] for e in events})
    sym = {n: chr(ord("A") + i % 26) for i, n in enumerate(names)}
    rows = []
    for rank in sorted({e["rank"] for e in events}):
        row = ["."] * width
        for e in events:
            if e["rank"] == rank:
                a, b = int(e["start"] / span * (width - 1)), int(e["end"] / span * (width - 1))
                for i in range(a, max(b, a) + 1):
                    row[i] = sym[e["name"]]
        rows.append(f"rank {rank:3d} |{''.join(row)}|")
    legend = "  ".join(f"{s}={n}" for n, s in sym.items())
    return "\n".join(rows + [f"span {span * 1e3:.1f} ms   {legend}"])


class TensorDetector:
    def __init__(self, include_cpu: bool = False, module: Optional[torch.nn.Module] = None):
        self.include_cpu = include_cpu
        self.names = {id(p): n for n, p in module.named_parameters()} if module is not None else {}
        self.seen: Dict[int, Tuple[str, Tuple[int, ...], str, int]] = {}

    def _snapshot(self) -> Dict[int, Tuple[str, Tuple[int, ...], str, int]]:
        import warnings
        out = {}
        for obj in gc.get_objects():
            try:
                with warnings.catch_warnings():      # isinstance on lazily deprecated module attributes warns
                    warnings.simplefilter("ignore")
                    if not isinstance(obj, torch.Tensor):
                        continue
                if self.include_cpu or obj.is_cuda:
                    out[id(obj)] = (self.names.get(id(obj), type(obj).__name__), tuple(obj.shape), str(obj.device),
                                    obj.untyped_storage().nbytes())
            except Exception:
                continue
        return out

    def detect(self) -> Dict[str, Any]:
        """-> {"new": [...], "gone": [...], "changed": [...], "bytes_per_device": {...}} relative to the previous call."""
        now = self._snapshot()
        new = [now[k] for k in now.keys() - self.seen.keys()]
        gone = [self.seen[k] for k in self.seen.keys() - now.keys()]
        changed = [(self.seen[k], now[k]) for k in now.keys() & self.seen.keys() if now[k][1:3] != self.seen[k][1:3]]
        per_dev: Dict[str, int] = {}
        for _, _, dev, nbytes in now.values():
            per_dev[dev] = per_dev.get(dev, 0) + nbytes
        self.seen = now
        return {"new": new, "gone": gone, "changed": changed, "bytes_per_device": per_dev}

    def close(self) -> None:
        self.seen.clear()

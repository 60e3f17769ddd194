"""Phase timers on CUDA events (host clock on CPU), NVTX ranges and roofline arithmetic."""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict
from typing import Dict, List, Optional

import torch


class PhaseTimer:
    def __init__(self, device=None):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.cuda = self.device.type == "cuda"
        self._events: Dict[str, List] = defaultdict(list)
        self._host: Dict[str, List[float]] = defaultdict(list)

    @contextlib.contextmanager
    def phase(self, name: str):
        if self.cuda:
            torch.cuda.nvtx.range_push(name)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                torch.cuda.nvtx.range_pop()
                self._events[name].append((a, b))
                if len(self._events[name]) > 4096:      # a long run keeps the most recent intervals only
                    del self._events[name][:2048]
        else:
            t = time.perf_counter()
            try:
                yield
            finally:
                self._host[name].append((time.perf_counter() - t) * 1e3)
                if len(self._host[name]) > 4096:
                    del self._host[name][:2048]

    def summary(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        if self.cuda:
            torch.cuda.synchronize(self.device)
            for k, evs in self._events.items():
                ms = [a.elapsed_time(b) for a, b in evs]
                out[k + "_ms"] = sum(ms) / max(len(ms), 1)
        for k, ms in self._host.items():
            out[k + "_ms"] = sum(ms) / max(len(ms), 1)
        return out


def measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Roofline denominators: the measured copy bandwidth and cuBLAS bf16 throughput of this pool when the
    file is present, else the documented fallback (6.65 TB/s, 1.59 PFLOP/s)."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def roofline_fraction(flops: float = 0.0, bytes_moved: float = 0.0, seconds: float = 1.0, sustained: bool = False) -> Dict[str, float]:
    pk = measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    bw = pk["hbm_gbs"] * 1e9
    ideal = max(flops / tf, bytes_moved / bw)
    return {"achieved_tflops": flops / seconds / 1e12, "achieved_gbs": bytes_moved / seconds / 1e9,
            "ideal_s": ideal, "fraction": ideal / seconds if seconds > 0 else 0.0, "peaks": pk["source"]}


def time_cuda(fn, warmup: int = 3, iters: int = 10, flush_l2: bool = True) -> float:
    """Median device time of ``fn`` in milliseconds: CUDA events on the launching stream, warm-up first,
    L2 flushed between iterations by writing a 256 MB buffer."""
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]

"""GPU / kernel diagnostics: what the reference's CUDA debug script reports (reference ``cuda_debug_script.py:1-502``:
driver, device, compiler, extension build, a smoke run of every kernel), for this framework's native library.

    python -m adaptivetrainingsystem_b200.utils.diagnostics [--json]
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Callable, Dict, List

import torch


def _timed(fn: Callable[[], Any]) -> Dict[str, Any]:
    t0 = time.time()
    try:
        fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return {"ok": True, "seconds": round(time.time() - t0, 4)}
    except Exception as e:  # a diagnostic reports, it does not raise
        return {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}


def collect() -> Dict[str, Any]:
    from ..ops import _lib
    rep: Dict[str, Any] = {"torch": torch.__version__, "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
                           "nvcc": _lib._nvcc(), "cuda_library": os.path.exists(_lib.CUDA_LIB), "host_library": os.path.exists(_lib.HOST_LIB)}
    host = _lib.host_lib()
    rep["cpu_isa"] = int(host.ats_cpu_isa()) if host is not None else None
    if not torch.cuda.is_available():
        rep["devices"] = []
        return rep
    rep["devices"] = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        rep["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                               "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    cap = torch.cuda.get_device_capability(0)
    rep["sm_100"] = cap[0] == 10
    from .. import ops
    dev = torch.device("cuda", 0)
    x = torch.randn(256, 512, device=dev).bfloat16()
    w = torch.randn(768, 512, device=dev).bfloat16()
    qkv = torch.randn(1, 256, (4 + 2 * 2) * 64, device=dev).bfloat16()
    checks: List = [
        ("gemm_nt", lambda: ops.gemm_nt(x, w)),
        ("rms_norm", lambda: ops.rms_norm(x, torch.ones(512, device=dev).bfloat16())),
        ("swiglu", lambda: ops.swiglu(torch.randn(256, 1024, device=dev).bfloat16())),
        ("attention", lambda: ops.attention_packed(qkv, 4, 2, 64)),
        ("cross_entropy", lambda: ops.cross_entropy(torch.randn(256, 1024, device=dev).bfloat16(), torch.randint(0, 1024, (256,), device=dev))),
        ("fp8_gemm", lambda: ops.fp8.gemm_nt_fp8(*ops.fp8.quantize_rows(x), *ops.fp8.quantize_rows(w))),
        ("sampling", lambda: ops.sample_tokens(torch.randn(4, 1024, device=dev), 0.8, 50, 0.9)),
        ("status", ops.check_status),
    ]
    rep["kernels"] = {name: _timed(fn) for name, fn in checks}
    return rep


def main(argv=None) -> int:
    rep = collect()
    if "--json" in (argv or sys.argv[1:]):
        print(json.dumps(rep, indent=1))
    else:
        for k, v in rep.items():
            if k == "kernels":
                for n, r in v.items():
                    print(f"  kernel {n:14s} {'ok' if r['ok'] else 'FAILED: ' + r.get('error', '')}")
            else:
                print(f"{k}: {v}")
    bad = [n for n, r in rep.get("kernels", {}).items() if not r["ok"]]
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())

"""One tcgen05 GEMM shape, timed against torch.matmul; small enough for a profiler capture:

    python benchmarks/bench_gemm_one.py --m 8192 --n 8192 --k 8192 --iters 5
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200.ops import gemm as G  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--mode", default="nt", choices=["nt", "nn", "tn", "swiglu"],
                    help="swiglu: n = 2 x intermediate rows [gate; up], SwiGLU epilogue writing h and the pre-activations")
    ap.add_argument("--phases", action="store_true", help="cycle totals of one CTA's MMA thread")
    a = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = torch.randn(a.n, a.k, device=dev).bfloat16()
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    if a.mode == "nt":
        ours, lib = (lambda: G.gemm_nt(x, w, out=out)), (lambda: torch.matmul(x, w.t(), out=out))
    elif a.mode == "nn":
        wt = w.t().contiguous()
        ours, lib = (lambda: G.gemm_nn(x, wt, out=out)), (lambda: torch.matmul(x, wt, out=out))
    elif a.mode == "swiglu":
        h = torch.empty(a.m, a.n // 2, device=dev, dtype=torch.bfloat16)

        def lib_swiglu():
            torch.matmul(x, w.t(), out=out)
            torch.mul(torch.nn.functional.silu(out[:, : a.n // 2]), out[:, a.n // 2:], out=h)
        ours, lib = (lambda: G.gemm_nt_swiglu(x, w, out=h, pre_act=out)), lib_swiglu
    else:
        xt, wt = x.t().contiguous(), w.t().contiguous()
        ours, lib = (lambda: G.gemm_tn(xt, wt, out=out)), (lambda: torch.matmul(xt.t(), wt, out=out))

    def timed(fn):
        for _ in range(3):
            fn()
        tot = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / a.iters
    t_o, t_l = timed(ours), timed(lib)
    phases = None
    if a.phases:
        import ctypes
        from adaptivetrainingsystem_b200.ops import _lib
        buf = torch.zeros(8, dtype=torch.int64, device=dev)
        lib_c = _lib.cuda_lib()
        lib_c.ats_gemm_set_profile.argtypes = [ctypes.c_void_p]
        lib_c.ats_gemm_set_profile(ctypes.c_void_p(buf.data_ptr()))
        ours()
        torch.cuda.synchronize()
        lib_c.ats_gemm_set_profile(None)
        phases = dict(zip(["total", "wait_stage", "wait_accumulator", "issue", "k_blocks"], buf.tolist()[:5]))
    fl = 2.0 * a.m * a.n * a.k
    print(json.dumps({"gemm": [a.m, a.n, a.k], "mode": a.mode, "ms": t_o, "tflops": fl / t_o / 1e9, "library_ms": t_l,
                      "library_tflops": fl / t_l / 1e9, "l2": "flushed between iterations", "mma_thread_cycles": phases}))


if __name__ == "__main__":
    main()

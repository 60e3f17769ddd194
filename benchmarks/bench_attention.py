"""Attention kernels alone: forward and backward of the tcgen05 flash attention at one shape, timed with CUDA events
against the library (SDPA) path.  Small enough to capture under a profiler:

    python benchmarks/bench_attention.py --batch 2 --seq 2048 --heads 32 --kv-heads 4 --dim 64 --iters 3
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402


def time_cuda(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-library", action="store_true")
    ap.add_argument("--phases", action="store_true", help="print per-phase cycle totals of one CTA of each backward pass")
    ap.add_argument("--fwd", default=None, help="forward variant: v1 | v2s | v2t")
    a = ap.parse_args()
    if a.fwd:
        from adaptivetrainingsystem_b200.ops import attention_native
        attention_native.FWD_VARIANT = a.fwd
    B, L, hq, hkv, d = a.batch, a.seq, a.heads, a.kv_heads, a.dim
    dev = torch.device("cuda")
    torch.manual_seed(0)
    qkv = torch.randn(B, L, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16).requires_grad_()
    go = torch.randn(B, L, hq, d, device=dev, dtype=torch.bfloat16)
    fl = 4.0 * B * hq * L * L * d / 2

    def fwd():
        with torch.no_grad():
            return ops.attention_packed(qkv, hq, hkv, d)

    def fwd_bwd():
        qkv.grad = None
        ops.attention_packed(qkv, hq, hkv, d).backward(go)

    t_f = time_cuda(fwd, a.iters)
    t_fb = time_cuda(fwd_bwd, a.iters)
    out = {"shape": [B, L, hq, hkv, d], "fwd_variant": a.fwd or "default", "fwd_ms": t_f, "fwd_tflops": fl / t_f / 1e9, "bwd_ms": t_fb - t_f,
           "bwd_tflops": 2.5 * fl / (t_fb - t_f) / 1e9}
    if not a.no_library:
        q = qkv.detach()[..., : hq * d].reshape(B, L, hq, d).transpose(1, 2).contiguous().requires_grad_()
        k = qkv.detach()[..., hq * d:(hq + hkv) * d].reshape(B, L, hkv, d).transpose(1, 2).contiguous().requires_grad_()
        v = qkv.detach()[..., (hq + hkv) * d:].reshape(B, L, hkv, d).transpose(1, 2).contiguous().requires_grad_()
        sdpa = torch.nn.functional.scaled_dot_product_attention

        def lib_f():
            with torch.no_grad():
                return sdpa(q, k, v, is_causal=True, enable_gqa=True)

        def lib_fb():
            q.grad = k.grad = v.grad = None
            sdpa(q, k, v, is_causal=True, enable_gqa=True).backward(go.transpose(1, 2))
        lf = time_cuda(lib_f, a.iters)
        lfb = time_cuda(lib_fb, a.iters)
        out.update({"library_fwd_ms": lf, "library_bwd_ms": lfb - lf})
    if a.phases:
        from adaptivetrainingsystem_b200.ops import attention_native as AN
        AN.PHASE_PROFILE = torch.zeros(32, dtype=torch.int64, device=dev)
        AN.FWD_PHASE_PROFILE = torch.zeros(16, dtype=torch.int64, device=dev)
        fwd_bwd()
        torch.cuda.synchronize()
        pp = AN.PHASE_PROFILE.tolist()
        fp = AN.FWD_PHASE_PROFILE.tolist()
        AN.PHASE_PROFILE = AN.FWD_PHASE_PROFILE = None
        out["phases_fwd"] = dict(zip(["total", "wait_v", "wait_p", "issue", "iterations"], fp[:5]))
        out["phases_fwd"].update(dict(zip(["sm_wait_s", "sm_tmem_load", "sm_max", "sm_exp_store", "sm_signal"], fp[8:13])))
        names = ["total", "wait_tile", "wait_scores_read", "wait_p_ds", "issue", "iterations", "", "", "sm_wait_scores", "sm_tmem_load", "sm_math",
                 "sm_wait_products", "sm_store"]
        out["phases_dkv"] = {n: v for n, v in zip(names, pp[:13]) if n}
        out["phases_dq"] = {n: v for n, v in zip(names, pp[16:29]) if n}
    ops.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()

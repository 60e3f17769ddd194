#!/usr/bin/env python
"""Kernel micro-benchmarks: device time (CUDA events, L2 flushed between iterations), achieved TFLOP/s or GB/s and
the fraction of the measured roofline (``MEASURED_PEAKS.json``: cuBLAS bf16 burst throughput, STREAM-style copy
bandwidth).  A library column (cuBLAS / PyTorch eager) is printed next to each kernel for comparison.

    python benchmarks/bench_kernels.py [--quick] [--json out.json] [--only gemm,fp8,int8,int4,swiglu,grouped,memory,adamw,attention]

``--only memory`` (or any other single section) keeps a run short enough for a profiler capture of one kernel.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402
from adaptivetrainingsystem_b200.ops import gemm as G  # noqa: E402
from adaptivetrainingsystem_b200.ops import moe as M  # noqa: E402
from adaptivetrainingsystem_b200.utils.profiler import measured_peaks, time_cuda  # noqa: E402

DEV = "cuda"


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="comma-separated sections: gemm, fp8, int8, int4, swiglu, grouped, memory, adamw, attention")
    args = ap.parse_args()
    only = {t.strip() for t in args.only.split(",") if t.strip()}

    def want(section):
        return not only or section in only
    pk = measured_peaks()
    rows = []

    def report(name, ms, flops=0.0, nbytes=0.0, lib_ms=None):
        tf = flops / ms / 1e9 if flops else 0.0
        gb = nbytes / ms / 1e6 if nbytes else 0.0
        ideal = max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)) * 1e3
        r = {"kernel": name, "ms": round(ms, 4), "tflops": round(tf, 1), "gbs": round(gb, 1),
             "roofline_frac": round(ideal / ms, 3), "library_ms": None if lib_ms is None else round(lib_ms, 4), "peaks": pk["source"]}
        rows.append(r)
        print(json.dumps(r), flush=True)

    shapes = [(8192, 2560, 2048), (8192, 2048, 2048), (8192, 11264, 2048), (8192, 2048, 5632), (4096, 6144, 4096),
              (4096, 28672, 4096), (4096, 4096, 14336), (8192, 8192, 8192)]
    if args.quick:
        shapes = shapes[:2] + shapes[-1:]
    for (m, n, k) in shapes if want("gemm") else []:
        a, b, bt, at = rnd(m, k), rnd(n, k), rnd(k, n), rnd(k, m)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        fl = 2.0 * m * n * k
        lib = time_cuda(lambda: torch.matmul(a, b.t(), out=out))
        report(f"gemm_nt {m}x{n}x{k}", time_cuda(lambda: G.gemm_nt(a, b, out=out)), fl, lib_ms=lib)
        report(f"gemm_nn {m}x{n}x{k}", time_cuda(lambda: G.gemm_nn(a, bt, out=out)), fl, lib_ms=time_cuda(lambda: torch.matmul(a, bt, out=out)))
        report(f"gemm_tn {m}x{n}x{k}", time_cuda(lambda: G.gemm_tn(at, bt, out=out)), fl, lib_ms=time_cuda(lambda: torch.matmul(at.t(), bt, out=out)))
    # fp8 (e4m3, per-row / per-channel scales) forward GEMM against the bf16 kernel and the library
    from adaptivetrainingsystem_b200.ops import fp8
    for (m, n, k) in [(8192, 8192, 8192), (16384, 2560, 2048)] if want("fp8") else []:
        a, b = rnd(m, k), rnd(n, k, scale=0.05)
        aq, sa = fp8.quantize_rows(a)
        bq, sb = fp8.quantize_rows(b)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        report(f"gemm_nt_fp8 {m}x{n}x{k}", time_cuda(lambda: fp8.gemm_nt_fp8(aq, sa, bq, sb, out=out)), 2.0 * m * n * k,
               lib_ms=time_cuda(lambda: torch.matmul(a, b.t(), out=out)))
        report(f"quantize_rows_e4m3 {m}x{k}", time_cuda(lambda: fp8.quantize_rows(a)), nbytes=3.0 * m * k)
    # int8 (kind::i8, s32 accumulation, the same scales) on the same shapes plus two decode-sized ones
    from adaptivetrainingsystem_b200.ops import int8
    for (m, n, k) in [(8192, 8192, 8192), (16384, 2560, 2048), (64, 28672, 4096), (64, 4096, 14336)] if want("int8") else []:
        a, b = rnd(m, k), rnd(n, k, scale=0.05)
        aq, sa = int8.quantize_rows(a)
        bq, sb = int8.quantize_rows(b)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        report(f"gemm_nt_int8 {m}x{n}x{k}", time_cuda(lambda: int8.gemm_nt_int8(aq, sa, bq, sb, out=out)), 2.0 * m * n * k,
               nbytes=float(n * k), lib_ms=time_cuda(lambda: torch.matmul(a, b.t(), out=out)))
        report(f"quantize_rows_int8 {m}x{k}", time_cuda(lambda: int8.quantize_rows(a)), nbytes=3.0 * m * k)
    # weight-only 4-bit: the streaming kernel for 1..16 token rows (bytes = packed weight + scales; library column = cuBLAS on the
    # bf16 weight, which reads four times the bytes) and the dequantise pass that feeds the tcgen05 GEMM for prompts
    from adaptivetrainingsystem_b200.ops import int4
    for (n, k) in [(28672, 4096), (4096, 14336), (11264, 2048), (2048, 5632)] if want("int4") else []:
        w = rnd(n, k, scale=0.05)
        q, sc, z = int4.quantize_rtn(w)
        packed, meta = int4.pack(q), int4.pack_meta(sc, z)
        wbytes = float(packed.numel() * 4 + meta.numel() * 4)
        for m in (1, 4, 8, 16):
            a = rnd(m, k)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
            report(f"gemv_int4 {m}x{n}x{k}", time_cuda(lambda: int4.gemv(a, packed, meta)), 2.0 * m * n * k, nbytes=wbytes,
                   lib_ms=time_cuda(lambda: torch.matmul(a, w.t(), out=out)))
        if n == 28672:
            a = rnd(4, k)
            report(f"gemv_int4_swiglu 4x{n}x{k}", time_cuda(lambda: int4.gemv(a, packed, meta, swiglu=True)), 2.0 * 4 * n * k, nbytes=wbytes)
            wd = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
            report(f"dequant_int4 {n}x{k}", time_cuda(lambda: int4.dequantize(packed, meta, out=wd)), nbytes=wbytes + 2.0 * n * k)
    # SwiGLU-fused GEMM
    for (m, k, i) in [(8192, 2048, 5632), (4096, 4096, 14336)] if want("swiglu") else []:
        a, w = rnd(m, k), rnd(2 * i, k, scale=0.05)
        h = torch.empty(m, i, dtype=torch.bfloat16, device=DEV)
        lib = time_cuda(lambda: ops.swiglu_reference(torch.matmul(a, w.t())))
        report(f"gemm_swiglu {m}x{2 * i}x{k}", time_cuda(lambda: G.gemm_nt_swiglu(a, w, out=h)), 2.0 * m * 2 * i * k, lib_ms=lib)
    # grouped expert GEMM (8 experts, capacity layout)
    for (e, c, k, n) in [(8, 2560, 2048, 11264), (8, 1280, 4096, 28672)][: 1 if args.quick else 2] if want("grouped") else []:
        x, w = rnd(e, c, k), rnd(e, n, k, scale=0.05)
        counts = torch.full((e,), c - 200, dtype=torch.int32, device=DEV)
        out = torch.empty(e, c, n // 2, dtype=torch.bfloat16, device=DEV)
        used = float((c - 200 + 127) // 128 * 128)
        lib = time_cuda(lambda: [torch.matmul(x[j], w[j].t()) for j in range(e)])
        report(f"grouped_swiglu E{e} C{c} {k}->{n}", time_cuda(lambda: G.grouped_nt(x, w, counts, swiglu=True, out=out)),
               2.0 * e * used * n * k, lib_ms=lib)
    def memory_section():
        # memory-bound kernels
        rows_, cols = 16384, 2048
        x, wn = rnd(rows_, cols), torch.ones(cols, device=DEV, dtype=torch.bfloat16)
        xg = x.detach().clone().requires_grad_()
        wg = wn.detach().clone().requires_grad_()
        yg = ops.rms_norm(xg, wg, 1e-6)
        gy = rnd(rows_, cols)
        report("rmsnorm_bwd 16384x2048", time_cuda(lambda: torch.autograd.grad(yg, (xg, wg), gy, retain_graph=True)), nbytes=3.0 * rows_ * cols * 2)
        report("rmsnorm_fwd 16384x2048", time_cuda(lambda: ops.rms_norm(x, wn, 1e-6)), nbytes=2.0 * rows_ * cols * 2,
               lib_ms=time_cuda(lambda: ops.rms_norm_reference(x, wn, 1e-6)))
        gu = rnd(rows_, 2 * 5632)
        report("swiglu_fwd 16384x5632", time_cuda(lambda: ops.swiglu(gu)), nbytes=3.0 * rows_ * 5632 * 2,
               lib_ms=time_cuda(lambda: ops.swiglu_reference(gu)))
        logits = rnd(4096, 32000)
        labels = torch.randint(0, 32000, (4096,), device=DEV)
        report("cross_entropy 4096x32000 (fwd+grad)", time_cuda(lambda: ops.cross_entropy(logits, labels)[0]), nbytes=2.0 * 4096 * 32000 * 2,
               lib_ms=time_cuda(lambda: torch.nn.functional.cross_entropy(logits.float(), labels)))

    if want("memory"):
        memory_section()

    def adamw_section():
        n = 256 * 1024 * 1024
        master, m1, v1 = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        g, p = rnd(n), rnd(n)
        hyper = torch.tensor([1e-3, 0.9, 0.95, 1e-8, 0.01, 1.0], device=DEV)
        report("adamw 256M", time_cuda(lambda: ops.adamw_step(master, m1, v1, g, p, hyper, None), iters=5), nbytes=n * (12 * 2 + 2 + 2))
        del master, m1, v1, g, p

    if want("adamw"):
        adamw_section()
    # attention
    for (bsz, L, hq, hkv, d) in [(4, 2048, 32, 4, 64), (1, 4096, 32, 8, 128)] if want("attention") else []:
        q, k, v = rnd(bsz, L, hq, d), rnd(bsz, L, hkv, d), rnd(bsz, L, hkv, d)
        fl = 4.0 * bsz * hq * L * L * d / 2
        from adaptivetrainingsystem_b200.ops import attn as A
        lib = time_cuda(lambda: torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True))
        report(f"attention_fwd[{A.backend_for(q, k)}] B{bsz} L{L} H{hq}/{hkv} d{d}", time_cuda(lambda: ops.attention(q, k, v)), fl, lib_ms=lib)
        # backward alone: time (fwd + bwd) - fwd for both
        go = rnd(bsz, L, hq, d)

        def fb_ours():
            qq, kk, vv = q.detach().requires_grad_(), k.detach().requires_grad_(), v.detach().requires_grad_()
            ops.attention(qq, kk, vv).backward(go)

        def fb_lib():
            qq, kk, vv = q.detach().requires_grad_(), k.detach().requires_grad_(), v.detach().requires_grad_()
            torch.nn.functional.scaled_dot_product_attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True,
                                                             enable_gqa=True).backward(go.transpose(1, 2))
        report(f"attention_fwd+bwd[{A.backend_for(q, k)}] B{bsz} L{L} H{hq}/{hkv} d{d}", time_cuda(fb_ours), fl * 3.5, lib_ms=time_cuda(fb_lib))
    ops.check_status()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()

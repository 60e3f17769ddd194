#!/usr/bin/env python
"""Device time and achieved bytes of the communication-side kernels on ONE GPU, each on a case small enough for a profiler
capture of a single launch: the MoE row exchange (``dispatch_rows``, ``combine_rows``), the sharded optimiser step
(``peer_reduce_shard``, ``adamw_push``), the ZeRO-3 side kernels (``peer_gather``, ``peer_reduce_rows``) and the Mixture-of-Depths
row kernels.  The "peers" of a kernel are separate buffers of this GPU, so the figures are against HBM; over NVLink the same
kernels are bounded by the link instead (``benchmarks/bench_fused_paths.py`` times them on 2 GPUs).

    python benchmarks/bench_comm_kernels.py [--only dispatch,combine,reduce_shard,adamw_push,gather,reduce_rows,mod] [--iters 5]

Algorithmic bytes per launch are counted from the tensors each kernel must read and write once.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402
from adaptivetrainingsystem_b200.ops import _lib  # noqa: E402
from adaptivetrainingsystem_b200.ops import moe as M  # noqa: E402
from adaptivetrainingsystem_b200.parallel import peer as P  # noqa: E402
from adaptivetrainingsystem_b200.utils.profiler import measured_peaks, time_cuda  # noqa: E402

DEV = torch.device("cuda", 0)


def table(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--world", type=int, default=2, help="number of emulated peers (buffers on this GPU)")
    a = ap.parse_args()
    only = {t for t in a.only.split(",") if t}
    want = lambda k: not only or k in only  # noqa: E731
    pk = measured_peaks()
    lib, st, stream = P._L(), _lib.status_tensor(DEV), _lib.stream_ptr(DEV)
    W = a.world

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 1), "gb_per_s": round(gbs, 1),
                          "of_measured_copy_bandwidth": round(gbs / pk["hbm_gbs"], 3), "peaks": pk["source"]}), flush=True)

    torch.manual_seed(0)
    if want("dispatch") or want("combine"):
        T, H, E, k = 16384, 2048, 8, 2
        x = torch.randn(T, H, device=DEV).bfloat16()
        idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(64)]).repeat(T // 64, 1).int()
        w = torch.rand(T, k, device=DEV)
        C = M.expert_capacity(T, E, k, 1.25)
        slot_pos, counts, totals = M.plan_slots(idx, E, C)
        buf = torch.empty(E, C, H, dtype=x.dtype, device=DEV)
        kept = int((slot_pos >= 0).sum())
        if want("dispatch"):
            report(f"dispatch_rows T{T} H{H} E{E} k{k}", time_cuda(lambda: M.dispatch(x, idx, slot_pos, counts, E, C, out=buf), iters=a.iters),
                   T * H * 2 + kept * H * 2)
        M.dispatch(x, idx, slot_pos, counts, E, C, out=buf)
        if want("combine"):
            res = torch.randn(T, H, device=DEV).bfloat16()
            report(f"combine_rows T{T} H{H} E{E} k{k} (+residual)", time_cuda(lambda: M.combine(buf, idx, slot_pos, w, T, res), iters=a.iters),
                   kept * H * 2 + 2 * T * H * 2)
    n = 64 * 1024 * 1024  # elements of the owned shard: 128 MB of bf16 per peer
    if want("reduce_shard") or want("adamw_push"):
        grads = [torch.randn(n, device=DEV).bfloat16() for _ in range(W)]
        g32 = torch.empty(n, dtype=torch.float32, device=DEV)
        partial = torch.zeros(2048, dtype=torch.float32, device=DEV)
        sumsq = torch.zeros(1, dtype=torch.float32, device=DEV)
        gt = table(grads)
        if want("reduce_shard"):
            def run():
                _lib.check(lib.ats_peer_reduce_shard(gt, W, 0, 0, n, _lib.ptr(g32), _lib.ptr(partial), _lib.ptr(sumsq), 0, _lib.ptr(st), stream),
                           "peer_reduce_shard")
            report(f"peer_reduce_shard {n >> 20}M x {W} peers -> fp32", time_cuda(run, iters=a.iters), W * n * 2 + n * 4)
        if want("adamw_push"):
            params = [torch.zeros(n, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
            master, m1, v1 = (torch.zeros(n, device=DEV) for _ in range(3))
            hyper = torch.tensor([1e-3, 0.9, 0.95, 1e-8, 0.01, 1.0], device=DEV)
            clip = torch.tensor([1.0, 1.0, 0.0, 0.0], device=DEV)
            pt = table(params)

            def run2():
                _lib.check(lib.ats_adamw_push(_lib.ptr(master), _lib.ptr(m1), _lib.ptr(v1), _lib.ptr(g32), pt, W, 0, 0, n, _lib.ptr(hyper),
                                              _lib.ptr(clip), 1.0, _lib.ptr(st), stream), "adamw_push")
            report(f"adamw_push {n >> 20}M -> {W} peers", time_cuda(run2, iters=a.iters), n * (4 + 3 * 8) + W * n * 2)
            del params, master, m1, v1
        del grads, g32
    if want("gather"):
        shard = 64 * 1024 * 1024  # bytes per peer
        shards = [torch.randn(shard // 2, device=DEV).bfloat16() for _ in range(W)]
        dst = torch.empty(W * shard // 2, dtype=torch.bfloat16, device=DEV)
        stt = table(shards)
        for blocks in (64, 0):
            def run3():
                _lib.check(lib.ats_peer_gather(stt, W, _lib.ptr(dst), shard, blocks, _lib.ptr(st), stream), "peer_gather")
            report(f"peer_gather {W} x {shard >> 20} MB, {'64 CTAs (side-stream setting)' if blocks else '592 CTAs'}", time_cuda(run3, iters=a.iters),
                   2 * W * shard)
        del shards, dst
    if want("reduce_rows"):
        grads = [torch.randn(n, device=DEV).bfloat16() for _ in range(W)]
        out32 = torch.zeros(n, dtype=torch.float32, device=DEV)
        gt = table(grads)

        def run4():
            _lib.check(lib.ats_peer_reduce_rows(gt, W, 0, 0, n, _lib.ptr(out32), 1, _lib.ptr(st), 0, stream), "peer_reduce_rows")
        report(f"peer_reduce_rows {n >> 20}M x {W} peers += fp32", time_cuda(run4, iters=a.iters), W * n * 2 + 2 * n * 4)
        del grads, out32
    if want("mod"):
        from adaptivetrainingsystem_b200.ops import mod as D
        B, L, H, keep = 8, 4096, 2048, 512
        h = torch.randn(B, L, H, device=DEV).bfloat16().requires_grad_()
        wr = (torch.randn(1, H, device=DEV) * 0.05).bfloat16().requires_grad_()
        br = torch.zeros(1, device=DEV).bfloat16().requires_grad_()
        base = torch.randn(B, L, H, device=DEV).bfloat16()
        report(f"mod route (scores + select + gather + aux) B{B} L{L} H{H} keep{keep}",
               time_cuda(lambda: D.route(h.detach(), wr.detach(), br.detach(), 1.0, keep), iters=a.iters), B * L * H * 2 + 2 * B * keep * H * 2)
        picked, weight, aux, sel, slot_of, _ = D.route(h, wr, br, 1.0, keep)
        y = picked.detach().clone()
        report(f"mod scatter (out = base + w * y) B{B} L{L} H{H}", time_cuda(lambda: D.scatter(base, y, weight.detach(), sel, slot_of, L), iters=a.iters),
               2 * B * L * H * 2 + B * keep * H * 2)
        gp = torch.randn_like(picked)

        def bwd():
            torch.autograd.grad((picked, aux), (h, wr, br), (gp, torch.ones_like(aux)), retain_graph=True)
        report(f"mod route backward (dh + router gradient) B{B} L{L} H{H}", time_cuda(bwd, iters=a.iters),
               2 * B * L * H * 2 + B * keep * H * 2)
    ops.check_status()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Fused compute+collective paths against their NCCL twins and their rooflines (2 to 8 GPUs of one node).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fused_paths.py

(1) optimiser step: peer-pull gradient reduce + AdamW + parameter push (``parallel/fused.py``) against NCCL reduce-scatter,
    the AdamW kernel and NCCL all-gather; roofline = max(bytes over NVLink / 770 GB/s, 30 B per owned parameter / HBM copy
    bandwidth).
(3) one expert-parallel MoE layer, forward + backward, peer-memory dispatch / pulled combine against ``all_to_all_single``.
Times are CUDA events on the launching stream after warm-up, maximum over ranks.  One JSON line from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402
from adaptivetrainingsystem_b200.config import ModelConfig  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed  # noqa: E402
from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel  # noqa: E402
from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine  # noqa: E402

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction on this pool


def hbm_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def timed(fn, iters, dev):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--inter", type=int, default=5632)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, _, world = init_distributed()
    assert world >= 2, "run under torch.distributed.run with at least two ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    import math
    ep = math.gcd(a.experts, world)
    mesh = ProcessMesh(world, rank, ep_size=ep)
    cfg = ModelConfig(vocab_size=32000, hidden_size=a.hidden, num_layers=a.layers, num_heads=a.hidden // 64, num_kv_heads=4,
                      intermediate_size=a.inter, seq_length=a.seq, use_moe=True, num_experts=a.experts, moe_top_k=2,
                      capacity_factor=1.25, tie_word_embeddings=False)
    g = torch.Generator().manual_seed(7 + rank)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=g).to(dev)
    out = {"n_gpus": world, "config": {"hidden": a.hidden, "layers": a.layers, "experts": a.experts, "tokens_per_rank": a.batch * a.seq,
                                       "parallelism": f"ep{ep}+dp{world}+zero1"}}
    for name, fused in (("nccl", False), ("fused", True)):
        torch.manual_seed(0)
        with torch.device(dev):
            torch.set_default_dtype(torch.bfloat16)
            model = DeepSeekTransformer(cfg, ep_size=mesh.ep_size, ep_rank=mesh.coord.ep)
            torch.set_default_dtype(torch.float32)
        model.rope.cos, model.rope.sin = model.rope.cos.float(), model.rope.sin.float()
        comm = attach_expert_parallel(model, mesh, None, use_fused=fused)
        eng = ShardedEngine(model, lr=1e-4, zero_stage=1, max_grad_norm=1.0, mesh=mesh, fused_comm=comm)

        def fwd_bwd():
            model.forward_loss(ids[:, :-1], ids[:, 1:])["loss"].backward()

        fwd_bwd()
        t_step = timed(eng.step, a.iters, dev)           # gradients stay in the buckets: every call does the full step
        t_fb = timed(fwd_bwd, max(a.iters // 2, 2), dev)  # forward + backward of all layers, expert exchange included
        ops.check_status()
        out[name] = {"optimizer_step_ms": t_step, "forward_backward_ms": t_fb}
        if fused:
            assert eng.fused is not None and eng.fused.usable(eng), "the fused step was not used"
            link_bytes = eng.fused.bytes_over_nvlink_per_step(eng)
            owned = sum(b.shard if b.W > 1 else b.flat_param.numel() for b in eng.buckets)
            t_link = link_bytes / (NVLINK_GBS * 1e6)
            t_hbm = owned * 30 / (hbm_gbs() * 1e6)
            out["optimizer_step_roofline"] = {"nvlink_bytes": link_bytes, "nvlink_ms": t_link, "owned_params": owned, "hbm_ms": t_hbm,
                                              "fraction": max(t_link, t_hbm) / t_step}
        del eng, comm, model
        torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

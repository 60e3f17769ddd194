#!/usr/bin/env python
"""MoE inference benchmark: batch of equal-length random prompts -> prefill, then greedy decode with the GQA KV cache.

    python benchmarks/bench_inference.py [--config mixtral_8x7b] [--batch 64] [--prompt 1024] [--new 256]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_inference.py ...

With several ranks the experts are spread over the ranks (EP = gcd(E, N)), every rank runs the same batch through the
replicated attention / router weights and the routed tokens travel through peer memory.  Prints one JSON line with
prefill and decode tokens/s (device-synchronised wall clock around each phase, max over ranks)."""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from adaptivetrainingsystem_b200 import ops  # noqa: E402
from adaptivetrainingsystem_b200.config import ConfigPresets  # noqa: E402
from adaptivetrainingsystem_b200.inference import GenerationEngine, SamplingParams  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="mixtral_8x7b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="debug only")
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--pack-experts", type=int, default=1, help="store the expert weights tile by tile for serving (1) or keep the training layout (0)")
    a = ap.parse_args()
    rank, local, world = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {"num_layers": a.layers} if a.layers else {}
    cfg = ConfigPresets.get(a.config, gradient_checkpointing=False, **over)
    ep = math.gcd(cfg.num_experts, world) if cfg.use_moe else 1
    mesh = ProcessMesh(world, rank, ep_size=ep)
    mc = cfg.to_model_config()
    # Decode never drops (64 tokens per step fit any expert's 128-row minimum capacity); prefill uses a generous
    # capacity factor so the exchange buffers stay bounded (a dropless prefill would reserve T rows per expert).
    mc.capacity_factor = 2.0
    mc.seq_length = max(mc.seq_length, a.prompt + a.new)
    torch.manual_seed(1234)
    with torch.device(dev):
        torch.set_default_dtype(torch.bfloat16)
        model = DeepSeekTransformer(mc, ep_size=ep, ep_rank=mesh.coord.ep)
        torch.set_default_dtype(torch.float32)
    model.eval()
    if world > 1:
        from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
        attach_expert_parallel(model, mesh, cfg, use_fused=True)
    eng = GenerationEngine(model, pack_experts=bool(a.pack_experts))
    g = torch.Generator().manual_seed(7)  # same prompts on every rank
    ids = torch.randint(0, mc.vocab_size, (a.batch, a.prompt), generator=g).to(dev)
    params = SamplingParams.from_mode("greedy", max_new_tokens=a.new)
    best = None
    for _ in range(a.repeat):
        if world > 1:
            dist.barrier()
        res = eng.generate(ids, params)
        ops.check_status()
        t = torch.tensor([res["prefill_s"], res["decode_s"]], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pre, dec = t.tolist()
        cur = {"prefill_s": pre, "decode_s": dec}
        if best is None or dec < best["decode_s"]:
            best = cur
    out = {"metric": "moe_decode_tokens_per_sec", "value": a.batch * (a.new - 1) / best["decode_s"], "unit": "tokens/s",
           "prefill_tokens_per_sec": a.batch * a.prompt / best["prefill_s"], "n_gpus": world, "dtype": "bf16", "data": "synthetic",
           "ms_per_decode_step": 1e3 * best["decode_s"] / (a.new - 1),
           "config": {"model": a.config, "batch": a.batch, "prompt": a.prompt, "new_tokens": a.new, "layers": mc.num_layers,
                      "parallelism": f"ep{ep}", "params_total": mc.num_parameters(),
                      "expert_weights": "tile-packed" if a.pack_experts else "row-major"},
           "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

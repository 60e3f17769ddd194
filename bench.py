#!/usr/bin/env python
"""Headline benchmark: MoE training throughput (tokens/s, whole job) on N B200s of one node.

    python bench.py --gpus N --steps K --warmup W [--config b1_moe] [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1
--master-port P bench.py --gpus N ...`` (one rank per GPU).  Rank 0 prints ONE JSON line.

* ``value``: K optimiser steps (forward + backward + gradient reduction + clipped AdamW) timed on the device with CUDA
  events between a barrier + synchronize on both sides, max over ranks; inputs already on the device.
* ``e2e``: the same K steps through the public trainer API (``train_step`` + ``optimizer_step``) with each step's batch
  copied from pinned host memory and the loss read back to the host every step.
* weak scaling: the per-GPU micro-batch is fixed, experts are spread over the N ranks (EP = gcd(E, N)), dense weights are
  replicated with ZeRO-1 optimiser sharding.
* ``decode``: the second half of the metric -- MoE decode tokens/s on the Mixtral-8x7B shape (batch 64 x 1024-token prompts, 256
  greedy steps, GQA KV cache, experts spread over the N ranks, batch split over the ranks), measured at the same N after the
  training model has been torn down; ``decode_b1_moe`` is the same workload on the training model's shape, the largest the
  reference's generator can hold (``--impl reference`` reports its cache-less generator on that shape).
* ``fused_check`` (N > 1): before the timed run a two-layer slice of the model takes two optimiser steps through the
  peer-memory kernels and through the NCCL twin of every fused path; the run fails when they disagree.

Synthetic uniform token ids, random-init N(0, 0.02) weights, bf16 compute with fp32 master weights.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_TOKENS_PER_S = {  # reference BENCHMARKS.md rows used for vs_baseline
    "b1_moe": 73000.0,        # "B1 MoE 8x top-2 ~73,000 tok/s" (A100-40GB), BENCHMARKS.md:112-120
    "mixtral_8x7b": 54000.0,  # "B7 MoE 8x top-2 ~54,000 tok/s" (2x A100-80GB), BENCHMARKS.md:168-176
    "dense_1b": 96000.0,      # "B1 dense ~96,000 tok/s" (RTX 4090), BENCHMARKS.md:98-107
    "hybrid_fp8": 91000.0,    # "B1 hybrid ~91,000 tok/s" (A100-40GB), BENCHMARKS.md:137-143
}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs (read-only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([s.strip() for s in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def fused_check(args, cfg_name, mesh, over) -> dict:
    """Two optimiser steps of a two-layer slice: fused peer-memory paths against their NCCL twins (same seeds, same batches).
    Returns the largest relative difference of the losses and of the gradient norms and the smallest cosine similarity of
    any updated parameter."""
    import torch
    import torch.distributed as dist
    from adaptivetrainingsystem_b200 import ops
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models import DeepSeekTransformer
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = ConfigPresets.get(cfg_name, num_workers=0, gradient_checkpointing=False, **{**over, "num_layers": 2})
    mc = cfg.to_model_config()
    g = torch.Generator().manual_seed(4321 + mesh.rank)
    ids = torch.randint(0, cfg.vocab_size, (2, 1025), generator=g).to(dev)
    runs = {}
    for name, fused in (("nccl", False), ("fused", True)):
        torch.manual_seed(77)
        with torch.device(dev):
            torch.set_default_dtype(torch.bfloat16)
            model = DeepSeekTransformer(mc, ep_size=mesh.ep_size, ep_rank=mesh.coord.ep)
            torch.set_default_dtype(torch.float32)
        model.rope.cos, model.rope.sin = model.rope.cos.float(), model.rope.sin.float()
        comm = attach_expert_parallel(model, mesh, cfg, use_fused=fused)
        if cfg.zero_stage >= 3 and mesh.ep_size == 1:
            from adaptivetrainingsystem_b200.parallel.zero3 import ZeRO3Engine
            eng = ZeRO3Engine(model, lr=1e-3, max_grad_norm=1.0, mesh=mesh, fused_comm=comm)
        else:
            eng = ShardedEngine(model, lr=1e-3, zero_stage=max(min(cfg.zero_stage, 2), 1), max_grad_norm=1.0, mesh=mesh, fused_comm=comm)
        losses = []
        for _ in range(2):
            out = model.forward_loss(ids[:, :-1], ids[:, 1:])
            out["loss"].backward()
            eng.step()
            losses.append(out["loss"].detach().float())
        torch.cuda.synchronize()
        ops.check_status()
        if hasattr(eng, "gather_full_parameters"):
            eng.gather_full_parameters()
            used = bool(fused and eng.fused)
        else:
            used = bool(fused and comm is not None and comm.usable(eng))
        runs[name] = (torch.stack(losses), float(eng.last_grad_norm), {k: v.detach().float().clone() for k, v in model.state_dict().items()}, used)
        ep_comm = getattr(model, "_ep_comm", None)
        if hasattr(eng, "close"):
            eng.close()
        del eng, model
        if ep_comm is not None:
            ep_comm.close()
        if comm is not None:
            comm.close()
        torch.cuda.empty_cache()
    (ln, gn, sn, _), (lf, gf, sf, used) = runs["nccl"], runs["fused"]
    loss_err = float(((ln - lf).abs() / ln.abs().clamp(min=1e-6)).max())
    norm_err = abs(gn - gf) / max(abs(gn), 1e-6)
    cos = min(float(torch.nn.functional.cosine_similarity(sf[k].flatten(), sn[k].flatten(), dim=0)) for k in sn if sn[k].numel() > 1)
    t = torch.tensor([loss_err, norm_err, -cos], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    loss_err, norm_err, cos = float(t[0]), float(t[1]), -float(t[2])
    ok = used and loss_err < 2e-2 and norm_err < 3e-2 and cos > 0.999
    return {"max_rel_err": max(loss_err, norm_err), "loss_rel_err": loss_err, "grad_norm_rel_err": norm_err, "min_param_cosine": cos,
            "fused_step_used": used, "layers": 2, "steps": 2, "ok": bool(ok)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from adaptivetrainingsystem_b200 import ops
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models import DeepSeekTransformer
    from adaptivetrainingsystem_b200.ops import _lib
    from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer

    rank, local_rank, world = init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {}
    if args.micro_batch:
        over.update(batch_size=args.micro_batch, micro_batch_size=args.micro_batch)
    if args.layers:
        over["num_layers"] = args.layers
    if args.seq:
        over["seq_length"] = args.seq
    if args.accum:
        over["gradient_accumulation_steps"] = args.accum
    if args.precision:
        over["precision"] = args.precision
    cfg = ConfigPresets.get(args.config, num_workers=0, gradient_checkpointing=bool(args.checkpoint), **over)
    cfg.fused_comm = not args.nccl_only
    ep = math.gcd(cfg.num_experts, world) if cfg.use_moe else 1
    mesh = ProcessMesh(world, rank, ep_size=ep)
    cfg.world_size, cfg.expert_parallel_size = world, ep
    check = None
    if world > 1 and cfg.fused_comm and not args.no_fused_check:
        check = fused_check(args, args.config, mesh, over)
        if not check["ok"]:
            raise SystemExit(f"fused paths disagree with their NCCL twins: {json.dumps(check)}")
    torch.manual_seed(1234)
    mc = cfg.to_model_config()
    with torch.device(dev):
        torch.set_default_dtype(torch.bfloat16)
        model = DeepSeekTransformer(mc, ep_size=ep, ep_rank=mesh.coord.ep)
        torch.set_default_dtype(torch.float32)
    model.rope.cos, model.rope.sin = model.rope.cos.float(), model.rope.sin.float()
    fused = attach_expert_parallel(model, mesh, cfg, use_fused=cfg.fused_comm) if world > 1 else None
    trainer = EnhancedConversationTrainer(model, None, cfg, mesh=mesh, fused_comm=fused)
    # a real schedule over the steps this run takes (warm-up, timed, end-to-end): the recorded losses show the model learning
    trainer._setup_scheduler(args.warmup + 2 * args.steps + 1)

    mb, L, V = cfg.micro_batch_size, cfg.seq_length, cfg.vocab_size
    g = torch.Generator().manual_seed(99 + rank)
    n_batches = 4
    host = []
    for _ in range(n_batches):
        ids = torch.randint(0, V, (mb, L + 1), generator=g)
        host.append({"input_ids": ids[:, :-1].contiguous().pin_memory(), "labels": ids[:, 1:].contiguous().pin_memory()})
    devb = [{k: v.to(dev) for k, v in b.items()} for b in host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    accum = max(cfg.gradient_accumulation_steps, 1)

    def step_device(i):
        out = None
        for a in range(accum):
            out = trainer.train_step(devb[(i * accum + a) % n_batches])
        trainer.optimizer_step()
        trainer._pending_device.clear()
        return out["loss"]

    def step_e2e(i):
        out = None
        for a in range(accum):
            b = host[(i * accum + a) % n_batches]
            batch = {k: v.to(dev, non_blocking=True) for k, v in b.items()}
            out = trainer.train_step(batch)
        trainer.optimizer_step()
        trainer._pending_device.clear()
        return float(out["loss"])  # device -> host read every step

    first_loss = None
    for i in range(args.warmup):
        loss = step_device(i)
        if i == 0:
            first_loss = float(loss)
    ops.check_status()
    barrier()
    ep_comm0 = getattr(model, "_ep_comm", None)
    bars = {"expert_exchange": getattr(ep_comm0, "barrier", None), "optimizer_step": getattr(fused, "barrier", None)}
    for b_ in bars.values():
        if b_ is not None:
            b_.wait_statistics(reset=True)
    launches0 = _lib.launch_count()
    with ClockSampler(torch.cuda.current_device()) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            step_device(i)
        e1.record()
        barrier()
    launches = _lib.launch_count() - launches0
    # time the flag barriers of the timed region spent waiting (per rank: the rank that waits least is the one the others wait for)
    barrier_wait = {}
    for name, b_ in bars.items():
        if b_ is None or world == 1:
            continue
        stt = b_.wait_statistics(reset=True)
        t_ = torch.tensor([stt["max_peer_ms"] / args.steps, float(stt["calls"]) / args.steps], device=dev)
        allr = [torch.zeros_like(t_) for _ in range(world)]
        dist.all_gather(allr, t_)
        barrier_wait[name] = {"calls_per_step": allr[0][1].item(), "wait_ms_per_step_by_rank": [round(a[0].item(), 2) for a in allr]}
    ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    ops.check_status()

    # end to end through the public API
    step_e2e(0)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    f0.record()
    last = 0.0
    for i in range(args.steps):
        last = step_e2e(i)
    f1.record()
    barrier()
    e2e_ms = max(f0.elapsed_time(f1), (time.perf_counter() - w0) * 1e3) / args.steps
    t = torch.tensor([e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t)

    tokens = mb * L * world * accum
    value = tokens / (ms / 1e3)
    routing = model.get_routing_statistics() if cfg.use_moe else {}
    dropped = [v["dropped_fraction"] for v in routing.values()]
    dropped_fraction = sum(dropped) / len(dropped) if dropped else 0.0
    pub = PUBLISHED_TOKENS_PER_S.get(args.config)
    h2d = accum * sum(v.numel() * v.element_size() for v in host[0].values())
    res = {
        "metric": "moe_train_tokens_per_sec" if cfg.use_moe else "train_tokens_per_sec", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": (value / pub) if pub else None, "dtype": "fp8+bf16" if "fp8" in str(cfg.precision) else "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": args.config, "global_batch": mb * world * accum, "micro_batch_per_gpu": mb, "grad_accumulation": accum, "seq_len": L, "parallelism": mesh.describe() + f"+zero{cfg.zero_stage}",
                   "hidden": cfg.hidden_size, "layers": cfg.num_layers, "experts": cfg.num_experts if cfg.use_moe else 0,
                   "top_k": cfg.moe_top_k if cfg.use_moe else 0, "params_total": mc.num_parameters(),
                   "params_active": mc.num_parameters(True), "l2": "working set per step (weights + activations) far exceeds the 126 MB L2",
                   "fused_comm": bool(cfg.fused_comm), "attention_backend": os.environ.get("ATS_ATTN", "native"),
                   "capacity_factor": cfg.capacity_factor if cfg.use_moe else None, "drop_tokens": bool(cfg.drop_tokens) if cfg.use_moe else None,
                   "dropped_slot_fraction": dropped_fraction, "lr_schedule_steps": args.warmup + 2 * args.steps + 1,
                   "loss_first": first_loss, "loss_last": last,
                   **({"precision_note": "e4m3 with per-token / per-channel scales for the forward and input-gradient products of every linear and expert; weight gradients, attention and the SwiGLU-backward product in bf16; fp32 accumulation, master weights and optimiser state"}
                      if "fp8" in str(cfg.precision) else {})},
        "clocks": clk.summary(),
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
    }
    if check is not None:
        res["fused_check"] = check
    if barrier_wait:
        res["barrier_wait"] = barrier_wait
    # tear the training job down (buckets and exchange buffers live outside PyTorch's allocator) before the serving models are built
    trainer.shutdown()
    ep_comm = getattr(model, "_ep_comm", None)
    if hasattr(trainer.engine, "close"):
        trainer.engine.close()
    del trainer, devb, model
    import gc
    gc.collect()
    if ep_comm is not None:
        ep_comm.close()
    if fused is not None:
        fused.close()
    torch.cuda.empty_cache()
    if not args.no_decode:
        from adaptivetrainingsystem_b200.inference.benchmark import run_decode_benchmark
        torch.cuda.reset_peak_memory_stats()
        res["decode"] = run_decode_benchmark("mixtral_8x7b", 64, 1024, 256, layers=args.decode_layers, repeat=2)
        torch.cuda.reset_peak_memory_stats()
        res["decode_b1_moe"] = run_decode_benchmark("b1_moe", 64, 1024, 256, layers=args.decode_layers, repeat=2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return res if rank == 0 else {}


def run_reference(args) -> dict:
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        from reference_arm import run as run_ref
    except Exception as e:
        return {"impl": "reference", "unavailable": f"reference arm not importable: {e!r}"[:300]}
    return run_ref(args, PUBLISHED_TOKENS_PER_S)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="b1_moe")
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: a run with fewer layers is not a benchmark number")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--accum", type=int, default=0)
    ap.add_argument("--checkpoint", type=int, default=0)
    ap.add_argument("--precision", default="", help="override the preset's precision (e.g. mixed_bf16 for the bf16 twin of hybrid_fp8)")
    ap.add_argument("--nccl-only", action="store_true", help="baseline path: NCCL collectives instead of the fused peer-memory kernels")
    ap.add_argument("--no-decode", action="store_true", help="skip the serving half of the metric")
    ap.add_argument("--no-fused-check", action="store_true", help="skip the fused-vs-NCCL check that precedes a multi-GPU run")
    ap.add_argument("--decode-layers", type=int, default=0, help="debug only: serving models with fewer layers")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res and int(os.environ.get("RANK", "0")) == 0:  # one JSON line per job
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()

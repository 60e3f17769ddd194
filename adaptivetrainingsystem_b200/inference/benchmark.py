"""Serving benchmark shared by ``bench.py`` and ``benchmarks/bench_inference.py``: a batch of equal-length random prompts is
prefilled, then decoded greedily with the grouped-query KV cache, the decode step replayed from a CUDA graph.

With several ranks the experts are spread over the ranks (EP = gcd(E, N)) and the batch is split: every rank serves
``batch / N`` sequences with their KV cache through the replicated attention / router weights, and the routed tokens of all
ranks meet at the experts through peer memory (``parallel/expert_parallel.py: ep_moe_serving``).  Both phases are timed on
the device with CUDA events between device-wide synchronisations; the figure of a phase is the maximum over the ranks.

The reference has no counterpart of this runtime: its generator re-runs the whole context for every token of one sequence
(reference ``Chat.py:355-465``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist


def run_decode_benchmark(config_name: str = "mixtral_8x7b", batch: int = 64, prompt: int = 1024, new_tokens: int = 256,
                         layers: int = 0, pack_experts: bool = True, repeat: int = 2, mesh=None, quantize: Optional[str] = None) -> Dict[str, Any]:
    """Builds the model of ``config_name`` with random bf16 weights on the current device (experts spread over the ranks of the
    initialised process group), runs ``repeat`` passes and returns the best prefill and decode figures.  Collective: every
    rank calls it; every rank gets the same dictionary."""
    from .. import ops
    from ..config import ConfigPresets
    from ..models import DeepSeekTransformer
    from ..parallel import ProcessMesh
    from .engine import GenerationEngine, SamplingParams, sample_next

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    if batch % world:
        raise ValueError(f"batch {batch} must be divisible by the number of ranks ({world})")
    over = {"num_layers": layers} if layers else {}
    cfg = ConfigPresets.get(config_name, gradient_checkpointing=False, **over)
    ep = math.gcd(cfg.num_experts, world) if cfg.use_moe else 1
    mesh = mesh or ProcessMesh(world, rank, ep_size=ep)
    mc = cfg.to_model_config()
    # A decode step never drops (every rank's rows fit the expert's row block); the prefill uses a generous capacity factor so
    # that the exchange buffers stay bounded (a dropless prefill would reserve one row per token and expert).
    mc.capacity_factor = 2.0
    mc.seq_length = max(mc.seq_length, prompt + new_tokens)
    torch.manual_seed(1234)
    with torch.device(dev):
        torch.set_default_dtype(torch.bfloat16)
        model = DeepSeekTransformer(mc, ep_size=ep, ep_rank=mesh.coord.ep)
        torch.set_default_dtype(torch.float32)
    model.eval()
    comm = None
    if world > 1 and ep > 1:
        from ..parallel.expert_parallel import attach_expert_parallel
        attach_expert_parallel(model, mesh, cfg, use_fused=True)
        comm = getattr(model, "_ep_comm", None)
    qm = None
    if quantize:
        # post-training quantisation (reported with its own dtype; the headline decode figure is the bf16 one)
        from types import SimpleNamespace
        from ..training.precision import QuantizationManager
        qm = QuantizationManager(SimpleNamespace(quantization_method=quantize, quantization_bits=4 if quantize in ("int4", "gptq") else 8))
        qm.quantize_model(model)
    eng = GenerationEngine(model, pack_experts=pack_experts)
    per = batch // world
    g = torch.Generator().manual_seed(7)  # one prompt set; every rank serves its own slice of it
    ids = torch.randint(0, mc.vocab_size, (batch, prompt), generator=g)[rank * per:(rank + 1) * per].to(dev)
    params = SamplingParams.from_mode("greedy", max_new_tokens=new_tokens)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    best: Optional[Dict[str, float]] = None
    tokens_out = None
    with torch.no_grad():
        for _ in range(max(repeat, 1)):
            cache = model.make_cache(per, prompt + new_tokens)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            sync()
            ev[0].record()
            logits = eng.prefill(ids, cache)
            ev[1].record()
            sync()
            decoder = eng.graph_decoder(cache)  # capture (and its warm-up steps) is not part of the steady-state figure
            out = []
            sync()
            ev[2].record()
            for step in range(new_tokens):
                nxt = sample_next(logits, params, None, None)
                out.append(nxt)
                if step + 1 < new_tokens:
                    logits = decoder.step(nxt)
            tokens_out = torch.stack(out, dim=1).cpu()  # the generated ids reach the host inside the timed region
            ev[3].record()
            sync()
            ops.check_status()
            t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            pre_ms, dec_ms = t.tolist()
            best = {"prefill_ms": pre_ms, "decode_ms": dec_ms} if best is None else {
                "prefill_ms": min(pre_ms, best["prefill_ms"]), "decode_ms": min(dec_ms, best["decode_ms"])}
            del decoder, cache
    steps = max(new_tokens - 1, 1)
    res = {"metric": "moe_decode_tokens_per_sec", "value": batch * steps / (best["decode_ms"] / 1e3), "unit": "tokens/s",
           "ms_per_decode_step": best["decode_ms"] / steps, "prefill_tokens_per_sec": batch * prompt / (best["prefill_ms"] / 1e3),
           "prefill_ms": best["prefill_ms"], "n_gpus": world, "dtype": "bf16" if not quantize else (f"{quantize} weights, bf16 activations and attention" if quantize in ("int4", "gptq")
                                                                   else f"{quantize} weights and activations, bf16 attention"), "data": "synthetic",
           "timing": "CUDA events, max over ranks; decode = sampling kernel + graph-replayed step, ids copied to the host at the end",
           "config": {"model": config_name, "batch": batch, "prompt": prompt, "new_tokens": new_tokens, "layers": mc.num_layers,
                      "parallelism": f"ep{ep}" if ep > 1 else "1 GPU", "sequences_per_rank": per, "params_total": mc.num_parameters(),
                      "expert_weights": "tile-packed" if pack_experts else "row-major", "kv_cache": "GQA, bf16, contiguous per sequence"},
           "tokens_checksum": int(tokens_out.sum()) if tokens_out is not None else 0,
           "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    # weights every rank streams per decode step: its experts plus the replicated attention / head weights
    dense = sum(p.numel() for n, p in model.named_parameters() if not getattr(p, "_ats_expert", False) and "embed_tokens" not in n)
    expert = sum(p.numel() for p in model.parameters() if getattr(p, "_ats_expert", False))
    res["weight_gb_per_step_per_gpu"] = 2 * (dense + expert) / 1e9
    res["weight_stream_tb_per_s_per_gpu"] = 2 * (dense + expert) / 1e12 / (res["ms_per_decode_step"] / 1e3)
    if qm is not None:
        from ..ops import fp8, int4, int8
        res["quantized_bytes"] = qm.quantized_bytes
        fp8.set_enabled(False)
        fp8.clear_weight_cache()
        int8.set_enabled(False)
        int8.clear()
        int4.set_enabled(False)
        int4.clear()
    del eng, model
    if comm is not None:
        comm.close()
    torch.cuda.empty_cache()
    return res

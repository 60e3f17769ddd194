"""Reference arm of bench.py: the UNMODIFIED reference (installed into ``baseline/_ref``) on the same metric and
config as our arm, through the reference's own public API and stock code path.

* N = 1: ``EnhancedConversationTrainer.train_step`` / ``optimizer_step`` on ``DeepSeekTransformer`` -- the "pytorch" backend
  its entry script selects on a single GPU (fp32 parameters, bf16 autocast, flash-attn, fused AdamW, clip 1.0).
* N > 1: its ``FSDPBackend`` wrapper (FULL_SHARD, bf16 mixed precision, NCCL) -- the only sharded backend of the reference
  that can run offline (DeepSpeed and ColossalAI are not installable here); loss = the trainer's cross-entropy + aux loss.

Nothing of this repository's models, kernels or engine is imported on this path.  Only the data differ from the
reference's pipeline: synthetic uniform token ids (there is no dataset and its tokenizer needs the network), fed as the
batch dictionaries its datasets produce.  If a micro-batch does not fit, the micro-batch is halved and accumulation
doubled (same tokens per optimiser step), which is what the reference's own OOM wrapper does.
"""
from __future__ import annotations

import json
import logging
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

SHAPES = {
    "b1_moe": dict(vocab_size=32000, hidden_size=2048, num_layers=22, num_heads=32, num_kv_heads=4, intermediate_size=5632,
                   seq_length=2048, use_moe=True, num_experts=8, moe_top_k=2, micro_batch=8, accum=4),
    "dense_1b": dict(vocab_size=32000, hidden_size=2048, num_layers=22, num_heads=32, num_kv_heads=4, intermediate_size=5632,
                     seq_length=2048, use_moe=False, num_experts=8, moe_top_k=2, micro_batch=8, accum=1),
    "mixtral_8x7b": dict(vocab_size=32000, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, intermediate_size=14336,
                         seq_length=4096, use_moe=True, num_experts=8, moe_top_k=2, micro_batch=1, accum=1),
}


def reference_decode(shape_name: str, prompt: int = 1024, new_tokens: int = 256, time_limit_s: float = 75.0) -> dict:
    """The reference's own generator (``Chat.GenerationEngine.generate``: one sequence, no KV cache, the whole context is
    re-run for every token, fp32 parameters as ``Chat.py`` loads them) on prompts of the serving workload, greedy
    (top_k = 1), for as many sequences as fit the time limit.  Tokens per second = generated tokens / device-synchronised
    wall time.  Runs on one GPU: the reference has no multi-device inference path."""
    import contextlib
    import io
    import torch
    shape = dict(SHAPES[shape_name])
    shape.pop("micro_batch"), shape.pop("accum")
    n_params_fp32_gb = None
    sink = io.StringIO()
    try:
        with contextlib.redirect_stdout(sink):
            import Chat  # the reference's chat script, installed next to its packages
            from core.model import DeepSeekConfig, DeepSeekTransformer
    except Exception as e:
        return {"unavailable": f"reference generator not importable: {e!r}"[:300]}
    dev = torch.device("cuda", torch.cuda.current_device())
    h, i, e, l, v = shape["hidden_size"], shape["intermediate_size"], shape["num_experts"], shape["num_layers"], shape["vocab_size"]
    kv = shape["num_kv_heads"] * (h // shape["num_heads"])
    n_params = l * ((e if shape["use_moe"] else 1) * 3 * h * i + h * (2 * h + 2 * kv)) + 2 * v * h
    n_params_fp32_gb = 4 * n_params / 1e9
    free_gb = torch.cuda.mem_get_info()[0] / 1e9
    if n_params_fp32_gb > 0.9 * free_gb:
        return {"unavailable": f"reference generator holds fp32 parameters on one device (Chat.py:544): {n_params / 1e9:.1f} B parameters "
                               f"= {n_params_fp32_gb:.0f} GB, {free_gb:.0f} GB free; it has no multi-device inference path"}
    try:
        with contextlib.redirect_stdout(sink):
            torch.manual_seed(1234)
            mcfg = DeepSeekConfig(tie_word_embeddings=False, use_flash_attention=True, gradient_checkpointing=False, **shape)
            model = DeepSeekTransformer(mcfg)
            for m in model.modules():
                if isinstance(m, (torch.nn.Linear, torch.nn.Embedding)):
                    torch.nn.init.normal_(m.weight, std=0.02)
            model = model.to(dev)  # fp32, as Chat.py:544 does

            class _Tok:
                def decode(self, ids):
                    return ""
            eng = Chat.GenerationEngine(model, _Tok(), dev)
            Chat.HardcodedConfig.CONTEXT_WINDOW = max(Chat.HardcodedConfig.CONTEXT_WINDOW, prompt + new_tokens + 16)
            g = torch.Generator().manual_seed(7)
            prompts = torch.randint(1, v, (64, prompt), generator=g)
            eng.generate(prompts[0, :64].tolist(), 4, 1.0, 1.0, 1, 1.0, stream=False)  # warm-up: short prompt, four tokens
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            total, seqs = 0, 0
            while seqs < 64 and time.perf_counter() - t0 < time_limit_s:
                budget = time_limit_s - (time.perf_counter() - t0)
                # a sequence that would overrun the limit by far is cut short: per-token cost is known after the first one
                n_new = new_tokens if seqs == 0 else max(8, min(new_tokens, int(budget / max(per_token, 1e-6))))
                toks, _ = eng.generate(prompts[seqs].tolist(), n_new, 1.0, 1.0, 1, 1.0, stream=False)
                torch.cuda.synchronize()
                total += len(toks)
                seqs += 1
                per_token = (time.perf_counter() - t0) / max(total, 1)
            dt = time.perf_counter() - t0
    except Exception as e:
        return {"unavailable": f"reference generator failed on its own code path: {type(e).__name__}: {e}"[:300]}
    res = {"metric": "moe_decode_tokens_per_sec", "value": total / dt, "unit": "tokens/s", "ms_per_token": 1e3 * dt / max(total, 1),
           "n_gpus": 1, "dtype": "fp32 parameters (Chat.py:544)", "data": "synthetic",
           "config": {"model": shape_name, "batch": 1, "prompt": prompt, "new_tokens": new_tokens, "sequences_run": seqs,
                      "tokens_generated": total, "time_limit_s": time_limit_s, "kv_cache": "none (whole context re-run per token)",
                      "sampling": "top_k = 1 through its multinomial sampler"},
           "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    del eng, model
    torch.cuda.empty_cache()
    return res


class _Tokenizer:
    """Stand-in with the attributes the reference trainer reads; the benchmark feeds token ids directly."""
    pad_token_id = -1  # no id of the synthetic data is padding
    special_tokens = {}

    def __init__(self, vocab):
        self.vocab_size = vocab

    def get_vocab_size(self):
        return self.vocab_size


def run(args, published) -> dict:
    if not os.path.isdir(os.path.join(REF, "core")):
        return {"impl": "reference", "unavailable": "baseline/_ref is empty: the reference was not installed on this machine"}
    if args.config not in SHAPES:
        return {"impl": "reference", "unavailable": f"no reference shape for config {args.config}"}
    sys.path.insert(0, REF)
    logging.disable(logging.WARNING)
    import contextlib
    import io
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        return {"impl": "reference", "unavailable": f"--gpus {args.gpus} but WORLD_SIZE={world}"}
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    shape = dict(SHAPES[args.config])
    mb, accum = shape.pop("micro_batch"), shape.pop("accum")
    if world > 1 and args.config in ("b1_moe", "dense_1b") and not args.layers and mb > 2:
        # the micro-batch the reference's single-GPU run settles at after its out-of-memory halving (8 -> 2: its attention keeps
        # the [heads, L, L] score tensors of every layer for the backward pass), with the accumulation raised so that the tokens
        # per step stay the same; ranks of a multi-GPU job cannot halve independently without desynchronising their collectives
        mb, accum = 2, accum * (mb // 2)
    if args.micro_batch:
        mb = args.micro_batch
    if args.accum:
        accum = args.accum
    if args.layers:
        shape["num_layers"] = args.layers
    sink = io.StringIO()
    try:
        with contextlib.redirect_stdout(sink):  # the reference prints banners on import
            from config.config_manager import Config
            from core.model import DeepSeekConfig, DeepSeekTransformer
            from training.trainer import EnhancedConversationTrainer
            from backend.backend_fsdp import FSDPBackend
    except Exception as e:
        return {"impl": "reference", "unavailable": f"reference import failed: {e!r}"[:300]}

    tokens_per_step = None
    trainer = backend = model = devb = host = None
    while True:
        try:
            with contextlib.redirect_stdout(sink):
                torch.manual_seed(1234)
                mcfg = DeepSeekConfig(tie_word_embeddings=False, use_flash_attention=True, gradient_checkpointing=False,
                                      **{k: v for k, v in shape.items()})
                cfg = Config(vocab_size=shape["vocab_size"], hidden_size=shape["hidden_size"], num_layers=shape["num_layers"],
                             num_heads=shape["num_heads"], num_kv_heads=shape["num_kv_heads"], seq_length=shape["seq_length"],
                             intermediate_size=shape["intermediate_size"], batch_size=mb, micro_batch_size=mb,
                             gradient_accumulation_steps=accum, precision="mixed_bf16", use_moe=shape["use_moe"], use_mod=False,
                             num_experts=shape["num_experts"], moe_top_k=shape["moe_top_k"], use_deepspeed=False, compile=False,
                             gradient_checkpointing=False, learning_rate=1e-4)
                cfg.max_grad_norm = 1.0
                cfg.fsdp_sharding_strategy = "FULL_SHARD"
                # The size-based wrap policy of the reference's FSDP backend calls a bool (backend_fsdp.py:183-185, "recurse(module)")
                # and raises TypeError under this PyTorch; its own switch for running without a policy is a threshold <= 0
                # (backend_fsdp.py:166-167), which wraps the model as one FSDP unit.
                cfg.fsdp_auto_wrap_threshold = 0
                model = DeepSeekTransformer(mcfg)
                for m in model.modules():  # the entry script re-initialises every Linear / Embedding with N(0, 0.02)
                    if isinstance(m, (torch.nn.Linear, torch.nn.Embedding)):
                        torch.nn.init.normal_(m.weight, std=0.02)
                if world == 1:
                    trainer = EnhancedConversationTrainer(model, _Tokenizer(shape["vocab_size"]), cfg, logging.getLogger("reference"))
                    backend = None
                else:
                    # bf16 MixedPrecision of the reference's FSDP backend breaks inside its own MoE layer (index_add_ of a float
                    # source into a bf16 buffer raises); the configuration of its single-GPU path -- fp32 parameters, bf16 autocast
                    # around the forward -- is what runs here as well (precision "fp32" selects no MixedPrecision policy).
                    cfg.precision = "fp32"
                    backend = FSDPBackend(model, cfg)
                    trainer = None
            L, V = shape["seq_length"], shape["vocab_size"]
            g = torch.Generator().manual_seed(99 + rank)
            host = []
            for _ in range(4):
                ids = torch.randint(0, V, (mb, L + 1), generator=g)
                host.append({"input_ids": ids[:, :-1].contiguous().pin_memory(), "labels": ids[:, 1:].contiguous().pin_memory(),
                             "attention_mask": torch.ones(mb, L).pin_memory(), "loss_weights": torch.ones(mb, L).pin_memory()})
            devb = [{k: v.to(dev) for k, v in b.items()} for b in host]

            def micro(batch):
                if trainer is not None:
                    with contextlib.redirect_stdout(sink):
                        return trainer.train_step(batch)["loss"]
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    out = backend(batch["input_ids"], batch["attention_mask"])
                    logits, aux = (out[0], out[1]) if isinstance(out, tuple) else (out, 0.0)
                    loss = F.cross_entropy(logits.float().view(-1, logits.size(-1)), batch["labels"].reshape(-1)) + aux
                backend.backward(loss / accum)
                return loss

            def opt_step():
                if trainer is not None:
                    with contextlib.redirect_stdout(sink):
                        trainer.optimizer_step()
                else:
                    backend.step()
                    backend.zero_grad()

            def step(i, from_host):
                last = None
                for a in range(accum):
                    b = host[(i * accum + a) % 4] if from_host else devb[(i * accum + a) % 4]
                    if from_host:
                        b = {k: v.to(dev, non_blocking=True) for k, v in b.items()}
                    last = micro(b)
                opt_step()
                return last

            def barrier():
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()

            for i in range(args.warmup):
                step(i, False)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step(i, False)
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1) / args.steps
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0 = time.perf_counter()
            f0.record()
            last = 0.0
            for i in range(args.steps):
                last = float(step(i, True))
            f1.record()
            barrier()
            e2e_ms = max(f0.elapsed_time(f1), (time.perf_counter() - w0) * 1e3) / args.steps
            tokens_per_step = mb * L * accum * world
            break
        except torch.cuda.OutOfMemoryError:
            if world > 1:  # ranks cannot halve independently without desynchronising their collectives
                return {"impl": "reference", "unavailable": f"reference FSDP backend runs out of memory on config {args.config} at {world} GPUs"}
            if mb == 1:
                return {"impl": "reference", "unavailable": f"reference runs out of memory on config {args.config} at {world} GPU(s) even with micro-batch 1"}
            trainer = backend = model = devb = host = None
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            mb, accum = mb // 2, accum * 2
        except Exception as e:  # a defect of the reference on this software stack: report, do not crash the benchmark
            return {"impl": "reference", "unavailable": f"reference failed on its own code path: {type(e).__name__}: {e}"[:300]}
    t = torch.tensor([ms, e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    value = tokens_per_step / (ms / 1e3)
    pub = published.get(args.config)
    res = {"impl": "reference", "metric": "moe_train_tokens_per_sec" if shape["use_moe"] else "train_tokens_per_sec", "value": value,
           "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": value / pub if pub else None, "dtype": "bf16 autocast, fp32 parameters", "data": "synthetic",
           "config": {"model": args.config, "global_batch": mb * accum * world, "micro_batch_per_gpu": mb, "grad_accumulation": accum,
                      "seq_len": shape["seq_length"], "layers": shape["num_layers"],
                      "parallelism": "single GPU, reference trainer" if world == 1 else f"reference FSDPBackend FULL_SHARD x{world}",
                      "loss_last": last},
           "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                   "h2d_bytes_per_step": accum * sum(v.numel() * v.element_size() for v in host[0].values()), "d2h_bytes_per_step": 4},
           "gpu_launches": 0, "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    if not getattr(args, "no_decode", False):
        # serving half of the metric: the reference's generator is single-device, so rank 0 runs it alone after the training
        # objects are gone (the other ranks wait at the barrier below)
        trainer = backend = model = devb = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        if rank == 0:
            res["decode"] = reference_decode("mixtral_8x7b")
            res["decode_b1_moe"] = reference_decode("b1_moe")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return res if rank == 0 else {}

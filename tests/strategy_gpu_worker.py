"""Worker run under ``torch.distributed.run`` by test_gpu_multi.py on 2 GPUs (NCCL): tensor, sequence and pipeline parallelism chosen
through ``Config`` and applied by the trainer, each against the same training steps of one process on this rank's GPU (bf16,
native kernels on both sides)."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402
from adaptivetrainingsystem_b200.config import Config  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed  # noqa: E402
from adaptivetrainingsystem_b200.parallel.strategy import gather_tensor_parallel_state  # noqa: E402
from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer  # noqa: E402


def config(tmp, **kw):
    base = dict(vocab_size=1024, hidden_size=256, num_layers=4, num_heads=4, num_kv_heads=2, intermediate_size=512, seq_length=256,
                use_moe=False, precision="mixed_bf16", gradient_checkpointing=False, tie_word_embeddings=False, learning_rate=2e-3,
                batch_size=2, micro_batch_size=2, gradient_accumulation_steps=2, zero_stage=1, output_dir=tmp, experiment_name="s",
                num_workers=0, heartbeat_interval_s=0.0, use_lr_scheduler=False, weight_decay=0.0, fused_comm=False)
    base.update(kw)
    return Config(**base)


def data(dev):
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 1024, (4, 257), generator=g).to(dev)
    return [{"input_ids": ids[2 * i:2 * i + 2, :-1], "labels": ids[2 * i:2 * i + 2, 1:]} for i in range(2)]


def train(trainer, dev, steps=3):
    losses = []
    for _ in range(steps):
        for mb in data(dev):
            out = trainer.train_step(mb)
            losses.append(float(out["loss"]))
        trainer.optimizer_step()
    return losses


def build(cfg, init, dev):
    with torch.device(dev):
        torch.set_default_dtype(torch.bfloat16)
        model = DeepSeekTransformer(cfg.to_model_config())
        torch.set_default_dtype(torch.float32)
    if init is not None:
        model.load_state_dict(init)
    return model


def main():
    rank, local, world = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    tmp = tempfile.mkdtemp(prefix=f"ats_strategy_r{rank}_")
    torch.manual_seed(0)
    ref_model = build(config(tmp), None, dev)
    init = {k: v.clone() for k, v in ref_model.state_dict().items()}
    for k in init:                       # the same start on every rank
        dist.broadcast(init[k], 0)
    ref_model.load_state_dict(init)
    ref_tr = EnhancedConversationTrainer(ref_model, None, config(tmp), mesh=ProcessMesh(1, 0, create_groups=False))
    ref_losses = train(ref_tr, dev)
    ref_final = {k: v.detach().float().clone() for k, v in ref_model.state_dict().items()}
    assert ref_losses[-1] < ref_losses[0] - 0.05, ref_losses
    report = {}
    for kind, extra in (("tp", dict(tensor_parallel_size=2)), ("sp", dict(sequence_parallel_size=2)),
                        ("pp", dict(pipeline_parallel_size=2)), ("pp_interleaved", dict(pipeline_parallel_size=2, pipeline_chunks=2))):
        cfg = config(os.path.join(tmp, kind), **extra)
        mesh = ProcessMesh.from_config(cfg, world, rank)
        model = build(cfg, init, dev)
        tr = EnhancedConversationTrainer(model, None, cfg, mesh=mesh)
        losses = train(tr, dev)
        torch.cuda.synchronize()
        ops.check_status()
        got = gather_tensor_parallel_state(model, mesh) if kind == "tp" else model.state_dict()
        worst, checked = 1.0, 0
        for k, v in ref_final.items():
            if k not in got or got[k].numel() == 0:
                continue
            a, b = got[k].detach().float().flatten().to(dev), v.flatten()
            assert a.shape == b.shape, (kind, k)
            cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
            worst = min(worst, cos)
            checked += 1
        assert checked >= (len(ref_final) if kind in ("tp", "sp") else 8), (kind, checked)
        assert worst > 0.999, (kind, worst)
        if kind in ("tp", "sp"):         # every rank sees the loss of the whole batch
            for a, b in zip(losses, ref_losses):
                assert abs(a - b) < 3e-2 * abs(b) + 2e-2, (kind, losses, ref_losses)
        else:
            m = tr._flush_metrics()
            assert m is not None and abs(m["loss"] - sum(ref_losses) / len(ref_losses)) < 0.3, (kind, m, ref_losses)  # mean over the steps
        report[kind] = round(worst, 6)
        tr.shutdown()
        dist.barrier()
    if rank == 0:
        print("STRATEGIES_GPU_OK", report, "reference losses", [round(x, 4) for x in ref_losses])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

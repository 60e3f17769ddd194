"""Where one training step spends its GPU time: busy / idle share and per-kernel totals from the PyTorch profiler (CUPTI).

    python benchmarks/step_breakdown.py [--layers 22] [--config b1_moe]

A measurement aid: kernel times under the profiler carry its overhead, so read SHARES here and take absolute step times
from ``bench.py``.  One GPU, synthetic tokens, the same model / trainer set-up as ``bench.py``.
"""
import argparse
import collections
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200.config import ConfigPresets  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed  # noqa: E402
from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the preset's)")
    ap.add_argument("--config", default="b1_moe")
    ap.add_argument("--top", type=int, default=28)
    a = ap.parse_args()
    rank, _, world = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {"num_layers": a.layers} if a.layers else {}
    cfg = ConfigPresets.get(a.config, num_workers=0, gradient_checkpointing=False, **over)
    mesh = ProcessMesh(world, rank, ep_size=1)
    cfg.world_size, cfg.expert_parallel_size = 1, 1
    torch.manual_seed(1234)
    with torch.device(dev):
        torch.set_default_dtype(torch.bfloat16)
        model = DeepSeekTransformer(cfg.to_model_config(), ep_size=1, ep_rank=0)
        torch.set_default_dtype(torch.float32)
    model.rope.cos, model.rope.sin = model.rope.cos.float(), model.rope.sin.float()
    trainer = EnhancedConversationTrainer(model, None, cfg, mesh=mesh, fused_comm=None)
    trainer._setup_scheduler(10 ** 6)
    mb, L, V = cfg.micro_batch_size, cfg.seq_length, cfg.vocab_size
    g = torch.Generator().manual_seed(99)
    batches = []
    for _ in range(4):
        ids = torch.randint(0, V, (mb, L + 1), generator=g)
        batches.append({"input_ids": ids[:, :-1].contiguous().to(dev), "labels": ids[:, 1:].contiguous().to(dev)})
    accum = max(cfg.gradient_accumulation_steps, 1)

    def step(i):
        for k in range(accum):
            trainer.train_step(batches[(i * accum + k) % 4])
        trainer.optimizer_step()
        trainer._pending_device.clear()

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step(3)
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    t0, t1 = evs[0].time_range.start, max(e.time_range.end for e in evs)
    busy, cur_end, gaps = 0.0, t0, []
    tot, cnt = collections.Counter(), collections.Counter()
    for e in evs:
        s, en = e.time_range.start, e.time_range.end
        name = e.name[:72]
        tot[name] += en - s
        cnt[name] += 1
        if s > cur_end:
            gaps.append(s - cur_end)
            busy += en - s
            cur_end = en
        elif en > cur_end:
            busy += en - cur_end
            cur_end = en
    span = t1 - t0
    gaps.sort()
    print(f"config {a.config} layers {cfg.num_layers} tokens/step {mb * L * accum}: span {span / 1e3:.1f} ms, busy {busy / 1e3:.1f} ms, "
          f"idle {(span - busy) / 1e3:.1f} ms ({100 * (span - busy) / span:.1f} %), {len(evs)} kernels, median gap "
          f"{gaps[len(gaps) // 2] if gaps else 0:.1f} us")
    for name, t in tot.most_common(a.top):
        print(f"{100 * t / span:6.2f} %  {t / 1e3:9.2f} ms  {cnt[name]:6d}  {name}")


if __name__ == "__main__":
    main()

"""Checkpoints across layouts on Gloo ranks: a model trained with expert parallelism 2 + ZeRO-1 is saved (single file and
sharded directory) and resumed by ONE process; both must continue exactly like the two-rank run would."""
import os

import pytest
import torch

from dist_utils import run_dist

from adaptivetrainingsystem_b200.config import ModelConfig
from adaptivetrainingsystem_b200.models import DeepSeekTransformer

CFG = dict(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=96, seq_length=32,
           use_moe=True, num_experts=4, moe_top_k=2, capacity_factor=4.0, tie_word_embeddings=False, routing_noise_std=0.0)


class _Cfg:
    save_optimizer_states = True
    save_total_limit = 0

    def to_dict(self):
        return {}


def _batches():
    g = torch.Generator().manual_seed(5)
    return torch.randint(0, 512, (4, 33), generator=g)


def _ep_save_worker(rank, world, out_dir):
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
    mesh = ProcessMesh(world, rank, ep_size=2)
    torch.manual_seed(0)
    full = DeepSeekTransformer(ModelConfig(**CFG))
    model = DeepSeekTransformer(ModelConfig(**CFG), ep_size=2, ep_rank=rank)
    model.load_state_dict(full.state_dict())
    attach_expert_parallel(model, mesh, None, use_fused=False)
    eng = ShardedEngine(model, lr=1e-2, zero_stage=1, max_grad_norm=1.0, mesh=mesh)
    ids = _batches()
    mine = ids[2 * rank:2 * rank + 2]
    for _ in range(2):
        model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
        eng.step()
    cm = CheckpointManager(_Cfg(), out_dir)
    p1 = cm.save_checkpoint(model, eng, None, 2, 0, suffix="single", mesh=mesh, sharded=False)
    p2 = cm.save_checkpoint(model, eng, None, 2, 0, suffix="shards", mesh=mesh, sharded=True)
    assert (p1 is not None) == (rank == 0) and (p2 is not None) == (rank == 0)
    # one more step: the reference for what a resumed run must reproduce
    model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
    eng.step()
    sd = CheckpointManager._gather_model_state(model, mesh)
    if rank == 0:
        torch.save(sd, os.path.join(out_dir, "after_step3.pt"))
    # same layout, sharded resume: every rank reads only what it owns
    model2 = DeepSeekTransformer(ModelConfig(**CFG), ep_size=2, ep_rank=rank)
    attach_expert_parallel(model2, mesh, None, use_fused=False)
    eng2 = ShardedEngine(model2, lr=1e-2, zero_stage=1, max_grad_norm=1.0, mesh=mesh)
    dist.barrier()
    info = cm.load_checkpoint(os.path.join(out_dir, "checkpoint_shards"), model2, eng2)
    assert info["global_step"] == 2 and eng2.step_count == 2
    model2.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
    eng2.step()
    for (k, a), (_, b) in zip(model.state_dict().items(), model2.state_dict().items()):
        assert torch.allclose(a, b, atol=1e-6), k


@pytest.mark.dist
def test_ep2_checkpoints_resume_on_one_process(tmp_path):
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
    out = str(tmp_path)
    run_dist(_ep_save_worker, 2, (out,))
    assert os.path.isfile(os.path.join(out, "checkpoint_single.pt"))
    shard_dir = os.path.join(out, "checkpoint_shards")
    assert sorted(os.listdir(shard_dir)) == ["index.json", "meta.pt", "model_dense.pt", "model_experts_ep0.pt", "model_experts_ep1.pt",
                                             "optim_rank00000.pt", "optim_rank00001.pt"]
    want = torch.load(os.path.join(out, "after_step3.pt"))
    ids = _batches()
    for which in ("checkpoint_single.pt", "checkpoint_shards"):
        model = DeepSeekTransformer(ModelConfig(**CFG))  # all four experts in one process
        eng = ShardedEngine(model, lr=1e-2, zero_stage=1, max_grad_norm=1.0, grad_accumulation_steps=2)
        cm = CheckpointManager(_Cfg(), out)
        info = cm.load_checkpoint(os.path.join(out, which), model, eng)
        assert info["global_step"] == 2 and eng.step_count == 2, which
        # the moments came back for every parameter, experts included (re-assembled by global expert index)
        for b in eng.buckets:
            assert float(b.exp_avg.abs().sum()) > 0 and float(b.exp_avg_sq.sum()) > 0, (which, b.name)
        # third step on two micro-batches (what the two ranks saw) == third step of the two-rank run
        for half in (ids[:2], ids[2:]):
            model.forward_loss(half[:, :-1], half[:, 1:])["loss"].backward()
        eng.step()
        sd = model.state_dict()
        for k, v in want.items():
            assert torch.allclose(sd[k], v, atol=5e-5, rtol=1e-4), (which, k, (sd[k] - v).abs().max())


def test_history_restores_best_metric(tmp_path):
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**dict(CFG, use_moe=False)))
    eng = ShardedEngine(model, lr=1e-2, zero_stage=0)
    cm = CheckpointManager(_Cfg(), str(tmp_path))
    cm.save_checkpoint(model, eng, None, 1, 0, eval_loss=3.0)
    cm.save_checkpoint(model, eng, None, 2, 0, eval_loss=2.5)
    again = CheckpointManager(_Cfg(), str(tmp_path))
    assert again.best_metric == 2.5
    again.save_checkpoint(model, eng, None, 3, 0, eval_loss=2.8)  # not better: the best link must stay on step 2
    assert os.path.realpath(os.path.join(str(tmp_path), "best_checkpoint.pt")).endswith("step_000002.pt")
    # sharded directories resolve as "latest" and load in one process
    p = again.save_checkpoint(model, eng, None, 4, 0, sharded=True)
    assert os.path.isdir(p) and again.resolve("latest") == p
    m2 = DeepSeekTransformer(ModelConfig(**dict(CFG, use_moe=False)))
    e2 = ShardedEngine(m2, lr=1e-2, zero_stage=0)
    info = again.load_checkpoint("latest", m2, e2)
    assert info["sharded"] and info["global_step"] == 4
    for (k, a), (_, b) in zip(model.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a, b), k

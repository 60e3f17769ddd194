"""Expert placement balancing: the swap search on plain numbers, and on two Gloo ranks (expert parallelism 2, two experts per
rank, ZeRO-1) the exchange of weights + optimiser state + router rows, which must leave the training trajectory unchanged."""
import random

import pytest
import torch

from dist_utils import run_dist

from adaptivetrainingsystem_b200.config import ModelConfig
from adaptivetrainingsystem_b200.models import DeepSeekTransformer
from adaptivetrainingsystem_b200.parallel.load_balance import imbalance, plan_swaps, rank_loads

CFG = dict(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=96, seq_length=32,
           use_moe=True, num_experts=4, moe_top_k=2, capacity_factor=4.0, tie_word_embeddings=False, routing_noise_std=0.0)


def test_swap_search_lowers_the_heaviest_rank():
    random.seed(3)
    for E, el in [(8, 2), (16, 4), (64, 8)]:
        load = [random.random() ** 3 * 1000 for _ in range(E)]
        swaps = plan_swaps(load, el)
        v = list(load)
        for a, b in swaps:
            assert a // el != b // el
            v[a], v[b] = v[b], v[a]
        assert sorted(v) == sorted(load)
        assert max(rank_loads(v, el)) <= max(rank_loads(load, el))
        if E > 8:   # many small experts: the heaviest rank ends close to the mean
            assert swaps and imbalance(v, el) < 1.15 < imbalance(load, el)
    assert plan_swaps([5.0, 1.0, 1.0, 1.0], 1) == []          # one expert per rank: nothing to gain
    assert plan_swaps([1.0, 1.0, 1.0, 1.0], 2) == []          # already even
    assert plan_swaps([10.0, 9.0, 1.0, 1.0], 2) in ([(0, 2)], [(0, 3)], [(1, 2)], [(1, 3)])


def _worker(rank, world, out_dir):
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.parallel.load_balance import ExpertLoadBalancer
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
    mesh = ProcessMesh(world, rank, ep_size=2)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    mine = ids[2 * rank:2 * rank + 2]

    def build():
        torch.manual_seed(0)
        full = DeepSeekTransformer(ModelConfig(**CFG))
        m = DeepSeekTransformer(ModelConfig(**CFG), ep_size=2, ep_rank=rank)
        m.load_state_dict(full.state_dict())
        attach_expert_parallel(m, mesh, None, use_fused=False)
        return m, ShardedEngine(m, lr=1e-2, zero_stage=1, max_grad_norm=1.0, mesh=mesh)

    def train(m, e, n):
        for _ in range(n):
            m.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
            e.step()

    plain, eng_plain = build()
    train(plain, eng_plain, 4)

    model, eng = build()
    train(model, eng, 2)
    bal = ExpertLoadBalancer(model, mesh, eng)
    layers = model.get_moe_layers()
    measured = bal.demand()
    assert all(float(d.sum()) == 2 * 2 * (2 * 32) * 2 for d in measured)     # steps x ranks x tokens per rank x top-k
    # a skew the router did not produce, so that both layers get a known plan: slots 0 and 1 (rank 0) are hot
    for l in layers:
        l.expert_demand.copy_(torch.tensor([10.0, 9.0, 1.0, 1.0], dtype=torch.float64) / world)
    model.eval()
    with torch.no_grad():
        before = model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].item()
    w1_before = [l.experts_w1.detach().clone() for l in layers]
    gate_before = [l.gate.weight.detach().clone() for l in layers]
    report = bal.balance()
    assert report["swaps"] == len(layers)
    for row in report["layers"]:
        assert row["before"] > 1.7 and row["after"] < 1.1 and len(row["swaps"]) == 1
    (a, b), = report["layers"][0]["swaps"]
    # the weights really moved: this rank's row now holds what the peer had, and the router rows traded places
    other = [torch.empty_like(w1_before[0]) for _ in range(world)]
    dist.all_gather(other, w1_before[0])
    mine_slot, peer_slot = (a, b) if rank == 0 else (b, a)
    assert torch.equal(layers[0].experts_w1[mine_slot % 2], other[1 - rank][peer_slot % 2])
    assert torch.equal(layers[0].gate.weight[a], gate_before[0][b]) and torch.equal(layers[0].gate.weight[b], gate_before[0][a])
    with torch.no_grad():
        after = model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].item()
    assert abs(before - after) < 1e-5, (before, after)      # same function, different placement
    model.train()
    train(model, eng, 2)                                       # moments came along: the trajectory continues
    model.eval()
    plain.eval()
    with torch.no_grad():
        l1 = model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].item()
        l2 = plain.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].item()
    assert abs(l1 - l2) < 2e-4, (l1, l2)
    # expert rows of the two runs agree once the exchange is undone
    sd_a = CheckpointManager._gather_model_state(model, mesh)
    sd_b = CheckpointManager._gather_model_state(plain, mesh)
    if rank == 0:
        perm = list(range(4))
        perm[a], perm[b] = perm[b], perm[a]
        for k in sd_a:
            if "layers.0." in k and ("experts_w" in k or "gate.weight" in k):
                assert torch.allclose(sd_a[k][perm], sd_b[k], atol=2e-4), k


@pytest.mark.dist
def test_experts_and_their_optimiser_state_change_ranks(tmp_path):
    run_dist(_worker, 2, (str(tmp_path),))


def _trainer_worker(rank, world, out_dir):
    import os
    from adaptivetrainingsystem_b200.config import Config
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer
    cfg = Config(vocab_size=256, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=96, seq_length=16,
                 use_moe=True, num_experts=4, moe_top_k=2, capacity_factor=4.0, expert_parallel_size=2, precision="fp32",
                 gradient_checkpointing=False, learning_rate=1e-2, batch_size=2, micro_batch_size=2, gradient_accumulation_steps=1,
                 zero_stage=1, output_dir=os.path.join(out_dir, f"r{rank}"), experiment_name="lb", num_workers=0, heartbeat_interval_s=0.0,
                 use_lr_scheduler=False, routing_noise_std=0.0, fused_comm=False, expert_rebalance_interval=1)
    mesh = ProcessMesh.from_config(cfg, world, rank)
    assert mesh.ep_size == 2
    torch.manual_seed(0)
    full = DeepSeekTransformer(cfg.to_model_config())
    model = DeepSeekTransformer(cfg.to_model_config(), ep_size=2, ep_rank=mesh.coord.ep)
    model.load_state_dict(full.state_dict())
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    attach_expert_parallel(model, mesh, cfg, use_fused=False)
    tr = EnhancedConversationTrainer(model, None, cfg, mesh=mesh)
    g = torch.Generator().manual_seed(3 + rank)
    ids = torch.randint(0, 256, (2, 17), generator=g)
    batch = {"input_ids": ids[:, :-1], "labels": ids[:, 1:]}
    tr.train_step(batch)
    tr.optimizer_step()
    for l in model.get_moe_layers():          # a skew with a known remedy
        l.expert_demand.copy_(torch.tensor([12.0, 8.0, 1.0, 1.0], dtype=torch.float64) / world)
    model.eval()
    with torch.no_grad():
        before = float(model.forward_loss(ids[:, :-1], ids[:, 1:])["loss"])
    report = tr.rebalance_experts()
    assert report is not None and report["swaps"] == 2 and all(r["after"] < r["before"] for r in report["layers"])
    with torch.no_grad():
        after = float(model.forward_loss(ids[:, :-1], ids[:, 1:])["loss"])
    assert abs(before - after) < 1e-5
    model.train()
    out = tr.train_step(batch)                # training goes on with the moved experts and their optimiser state
    tr.optimizer_step()
    assert float(out["loss"]) == float(out["loss"])
    tr.shutdown()


@pytest.mark.dist
def test_trainer_rebalances_experts_between_steps(tmp_path):
    run_dist(_trainer_worker, 2, (str(tmp_path),))

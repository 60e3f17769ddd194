"""Multi-rank host logic on CPU (Gloo, world size 2): ZeRO partition bookkeeping, expert-parallel permutation and
exchange, checkpoint gather."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_dist  # noqa: E402

from adaptivetrainingsystem_b200.config import ModelConfig  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402

pytestmark = pytest.mark.dist

CFG = dict(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32,
           use_moe=True, num_experts=4, moe_top_k=2, capacity_factor=8.0, tie_word_embeddings=False)


def _single_process_reference(stage_steps=2):
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    eng = ShardedEngine(model, lr=1e-2, zero_stage=0, max_grad_norm=1.0, grad_accumulation_steps=2)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    for _ in range(stage_steps):
        # two micro-batches of 2 sequences = what two ranks see
        for half in (ids[:2], ids[2:]):
            model.forward_loss(half[:, :-1], half[:, 1:])["loss"].backward()
        eng.step()
    return {k: v.clone() for k, v in model.state_dict().items()}


def _zero_worker(rank, world, stage, ref_path):
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    mesh = ProcessMesh(world, rank)
    eng = ShardedEngine(model, lr=1e-2, zero_stage=stage, max_grad_norm=1.0, mesh=mesh)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    mine = ids[2 * rank:2 * rank + 2]
    for _ in range(2):
        model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
        eng.step()
    ref = torch.load(ref_path)
    sd = model.state_dict()
    for k, v in ref.items():
        assert torch.allclose(sd[k], v, atol=2e-5, rtol=1e-4), (k, (sd[k] - v).abs().max())
    if stage >= 1:
        b = eng.buckets[0]
        assert b.master.numel() == b.shard and b.shard * world == b.padded
    full = eng.state_dict()
    assert set(full["state"]) == {n for n, _ in model.named_parameters()}


@pytest.mark.parametrize("stage", [0, 1, 2])
def test_zero_matches_single_process(stage, tmp_path):
    ref = _single_process_reference()
    path = str(tmp_path / "ref.pt")
    torch.save(ref, path)
    run_dist(_zero_worker, 2, (stage, path))


def _ep_worker(rank, world, ref_path):
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    ref = torch.load(ref_path)
    mesh = ProcessMesh(world, rank, ep_size=2)
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG), ep_size=2, ep_rank=rank)
    model.load_state_dict(ref["init"])  # each rank picks its own experts out of the full checkpoint
    attach_expert_parallel(model, mesh, None, use_fused=False)
    eng = ShardedEngine(model, lr=1e-2, zero_stage=1, max_grad_norm=1.0, mesh=mesh)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    mine = ids[2 * rank:2 * rank + 2]
    for _ in range(2):
        model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
        eng.step()
    sd = model.state_dict()
    for k, v in sd.items():
        assert torch.allclose(v, ref["final"][k], atol=3e-5, rtol=1e-4), (k, (v - ref["final"][k]).abs().max())
    # checkpoint gather: the expert-parallel ranks together produce the full state dict
    from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
    full = CheckpointManager._gather_model_state(model, mesh)
    assert set(full) == set(ref["final"])


def test_expert_parallel_matches_local(tmp_path):
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    init = {k: v.clone() for k, v in model.state_dict().items()}
    final = _single_process_reference()
    path = str(tmp_path / "ref.pt")
    torch.save({"init": init, "final": final}, path)
    run_dist(_ep_worker, 2, (path,))


def _zero3_worker(rank, world, ref_path):
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.zero3 import ZeRO3Engine
    cfg = dict(CFG, use_moe=False)
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**cfg))
    mesh = ProcessMesh(world, rank)
    eng = ZeRO3Engine(model, lr=1e-2, max_grad_norm=1.0, mesh=mesh)
    assert model.layers[0].self_attn.qkv_proj.numel() == 0  # released at rest: only the shard lives on this rank
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    mine = ids[2 * rank:2 * rank + 2]
    for _ in range(2):
        model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
        eng.step()
    assert model.layers[1].ffn.down_proj.numel() == 0
    eng.gather_full_parameters()
    ref = torch.load(ref_path)
    sd = model.state_dict()
    for k, v in ref.items():
        assert torch.allclose(sd[k], v, atol=3e-5, rtol=1e-4), (k, (sd[k] - v).abs().max())
    m = eng.matrices[0]
    assert m.master.numel() * world == m.numel and m.shard.shape == (m.N // world, m.K)  # row shards of every block matrix
    assert eng.root.master.numel() * world == eng.root.padded                           # flat shard of everything else


def test_zero3_matches_single_process(tmp_path):
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    cfg = dict(CFG, use_moe=False)
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**cfg))
    eng = ShardedEngine(model, lr=1e-2, zero_stage=0, max_grad_norm=1.0, grad_accumulation_steps=2)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 33), generator=g)
    for _ in range(2):
        for half in (ids[:2], ids[2:]):
            model.forward_loss(half[:, :-1], half[:, 1:])["loss"].backward()
        eng.step()
    path = str(tmp_path / "ref3.pt")
    torch.save({k: v.clone() for k, v in model.state_dict().items()}, path)
    run_dist(_zero3_worker, 2, (path,))


def _ep_add_prune_worker(rank, world, out_dir):
    """Expert add / prune under expert parallelism: every rank grows / shrinks by one local expert, the replicated gate is
    re-planned identically on all ranks, optimiser state of the surviving experts is kept, and training goes on."""
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.config import Config
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer
    cfg = Config(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32,
                 batch_size=2, micro_batch_size=2, gradient_accumulation_steps=1, num_epochs=1, precision="fp32", use_moe=True,
                 num_experts=4, moe_top_k=2, capacity_factor=8.0, learning_rate=1e-3, output_dir=out_dir, experiment_name=f"r{rank}",
                 log_every_n_steps=1, num_workers=0, gradient_checkpointing=False, zero_stage=1)
    mesh = ProcessMesh(world, rank, ep_size=2)
    cfg.world_size, cfg.expert_parallel_size = world, 2
    torch.manual_seed(0)
    full = DeepSeekTransformer(cfg.to_model_config())
    model = DeepSeekTransformer(cfg.to_model_config(), ep_size=2, ep_rank=rank)
    model.load_state_dict(full.state_dict())
    attach_expert_parallel(model, mesh, cfg, use_fused=False)
    tr = EnhancedConversationTrainer(model, None, cfg, mesh=mesh)
    g = torch.Generator().manual_seed(11 + rank)
    ids = torch.randint(0, 512, (2, 33), generator=g)
    batch = {"input_ids": ids[:, :-1], "labels": ids[:, 1:]}

    def one_step():
        out = tr.train_step(batch)
        tr.optimizer_step()
        assert torch.isfinite(torch.as_tensor(float(out["loss"])))

    one_step()
    layer = model.get_moe_layers()[0]
    w1_before = layer.experts_w1.data.clone()
    st_before = tr.engine.state_dict()["state"]["layers.0.ffn.experts_w1"]["exp_avg"].clone()
    assert tr.add_expert(0) == 1
    assert layer.num_experts == 6 and layer.experts_w1.shape[0] == 3 and layer.gate.weight.shape[0] == 6 and layer.ep.num_experts == 6
    assert torch.equal(layer.experts_w1.data[:2], w1_before)  # surviving local experts untouched
    st_after = tr.engine.state_dict()["state"]["layers.0.ffn.experts_w1"]["exp_avg"]
    assert torch.equal(st_after[:2], st_before) and float(st_after[2].abs().sum()) == 0.0  # moments kept / zero for the new expert
    gate = layer.gate.weight.data.clone()
    ref = gate.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(gate, ref), "gate rows differ across ranks after add_expert"
    one_step()
    one_step()
    # prune the expert with global id 4 (= rank 1, local slot 1): slot 1 goes on every rank
    assert tr.prune_expert(0, 4)
    assert layer.num_experts == 4 and layer.experts_w1.shape[0] == 2 and layer.gate.weight.shape[0] == 4
    gate = layer.gate.weight.data.clone()
    ref = gate.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(gate, ref)
    one_step()
    assert not tr.prune_expert(0, 99)
    # the other layer is untouched
    assert model.get_moe_layers()[1].num_experts == 4


def test_expert_add_prune_under_expert_parallelism(tmp_path):
    run_dist(_ep_add_prune_worker, 2, (str(tmp_path),))


def _ep_eval_worker(rank, world):
    """Without autograd all MoE layers share one set of exchange buffers: the expert-parallel forward still equals the
    single-process forward, for two different batch shapes in a row (buffers re-created on the capacity change)."""
    from adaptivetrainingsystem_b200.inference import GenerationEngine
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
    mesh = ProcessMesh(world, rank, ep_size=2)
    torch.manual_seed(0)
    full = DeepSeekTransformer(ModelConfig(**CFG)).eval()
    model = DeepSeekTransformer(ModelConfig(**CFG), ep_size=2, ep_rank=rank)
    model.load_state_dict(full.state_dict())
    comm = attach_expert_parallel(model, mesh, None, use_fused=False)
    eng = GenerationEngine(model, pack_experts=True)  # packing is a GPU layout: a no-op for CPU weights
    assert not getattr(model.get_moe_layers()[0].experts_w1, "_ats_packed", False)
    g = torch.Generator().manual_seed(3)  # the same batch on every rank, as the serving path runs it
    for shape in ((2, 32), (3, 17)):
        ids = torch.randint(0, 512, shape, generator=g)
        with torch.no_grad():
            ref = full(ids, return_aux_loss=False)
            out = eng.model(ids, return_aux_loss=False)
        assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4), (shape, (out - ref).abs().max())
    ep_comm = model.get_moe_layers()[0].ep.comm
    assert all(k[0] == -1 for k in ep_comm._layers), list(ep_comm._layers)  # one shared set, none per layer


def test_expert_parallel_eval_shares_buffers():
    run_dist(_ep_eval_worker, 2)


def _fsdp_backend_worker(rank, world):
    """The backend factories of the reference's wrapper API reach the stage-3 engine: FULL_SHARD / gemini / zero_stage 3."""
    from adaptivetrainingsystem_b200.backend import create_colossalai_backend, create_deepspeed_backend, create_fsdp_backend
    from adaptivetrainingsystem_b200.config import Config
    from adaptivetrainingsystem_b200.parallel.zero3 import ZeRO3Engine
    cfg = Config(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32, use_moe=False,
                 precision="fp32", gradient_checkpointing=False, zero_stage=3, output_dir="/tmp/ats_backend_test", experiment_name=f"r{rank}")
    full_numel = None
    for make in (lambda m: create_fsdp_backend(m, cfg), lambda m: create_deepspeed_backend(m, cfg), lambda m: create_colossalai_backend(m, cfg, "gemini")):
        torch.manual_seed(0)
        model = DeepSeekTransformer(cfg.to_model_config())
        full_numel = sum(p.numel() for p in model.parameters())
        be = make(model)
        assert isinstance(be.engine, ZeRO3Engine) and be.engine.zero_stage == 3
        block_params = sum(m.numel for m in be.engine.matrices)
        assert sum(m.shard_numel for m in be.engine.matrices) * world == block_params  # this rank holds 1 / world of every block matrix
        assert all(m.param.numel() == 0 for m in be.engine.matrices)                      # nothing is gathered at rest
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, 512, (2, 33), generator=g)
        out = be._model.forward_loss(ids[:, :-1], ids[:, 1:])
        be.backward(out["loss"])
        stats = be.step()
        assert float(stats["grad_norm"]) > 0
    cfg.fsdp_sharding_strategy = "SHARD_GRAD_OP"
    be = create_fsdp_backend(DeepSeekTransformer(cfg.to_model_config()), cfg)
    assert not isinstance(be.engine, ZeRO3Engine) and be.engine.zero_stage == 2
    assert full_numel > 0


def test_backend_factories_build_the_stage3_engine():
    run_dist(_fsdp_backend_worker, 2)

"""Pipeline (1F1B), tensor parallel, vocabulary-parallel loss and head-scatter sequence parallel against single-process
results, on Gloo ranks."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_dist  # noqa: E402

from adaptivetrainingsystem_b200.config import ModelConfig  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402

pytestmark = pytest.mark.dist
CFG = dict(vocab_size=256, hidden_size=64, num_layers=4, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=16,
           tie_word_embeddings=False)


def _pp_worker(rank, world, path):
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.parallel.pipeline import OneFOneBSchedule, PipelineStage, partition_layers
    assert partition_layers(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    ref = torch.load(path)
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    model.load_state_dict(ref["init"])
    stage = PipelineStage(model, rank, world)
    # the stage holds its own two layers only: the others' weights are gone, not just frozen
    foreign = [i for i in range(4) if not (stage.start <= i < stage.end)]
    assert stage.freed > 0 and all(p.numel() == 0 for i in foreign for p in model.layers[i].parameters())
    assert all(p.numel() > 0 for i in range(stage.start, stage.end) for p in model.layers[i].parameters())
    sched = OneFOneBSchedule(stage, dist.group.WORLD, 4, (2, 16, 64), torch.float32, torch.device("cpu"))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (8, 17), generator=g)
    mbs = [{"input_ids": ids[2 * i:2 * i + 2, :-1], "labels": ids[2 * i:2 * i + 2, 1:]} for i in range(4)]
    loss = sched.run(mbs)
    if rank == world - 1:
        assert abs(loss.item() - ref["loss"]) < 1e-4, (loss.item(), ref["loss"])
    for n, p in model.named_parameters():
        if p.requires_grad and p.grad is not None:
            assert torch.allclose(p.grad, ref["grads"][n], atol=1e-5), n


def _pp_interleaved_worker(rank, world, path):
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.parallel.pipeline import InterleavedSchedule, InterleavedStages
    ref = torch.load(path)
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    model.load_state_dict(ref["init"])
    stages = InterleavedStages(model, rank, world, chunks=2)  # 4 layers -> 4 virtual stages, two per rank
    assert stages.virtual == [rank, world + rank]
    sched = InterleavedSchedule(stages, dist.group.WORLD, 4, (2, 16, 64), torch.float32, torch.device("cpu"))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (8, 17), generator=g)
    mbs = [{"input_ids": ids[2 * i:2 * i + 2, :-1], "labels": ids[2 * i:2 * i + 2, 1:]} for i in range(4)]
    from adaptivetrainingsystem_b200.parallel.pipeline import interleaved_order
    order = interleaved_order(rank, world, 2, 4)
    assert len(order) == 16 and [o[0] for o in order[:2 * (world - rank - 1) + world]] == ["F"] * (2 * (world - rank - 1) + world)
    assert sorted(o for o in order if o[0] == "F") == sorted(("F", c, i) for c in range(2) for i in range(4))
    loss = sched.run(mbs)
    assert sched.max_alive < 8  # 1F1B: fewer activations alive than chunks x micro-batches (a breadth-first order would keep all 8)
    if rank == world - 1:
        assert abs(loss.item() - ref["loss"]) < 1e-4, (loss.item(), ref["loss"])
    checked = 0
    for n, p in model.named_parameters():
        if p.requires_grad and p.grad is not None:
            assert torch.allclose(p.grad, ref["grads"][n], atol=1e-5), n
            checked += 1
    assert checked > 0


def test_pipeline_1f1b_matches_single_process(tmp_path):
    torch.manual_seed(0)
    model = DeepSeekTransformer(ModelConfig(**CFG))
    init = {k: v.clone() for k, v in model.state_dict().items()}
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (8, 17), generator=g)
    total = 0.0
    for i in range(4):
        out = model.forward_loss(ids[2 * i:2 * i + 2, :-1], ids[2 * i:2 * i + 2, 1:])
        (out["loss"] / 4).backward()
        total += out["loss"].item() / 4
    path = str(tmp_path / "ref.pt")
    torch.save({"init": init, "loss": total, "grads": {n: p.grad.clone() for n, p in model.named_parameters()}}, path)
    run_dist(_pp_worker, 2, (path,))
    run_dist(_pp_interleaved_worker, 2, (path,))


def _tp_worker(rank, world):
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.parallel.sequence_parallel import ulysses_attention
    from adaptivetrainingsystem_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding,
                                                                      vocab_parallel_cross_entropy)
    from adaptivetrainingsystem_b200 import ops
    torch.manual_seed(0)
    w1, w2 = torch.randn(32, 16) * 0.1, torch.randn(16, 32) * 0.1
    x = torch.randn(2, 8, 16)
    for sp in (False, True):
        xin = (x.chunk(world, dim=1)[rank] if sp else x).clone().requires_grad_()
        col = ColumnParallelLinear.from_full(w1, None, sequence_parallel=sp)
        row = RowParallelLinear.from_full(w2, None, sequence_parallel=sp)
        y = row(torch.relu(col(xin)))
        y.sum().backward()
        xr = x.clone().requires_grad_()
        w1r = w1.clone().requires_grad_()
        yr = torch.relu(xr @ w1r.t()) @ w2.t()
        yr.sum().backward()
        y_ref = yr.chunk(world, dim=1)[rank] if sp else yr
        g_ref = xr.grad.chunk(world, dim=1)[rank] if sp else xr.grad
        assert torch.allclose(y, y_ref, atol=1e-5) and torch.allclose(xin.grad, g_ref, atol=1e-5), sp
        assert torch.allclose(col.weight.grad, w1r.grad.chunk(world, 0)[rank], atol=1e-5), sp
    # vocabulary-parallel embedding and loss
    table = torch.randn(20, 8)
    emb = VocabParallelEmbedding(20, 8)
    emb.weight.data.copy_(table.chunk(world, 0)[rank])
    ids = torch.randint(0, 20, (3, 5))
    assert torch.allclose(emb(ids), table[ids], atol=1e-6)
    logits = torch.randn(15, 20)
    labels = torch.randint(0, 20, (15,))
    labels[0] = -100
    ll = logits.chunk(world, -1)[rank].clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(ll, labels)
    loss.backward()
    lr = logits.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, labels, ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-5 and torch.allclose(ll.grad, lr.grad.chunk(world, -1)[rank], atol=1e-6)
    # head-scatter sequence parallel attention
    q, k, v = torch.randn(1, 8, 4, 8), torch.randn(1, 8, 2, 8), torch.randn(1, 8, 2, 8)
    o_ref = ops.attention_reference(q, k, v)
    o = ulysses_attention(*(t.chunk(world, dim=1)[rank].contiguous() for t in (q, k, v)))
    assert torch.allclose(o, o_ref.chunk(world, dim=1)[rank], atol=1e-5)


def test_tensor_sequence_vocab_parallel():
    run_dist(_tp_worker, 2)


def _ring_worker(rank, world):
    import torch
    import torch.distributed as dist
    from adaptivetrainingsystem_b200 import ops
    from adaptivetrainingsystem_b200.parallel.ring import linear_ring_reducescatter, ring_allgather_linear, ring_attention
    torch.manual_seed(0)
    L, K, N = 8 * world, 12, 10
    x_full = torch.randn(L, K, dtype=torch.float64)
    w_full = torch.randn(N * world, K, dtype=torch.float64)
    Lc = L // world
    # column-parallel linear behind a ring all-gather of the sequence shards
    x = x_full[rank * Lc:(rank + 1) * Lc].clone().requires_grad_()
    w = w_full[rank * N:(rank + 1) * N].clone().requires_grad_()
    y = ring_allgather_linear(x, w)
    xr = x_full.clone().requires_grad_()
    wr = w_full.clone().requires_grad_()
    yr = xr @ wr.t()
    assert torch.allclose(y, yr[:, rank * N:(rank + 1) * N].detach())
    gy = torch.randn(L, N * world, dtype=torch.float64)
    y.backward(gy[:, rank * N:(rank + 1) * N])
    yr.backward(gy)
    assert torch.allclose(w.grad, wr.grad[rank * N:(rank + 1) * N])
    assert torch.allclose(x.grad, xr.grad[rank * Lc:(rank + 1) * Lc])
    # row-parallel linear followed by a ring reduce-scatter back to sequence shards
    Kl = K // world if K % world == 0 else K
    x2_full = torch.randn(L, Kl * world, dtype=torch.float64)
    w2_full = torch.randn(N, Kl * world, dtype=torch.float64)
    x2 = x2_full[:, rank * Kl:(rank + 1) * Kl].clone().requires_grad_()
    w2 = w2_full[:, rank * Kl:(rank + 1) * Kl].clone().requires_grad_()
    y2 = linear_ring_reducescatter(x2, w2)
    ref2 = (x2_full @ w2_full.t())
    assert torch.allclose(y2, ref2[rank * Lc:(rank + 1) * Lc])
    g2 = torch.randn(L, N, dtype=torch.float64)
    y2.backward(g2[rank * Lc:(rank + 1) * Lc])
    assert torch.allclose(x2.grad, (g2 @ w2_full)[:, rank * Kl:(rank + 1) * Kl])
    assert torch.allclose(w2.grad, (g2.t() @ x2_full)[:, rank * Kl:(rank + 1) * Kl])
    # ring attention against full causal attention
    B, Hq, Hkv, D = 2, 4, 2, 8
    q_full = torch.randn(B, L, Hq, D)
    k_full = torch.randn(B, L, Hkv, D)
    v_full = torch.randn(B, L, Hkv, D)
    sl = slice(rank * Lc, (rank + 1) * Lc)
    q, k, v = (t[:, sl].clone().requires_grad_() for t in (q_full, k_full, v_full))
    o = ring_attention(q, k, v)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q_full, k_full, v_full))
    o_ref = ops.attention_reference(qr, kr, vr)
    assert torch.allclose(o, o_ref[:, sl].detach(), atol=1e-5)
    go = torch.randn(B, L, Hq, D)
    o.backward(go[:, sl])
    o_ref.backward(go)
    assert torch.allclose(q.grad, qr.grad[:, sl], atol=1e-4)
    assert torch.allclose(k.grad, kr.grad[:, sl], atol=1e-4)
    assert torch.allclose(v.grad, vr.grad[:, sl], atol=1e-4)


def test_ring_sequence_parallel_and_ring_attention():
    from dist_utils import run_dist
    run_dist(_ring_worker, world=2)
    run_dist(_ring_worker, world=3)


def _pp_generate_worker(rank, world, path):
    from adaptivetrainingsystem_b200.config import ModelConfig
    from adaptivetrainingsystem_b200.inference import PipelineGenerator, SamplingParams
    from adaptivetrainingsystem_b200.models import DeepSeekTransformer
    from adaptivetrainingsystem_b200.parallel.pipeline import PipelineStage
    ref = torch.load(path)
    cfg = ModelConfig(**ref["cfg"])
    model = DeepSeekTransformer(cfg)
    model.load_state_dict(ref["state"])
    model.eval()
    stage = PipelineStage(model, rank, world)
    assert stage.freed > 0
    gen = PipelineGenerator(stage)
    for mb in (1, 2, 4):
        out = gen.generate(ref["prompts"], SamplingParams.from_mode("greedy", max_new_tokens=6), micro_batches=mb)
        assert torch.equal(out.cpu(), ref["tokens"]), (mb, out.tolist(), ref["tokens"].tolist())


@pytest.mark.dist
@pytest.mark.parametrize("moe", [False, True])
def test_pipeline_generation_matches_one_process(moe, tmp_path):
    """Generation across two pipeline stages (each with the cache of its own layers, 1 / 2 / 4 micro-batches in flight) gives the
    tokens of the single-process cached generator."""
    from adaptivetrainingsystem_b200.config import ModelConfig
    from adaptivetrainingsystem_b200.inference import GenerationEngine, SamplingParams
    from adaptivetrainingsystem_b200.models import DeepSeekTransformer
    cfgd = dict(vocab_size=128, hidden_size=32, num_layers=4, num_heads=4, num_kv_heads=2, intermediate_size=64, seq_length=32,
                use_moe=moe, num_experts=4, moe_top_k=2, capacity_factor=8.0, routing_noise_std=0.0, tie_word_embeddings=False)
    torch.manual_seed(1)
    model = DeepSeekTransformer(ModelConfig(**cfgd)).eval()
    prompts = torch.randint(0, 128, (4, 7))
    tokens = GenerationEngine(model).generate(prompts, SamplingParams.from_mode("greedy", max_new_tokens=6), use_graph=False)["tokens"]
    path = str(tmp_path / "ref.pt")
    torch.save({"cfg": cfgd, "state": model.state_dict(), "prompts": prompts, "tokens": tokens}, path)
    run_dist(_pp_generate_worker, 2, (path,))

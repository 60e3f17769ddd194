"""Update rules (CPU bodies), host AdamW library, data-index and checkpoint-planner helpers."""
import os
import ctypes

import numpy as np
import pytest
import torch

from adaptivetrainingsystem_b200 import optim
from adaptivetrainingsystem_b200.ops import _lib


def _hyper(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, step=1.0):
    return torch.tensor([lr, b1, b2, eps, wd, step])


def test_sgd_rule_matches_torch():
    torch.manual_seed(0)
    w = torch.randn(1000)
    ref = w.clone().requires_grad_()
    opt = torch.optim.SGD([ref], lr=1e-2, momentum=0.9, weight_decay=0.1, nesterov=True)
    rule = optim.SGDRule(momentum=0.9, nesterov=True)
    master = w.clone()
    st = rule.init_state(master)
    out = torch.zeros(1000)
    for step in range(1, 4):
        g = torch.randn(1000)
        ref.grad = g.clone()
        opt.step()
        rule.update(st, master, g, out, _hyper(step=float(step)), None, True)
        assert torch.allclose(master, ref.detach(), atol=1e-6)
    assert torch.allclose(out, master)


def test_lamb_rule_trust_ratio_and_segments():
    torch.manual_seed(1)
    master = torch.randn(96)
    segs = [(0, 64, 0), (64, 32, 1)]
    rule = optim.LAMBRule()
    st = rule.init_state(master)
    out = torch.zeros(96)
    g = torch.randn(96)
    before = master.clone()
    rule.update(st, master, g, out, _hyper(step=1.0), None, True, segments=segs)
    # per segment: the step has norm lr * |w| (trust ratio rescales the direction to the weight norm)
    for s, n, _ in segs:
        d = (before[s:s + n] - master[s:s + n]).norm().item()
        assert d == pytest.approx(1e-2 * before[s:s + n].norm().item(), rel=1e-4)
    # skip flag leaves everything untouched
    frozen = master.clone()
    rule.update(st, master, g, out, _hyper(step=2.0), torch.tensor([1.0, 0.0, 1.0, 0.0]), True, segments=segs)
    assert torch.equal(master, frozen)


def test_lars_rule_scales_every_tensor_by_its_own_trust_ratio():
    torch.manual_seed(3)
    master = torch.randn(96)
    segs = [(0, 64, 0), (64, 32, 1)]
    rule = optim.LARSRule(momentum=0.9, trust_coefficient=0.5)
    st = rule.init_state(master)
    out = torch.zeros(96)
    g = torch.randn(96) * torch.cat([torch.full((64,), 10.0), torch.full((32,), 0.1)])     # very different gradient scales
    before = master.clone()
    h = _hyper(step=1.0)
    lr, wd = float(h[0]), float(h[4])
    rule.update(st, master, g, out, h, None, True, segments=segs)
    for s, n, _ in segs:
        w, gg = before[s:s + n], g[s:s + n]
        ratio = 0.5 * w.norm() / (gg.norm() + wd * w.norm() + 1e-8)
        assert torch.allclose(before[s:s + n] - master[s:s + n], lr * ratio * (gg + wd * w), atol=1e-6)
    assert torch.allclose(out, master)
    # second step: the momentum buffer carries 0.9 of the first
    first = (before - master).clone()
    mid = master.clone()
    rule.update(st, master, torch.zeros(96), out, h, None, False, segments=segs)
    assert torch.allclose(mid - master, 0.9 * first, atol=1e-6)
    frozen = master.clone()
    rule.update(st, master, g, out, h, torch.tensor([1.0, 0.0, 1.0, 0.0]), True, segments=segs)
    assert torch.equal(master, frozen)


def test_host_adamw_matches_torch_all_isa_levels():
    lib = _lib.host_lib()
    if lib is None:
        pytest.skip("host library not built")
    torch.manual_seed(2)
    n = 70001  # odd: exercises the vector tails
    w0 = torch.randn(n)
    for level in range(0, optim.HostAdamWRule.isa() + 1):
        ref = w0.clone().requires_grad_()
        topt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        rule = optim.HostAdamWRule(pin=False)
        master = w0.clone()
        st = rule.init_state(master)
        out = torch.zeros(n, dtype=torch.bfloat16)
        for step in range(1, 4):
            g = torch.randn(n).bfloat16()
            ref.grad = g.float()
            topt.step()
            rule.update(st, master, g, out, _hyper(step=float(step)), torch.tensor([1.0, 0.0, 0.0, 0.0]), True, force_isa=level)
        assert torch.allclose(st["master_host"], ref.detach(), atol=2e-6), level
        assert torch.equal(out, st["master_host"].bfloat16()), level


def test_engine_with_lamb_and_sgd_trains():
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models.transformer import DeepSeekTransformer
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    for name in ("lamb", "sgd", "adamw_host", "lars"):
        torch.manual_seed(0)
        cfg = ConfigPresets.tiny_cpu()
        model = DeepSeekTransformer(cfg.to_model_config())
        kw = dict(optimizer_kwargs=dict(trust_coefficient=0.02)) if name == "lars" else {}
        eng = ShardedEngine(model, lr={"sgd": 5e-2, "lars": 1.0}.get(name, 5e-3), optimizer=name, **kw)
        ids = torch.randint(0, cfg.vocab_size, (2, 17))
        losses = []
        for _ in range(6):
            loss = model.forward_loss(ids[:, :-1], ids[:, 1:])["loss"]
            loss.backward()
            eng.step()
            losses.append(float(loss))
        assert losses[-1] < losses[0], (name, losses)


def test_data_index_helpers():
    lib = _lib.host_lib()
    if lib is None:
        pytest.skip("host library not built")
    lens = np.array([5, 3, 10, 2, 7], dtype=np.int32)
    lib.ats_build_sample_index.restype = ctypes.c_longlong
    n = lib.ats_build_sample_index(lens.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(5), 4, None, None, ctypes.c_longlong(0))
    assert n == (27 - 1) // 4
    doc = np.zeros(n, dtype=np.int64)
    off = np.zeros(n, dtype=np.int32)
    lib.ats_build_sample_index(lens.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(5), 4, doc.ctypes.data_as(ctypes.c_void_p),
                               off.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(n))
    starts = np.concatenate([[0], np.cumsum(lens)])
    flat = starts[doc] + off
    assert flat.tolist() == [4 * i for i in range(n)]
    idx = np.zeros(1000, dtype=np.int64)
    lib.ats_shuffle_index(idx.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(1000), ctypes.c_ulonglong(7))
    idx2 = np.zeros(1000, dtype=np.int64)
    lib.ats_shuffle_index(idx2.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(1000), ctypes.c_ulonglong(7))
    assert sorted(idx.tolist()) == list(range(1000)) and idx.tolist() != list(range(1000)) and (idx == idx2).all()
    toks = np.arange(12, dtype=np.int64)
    offs = np.array([0, 3, 3, 12], dtype=np.int64)
    out = np.zeros((3, 5), dtype=np.int64)
    mask = np.zeros((3, 5), dtype=np.uint8)
    lib.ats_pack_rows(toks.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(3), 5,
                      ctypes.c_int64(-1), out.ctypes.data_as(ctypes.c_void_p), mask.ctypes.data_as(ctypes.c_void_p))
    assert out.tolist() == [[0, 1, 2, -1, -1], [-1] * 5, [3, 4, 5, 6, 7]]
    assert mask.sum(1).tolist() == [3, 0, 5]
    which = np.zeros(100, dtype=np.int32)
    within = np.zeros(100, dtype=np.int64)
    wts = np.array([3.0, 1.0])
    lib.ats_blend_index(wts.ctypes.data_as(ctypes.c_void_p), 2, ctypes.c_longlong(100), which.ctypes.data_as(ctypes.c_void_p),
                        within.ctypes.data_as(ctypes.c_void_p))
    assert (which == 0).sum() == 75 and within[which == 1].tolist() == list(range(25))


def test_checkpoint_planner():
    lib = _lib.host_lib()
    if lib is None:
        pytest.skip("host library not built")
    lib.ats_ckpt_plan.restype = ctypes.c_double
    n = 8
    act = np.full(n, 10.0)
    inp = np.full(n, 1.0)
    cost = np.arange(1, n + 1, dtype=np.float64)  # cheaper blocks first
    flags = np.zeros(n, dtype=np.uint8)

    def plan(budget):
        r = lib.ats_ckpt_plan(n, act.ctypes.data_as(ctypes.c_void_p), inp.ctypes.data_as(ctypes.c_void_p), cost.ctypes.data_as(ctypes.c_void_p),
                              ctypes.c_double(budget), 256, flags.ctypes.data_as(ctypes.c_void_p))
        return r, flags.copy()
    r, f = plan(100.0)
    assert r == 0.0 and f.sum() == 0
    r, f = plan(60.0)  # stored s blocks, k = 8 - s checkpointed: 10 s + k + 10 <= 60 -> k >= 4 (cheapest four: cost 10)
    assert f.sum() == 4 and r == pytest.approx(10.0) and f[:4].all()
    mem = (act * (1 - f)).sum() + (inp * f).sum() + act[f.astype(bool)].max()
    assert mem <= 60.0
    r, f = plan(5.0)
    assert r == -1.0


def _lamb_sharded_worker(rank, world):
    """ZeRO-sharded LAMB: per-tensor trust ratios are completed across the shards, so two ranks with sharded state move the
    parameters exactly like one process with the summed gradient."""
    import torch.distributed as dist
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models.transformer import DeepSeekTransformer
    from adaptivetrainingsystem_b200.parallel.bootstrap import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    torch.manual_seed(0)
    cfg = ConfigPresets.tiny_cpu()
    mesh = ProcessMesh(world, rank)
    model = DeepSeekTransformer(cfg.to_model_config())
    eng = ShardedEngine(model, lr=1e-2, optimizer="lamb", zero_stage=1, mesh=mesh, max_grad_norm=0.0)
    ref_model = DeepSeekTransformer(cfg.to_model_config())
    ref_model.load_state_dict(model.state_dict())
    ref = ShardedEngine(ref_model, lr=1e-2, optimizer="lamb", zero_stage=0, mesh=ProcessMesh(1, 0, create_groups=False), max_grad_norm=0.0)
    g = torch.Generator().manual_seed(5)
    ids_all = torch.randint(0, cfg.vocab_size, (2 * world, 17), generator=g)
    for _ in range(2):
        mine = ids_all[2 * rank:2 * rank + 2]
        model.forward_loss(mine[:, :-1], mine[:, 1:])["loss"].backward()
        eng.step()
        # reference: the mean over both ranks' batches in one process
        for r in range(world):
            b = ids_all[2 * r:2 * r + 2]
            (ref_model.forward_loss(b[:, :-1], b[:, 1:])["loss"] / world).backward()
        ref.step()
    for (n, p), (_, q) in zip(model.named_parameters(), ref_model.named_parameters()):
        assert torch.allclose(p, q, atol=2e-5, rtol=1e-4), (n, (p - q).abs().max().item())


def test_lamb_sharded_over_two_gloo_ranks():
    from dist_utils import run_dist
    run_dist(_lamb_sharded_worker, world=2)


def test_host_adamw_with_file_backed_state(tmp_path):
    """Optimiser state in memory-mapped files (the nvme_offload_optimizer / nvme_path flags): same numbers as the in-memory
    rule, state files on disk, and a trainer built from the flags uses them."""
    torch.manual_seed(3)
    n = 4099
    w0 = torch.randn(n)
    a, b = optim.HostAdamWRule(pin=False), optim.HostAdamWRule(pin=False, spill_dir=str(tmp_path / "spill"))
    ma, mb = w0.clone(), w0.clone()
    sa, sb = a.init_state(ma), b.init_state(mb)
    oa, ob = torch.zeros(n, dtype=torch.bfloat16), torch.zeros(n, dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n).bfloat16()
        a.update(sa, ma, g, oa, _hyper(step=float(step)), torch.tensor([1.0, 0.0, 0.0, 0.0]), True)
        b.update(sb, mb, g, ob, _hyper(step=float(step)), torch.tensor([1.0, 0.0, 0.0, 0.0]), True)
    assert torch.equal(sa["master_host"], sb["master_host"]) and torch.equal(oa, ob)
    files = sorted(os.listdir(tmp_path / "spill"))
    assert len(files) == 3 and all(os.path.getsize(tmp_path / "spill" / f) >= 4 * n for f in files)
    # through the trainer's configuration flags
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models.transformer import DeepSeekTransformer
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer
    cfg = ConfigPresets.tiny_cpu()
    cfg.nvme_offload_optimizer, cfg.nvme_path, cfg.output_dir = True, str(tmp_path / "nvme"), str(tmp_path / "out")
    torch.manual_seed(0)
    model = DeepSeekTransformer(cfg.to_model_config())
    tr = EnhancedConversationTrainer(model, None, cfg)
    assert tr.engine.optimizer_name == "adamw_host" and tr.engine.rule.spill_dir.startswith(str(tmp_path / "nvme"))
    ids = torch.randint(0, cfg.vocab_size, (2, 17))
    first = None
    for _ in range(4):
        out = tr.train_step({"input_ids": ids[:, :-1], "labels": ids[:, 1:]})
        tr.optimizer_step()
        first = first if first is not None else float(out["loss"])
    assert float(out["loss"]) < first
    assert os.listdir(tmp_path / "nvme" / "ats_optimizer_state")

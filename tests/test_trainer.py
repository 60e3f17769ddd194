"""Trainer API on CPU: loss dictionary, steps, interventions, checkpoints, rollback, OOM recovery."""
import math
import os
import time

import pytest
import torch

from adaptivetrainingsystem_b200.config import Config
from adaptivetrainingsystem_b200.data import SyntheticTokenDataset
from adaptivetrainingsystem_b200.models import DeepSeekTransformer
from adaptivetrainingsystem_b200.training import CheckpointError, CheckpointManager, EnhancedConversationTrainer


def make(tmp_dir, **kw):
    base = dict(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32,
                batch_size=4, micro_batch_size=4, gradient_accumulation_steps=1, num_epochs=1, precision="fp32", use_moe=True,
                num_experts=4, moe_top_k=2, capacity_factor=2.0, learning_rate=1e-3, output_dir=tmp_dir, experiment_name="t",
                log_every_n_steps=1, num_workers=0, gradient_checkpointing=False, save_total_limit=3)
    base.update(kw)
    cfg = Config(**base)
    torch.manual_seed(0)
    model = DeepSeekTransformer(cfg.to_model_config())
    return EnhancedConversationTrainer(model, None, cfg), cfg


def test_compute_loss_contract(tmp_dir):
    tr, cfg = make(tmp_dir)
    logits = torch.randn(2, 8, 512, requires_grad=True)
    labels = torch.randint(0, 512, (2, 8))
    d = tr.compute_loss(logits, labels)
    assert set(d) >= {"loss", "raw_loss", "perplexity", "valid_tokens", "accuracy"}
    assert d["loss"].requires_grad and not d["raw_loss"].requires_grad
    assert d["perplexity"].item() == pytest.approx(math.exp(min(d["raw_loss"].item(), 15.0)), rel=1e-5)
    w = torch.ones(2, 8)
    w[:, :4] = 3.0
    dw = tr.compute_loss(logits, labels, w)
    assert dw["raw_loss"].item() == pytest.approx(d["raw_loss"].item(), rel=1e-6)  # weighting leaves raw_loss unchanged
    big = tr.compute_loss(logits * 100, labels)
    assert torch.isfinite(big["loss"])
    allpad = tr.compute_loss(logits, torch.full((2, 8), -100))
    assert allpad["loss"].item() == 0.0 and math.isinf(allpad["perplexity"].item())
    assert int(allpad["valid_tokens"]) == 0


def test_train_step_and_optimizer_step_change_parameters(tmp_dir):
    tr, cfg = make(tmp_dir)
    ds = SyntheticTokenDataset(512, 32, 8, seed=1)
    batch = next(iter(tr._make_loader(ds, False)))
    before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    out = tr.train_step(batch)
    assert torch.isfinite(out["loss"])
    stats = tr.optimizer_step()
    assert float(stats["grad_norm"]) > 0 and tr.global_step == 1
    changed = [n for n, p in tr.model.named_parameters() if not torch.equal(p, before[n])]
    assert len(changed) == len(before)
    m = tr.get_current_metrics()
    assert m.step == 1 and m.loss > 0 and m.grad_norm > 0 and m.learning_rate > 0


def test_lr_interventions_and_scheduler_override(tmp_dir):
    tr, cfg = make(tmp_dir)
    tr._setup_scheduler(100)
    lr0 = tr.engine.get_lr()
    tr.adjust_learning_rate(5e-4, grace_period=2)
    assert tr.adaptive_lr_override and tr.engine.get_lr() == pytest.approx(5e-4)
    ds = SyntheticTokenDataset(512, 32, 16, seed=1)
    it = iter(tr._make_loader(ds, False))
    for _ in range(2):
        tr.train_step(next(it))
        tr.optimizer_step()
    assert not tr.adaptive_lr_override  # grace period over, scheduler resumes
    new = tr.emergency_lr_reduction(10.0)
    assert tr.engine.get_lr() == pytest.approx(new) and cfg.learning_rate == pytest.approx(5e-5)
    tr.adjust_weight_decay(0.05)
    assert tr.engine._hyper_host[4] == pytest.approx(0.05)
    tr.adjust_batch_size(2)
    assert cfg.micro_batch_size == 2 and cfg.gradient_accumulation_steps == 2


def test_moe_and_mod_interventions(tmp_dir):
    tr, cfg = make(tmp_dir, use_mod=True, moe_pattern="odd")
    tr.adjust_capacity_factor(1.5)
    tr.adjust_routing_temperature(0.7)
    tr.enable_expert_dropout(0.1)
    layer = tr.model.get_moe_layers()[0]
    assert layer.capacity_factor == 1.5 and layer.routing_temperature == 0.7 and layer.expert_dropout == 0.1
    tr.adjust_mod_capacity(0.3)
    assert tr.model.get_mod_layers()[0].router.capacity_factor == 0.3
    ds = SyntheticTokenDataset(512, 32, 8, seed=1)
    batch = next(iter(tr._make_loader(ds, False)))
    tr.train_step(batch)
    tr.optimizer_step()
    n_before = tr.model.num_parameters()
    assert tr.add_expert() == 1 and layer.num_experts == 5 and tr.model.num_parameters() > n_before
    tr.train_step(batch)
    tr.optimizer_step()  # the optimiser follows the new parameter set
    assert tr.prune_expert(layer.layer_idx, 1) and layer.num_experts == 4
    tr.train_step(batch)
    tr.optimizer_step()
    st = tr.get_expert_statistics()
    assert st["max_imbalance"] >= 1.0 and "layers" in st
    ms = tr.get_mod_statistics()
    assert 0 < ms["avg_selected_ratio"] <= 1 and ms["total_compute_savings"] >= 0


def test_train_checkpoint_resume_and_rollback(tmp_dir):
    tr, cfg = make(tmp_dir, num_epochs=2)
    ds = SyntheticTokenDataset(512, 32, 16, seed=1)
    summary = tr.train(ds, ds)
    assert tr.global_step == 8 and len(summary["epochs"]) == 2 and "eval_loss" in summary["epochs"][0]
    assert len(tr.metrics["train_losses"]) == 8 and len(tr.checkpoint_history) == 2
    files = os.listdir(tr.checkpoint_manager.directory)
    assert "checkpoint_final.pt" in files and "checkpoint_history.json" in files
    ck = torch.load(os.path.join(tr.checkpoint_manager.directory, "checkpoint_final.pt"), weights_only=False)
    assert {"model_state_dict", "optimizer_state_dict", "scheduler_state_dict", "global_step", "epoch", "config", "model_config",
            "rng_state", "precision_info", "quantization_info"} <= set(ck)
    assert ck["quantization_info"]["is_quantized"] is False and ck["precision_info"]["name"] == cfg.precision
    assert "layers.0.self_attn.q_proj.weight" in ck["model_state_dict"]
    # resume into a fresh trainer: same parameters and optimiser state
    tr2, _ = make(tmp_dir, num_epochs=2)
    info = tr2.load_checkpoint("latest")
    assert info["global_step"] == 8
    for (n, a), (_, b) in zip(tr.model.named_parameters(), tr2.model.named_parameters()):
        assert torch.equal(a, b), n
    assert torch.allclose(tr.engine.buckets[0].exp_avg, tr2.engine.buckets[0].exp_avg)
    # rollback goes to the checkpoint nearest to step - n
    assert tr.rollback_steps(4) and tr.global_step == 4 and len(tr.metrics["train_losses"]) == 4


def test_wall_clock_backup_and_retry_cap_from_config(tmp_dir):
    """``backup_every_n_hours``: a rolling backup checkpoint once the period has passed; ``max_retries`` caps the OOM retries."""
    tr, cfg = make(tmp_dir, num_epochs=1)
    cfg.backup_every_n_hours = 1
    tr._last_backup -= 2 * 3600.0                       # as if two hours had passed
    ds = SyntheticTokenDataset(512, 32, 8, seed=1)
    tr.train(ds)
    files = os.listdir(tr.checkpoint_manager.directory)
    assert "checkpoint_backup.pt" in files and time.time() - tr._last_backup < 60
    cfg.max_retries = 2
    calls = []

    def boom(*a, **k):
        calls.append(1)
        raise RuntimeError("CUDA out of memory (synthetic)")
    tr.train = boom
    with pytest.raises(RuntimeError):
        tr.train_with_oom_fallback(ds)
    assert len(calls) == 3                              # the first attempt and max_retries retries


def test_profiling_flags_collect_phases_memory_and_collectives(tmp_dir):
    """``enable_profiling`` / ``profile_memory`` / ``profile_communication`` / ``log_throughput`` each change what a run reports."""
    tr, cfg = make(tmp_dir, num_epochs=1, enable_profiling=True, profile_memory=True, profile_communication=True, log_throughput=False)
    summary = tr.train(SyntheticTokenDataset(512, 32, 8, seed=1))
    prof = summary["profiling"]
    assert {"to_device_ms", "forward_ms", "backward_ms", "optimizer_ms"} <= set(prof["phase_ms"]) and prof["phase_ms"]["forward_ms"] > 0
    assert len(prof["peak_memory_gb_per_epoch"]) == 1 and prof["peak_memory_gb_per_epoch"][0] > 0
    assert prof["communication_ms"] == {}                 # one rank: no collective ran
    tr2, _ = make(tmp_dir, num_epochs=1)
    assert tr2.phase_timer is None and tr2.engine.comm_timer is None and tr2.profiling_summary() == {}


def test_checkpoint_manager_errors_and_retention(tmp_dir):
    tr, cfg = make(tmp_dir)
    cm = CheckpointManager(cfg, os.path.join(tmp_dir, "ck"))
    for s in range(5):
        cm.save_checkpoint(tr.model, tr.engine, None, s, 0, eval_loss=5.0 - s)
    kept = [f for f in os.listdir(cm.directory) if f.startswith("checkpoint_epoch")]
    assert len(kept) == 3 and os.path.lexists(os.path.join(cm.directory, "best_checkpoint.pt"))
    bad = os.path.join(tmp_dir, "corrupt.pt")
    with open(bad, "wb") as f:
        f.write(b"not a checkpoint")
    with pytest.raises(CheckpointError):
        cm.load_checkpoint(bad, tr.model)
    other, _ = make(tmp_dir, hidden_size=128)
    with pytest.raises(CheckpointError):
        cm.load_checkpoint("latest", other.model)
    assert cm.create_backup("latest") and cm.emergency_save(tr.model, tr.engine, 9, 0)


def test_oom_fallback_halves_batch(tmp_dir):
    tr, cfg = make(tmp_dir)
    ds = SyntheticTokenDataset(512, 32, 16, seed=1)
    tr.inject_oom(at_micro_step=1)  # host-side injection: no device is driven out of memory
    tr.train_with_oom_fallback(ds)
    assert cfg.micro_batch_size == 2 and cfg.gradient_accumulation_steps == 2
    assert os.path.exists(os.path.join(tr.checkpoint_manager.directory, "optimal_batch_config.json"))


def test_nan_gradients_skip_the_step(tmp_dir):
    tr, cfg = make(tmp_dir)
    ds = SyntheticTokenDataset(512, 32, 8, seed=1)
    batch = next(iter(tr._make_loader(ds, False)))
    tr.train_step(batch)
    tr.model.layers[0].self_attn.qkv_proj.grad[0, 0] = float("nan")  # poisoned on the host side of the test
    before = tr.engine.buckets[0].flat_param.clone()
    stats = tr.optimizer_step()
    assert float(stats["skipped"]) == 1.0 and torch.equal(before, tr.engine.buckets[0].flat_param)

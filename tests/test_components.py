"""Config, data, tokenizer, orchestrator, Chinchilla planner, monitoring, inference sampling, security -- all on CPU."""
import json
import math
import os
import time

import pytest
import torch

from adaptivetrainingsystem_b200.config import Config, ConfigManager, ConfigPresets, ModelConfig
from adaptivetrainingsystem_b200.data import (BaseTrainingDataset, ConversationDataset, InterleavedDataset, SyntheticTokenDataset,
                                              create_dataloader, setup_datasets)
from adaptivetrainingsystem_b200.data.tokenizer import ConversationTokenizer
from adaptivetrainingsystem_b200.inference import KVSlotManager, SamplingParams, sample_next
from adaptivetrainingsystem_b200.models import DeepSeekTransformer
from adaptivetrainingsystem_b200.monitoring.logger import MetricsCollector, TrainingHealthMonitor
from adaptivetrainingsystem_b200.security import AuthManager, InputValidator, RateLimiter
from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer, LRSchedule
from adaptivetrainingsystem_b200.training.chinchilla import ConvergenceDetector, EnhancedChinchillaScaler
from adaptivetrainingsystem_b200.training.orchestrator import (AdaptiveTrainingOrchestrator, ArchitectureEvolution, MetaLearningEngine,
                                                               RealTimeAnalytics)
from adaptivetrainingsystem_b200.training.trainer import TrainingMetrics


# -- config -------------------------------------------------------------------------------------------------------
def test_config_validation_presets_and_round_trip(tmp_dir):
    with pytest.raises(ValueError):
        Config(hidden_size=100, num_heads=8)
    with pytest.raises(ValueError):
        Config(precision="fp7")
    c = Config(num_experts=4, precision="mixed_fp8")  # both rejected by the reference, documented as supported
    assert c.to_model_config().fp8 and c.intermediate_size % 64 == 0 and c.vocab_size % 64 == 0
    for name in ConfigPresets.names():
        p = ConfigPresets.get(name)
        assert p.hidden_size % p.num_heads == 0 and p.num_parameters() > 0
    mix = ConfigPresets.mixtral_8x7b()
    assert 45e9 < mix.num_parameters() < 48e9 and 12e9 < mix.num_parameters(True) < 14e9
    for ext in ("yaml", "json"):
        path = os.path.join(tmp_dir, f"c.{ext}")
        c.some_runtime_flag = 3
        c.save(path)
        d = Config.load(path)
        assert d.hidden_size == c.hidden_size and d.some_runtime_flag == 3 and d.precision == "mixed_fp8"
    ds = c.to_deepspeed_config()
    assert ds["zero_optimization"]["stage"] == c.zero_stage and ds["moe"]["num_experts"] == 4
    fitted = ConfigManager.optimize_for_hardware(ConfigPresets.b7(), device_memory_gb=180, world_size=8)
    assert fitted.zero_stage >= 1 and fitted.expert_parallel_size == 8
    assert isinstance(ConfigManager.validate_config(Config(learning_rate=0.1)), list)
    assert "b7" in ConfigPresets.compare_presets()


def test_model_config_layer_patterns():
    m = ModelConfig(num_layers=8, use_moe=True, moe_pattern="every_4th", use_mod=True)
    assert [m.is_moe_layer(i) for i in range(8)] == [False, False, False, True, False, False, False, True]
    assert m.is_mod_layer(0) and not m.is_mod_layer(3)
    s = ModelConfig(num_layers=8, use_moe=True, moe_pattern="sandwich")
    assert [s.is_moe_layer(i) for i in range(8)] == [False, False, True, True, True, True, False, False]


# -- data ---------------------------------------------------------------------------------------------------------
def test_datasets_and_loader(tmp_dir):
    tok = ConversationTokenizer()
    conv = os.path.join(tmp_dir, "c.jsonl")
    with open(conv, "w") as f:
        for i in range(10):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"question {i}"}, {"role": "assistant", "content": f"answer {i}"}]}) + "\n")
        f.write("not json\n")
        f.write(json.dumps({"messages": [{"role": "alien", "content": "x"}]}) + "\n")
    txt = os.path.join(tmp_dir, "b.txt")
    with open(txt, "w") as f:
        f.write("\n\n".join("paragraph %d " % i * 20 for i in range(30)))
    cd = ConversationDataset([conv], tok, 64, assistant_loss_weight=2.0)
    assert len(cd) == 10 and cd.stats["invalid"] == 2
    item = cd[0]
    assert set(item) == {"input_ids", "labels", "attention_mask", "loss_weights"} and item["input_ids"].shape == (64,)
    assert item["loss_weights"].max() == 2.0 and (item["labels"] == -100).any()
    valid = item["labels"] != -100
    assert torch.equal(item["labels"][valid][:-1], item["input_ids"][1:][valid[:-1]][: valid.sum() - 1])
    bd = BaseTrainingDataset([txt], tok, 64)
    assert len(bd) > 0 and torch.equal(bd[0]["labels"][:-1], bd[0]["input_ids"][1:])
    cfg = Config(seq_length=64, batch_size=2, training_mode="interleaved", base_training_paths=[txt], finetuning_paths=[conv],
                 train_data_path=conv, eval_data_path=conv, num_workers=0, vocab_size=tok.vocab_size)
    tr, ev = setup_datasets(cfg, tok)
    assert isinstance(tr, InterleavedDataset) and len(tr) == len(bd) + len(cd) and len(ev) == 10
    batch = next(iter(create_dataloader(tr, cfg)))
    assert batch["input_ids"].shape == (2, 64)
    s = SyntheticTokenDataset(1000, 16, 4, seed=3)
    assert torch.equal(s[2]["input_ids"], SyntheticTokenDataset(1000, 16, 4, seed=3)[2]["input_ids"])


def test_tokenizer():
    t = ConversationTokenizer()
    assert t.vocab_size % 128 == 0 and t.pad_token_id >= t.base_vocab_size and len(t.special_tokens) == 13
    text = "héllo wörld ✓"
    assert t.decode(t.encode(text)) == text
    enc = t.encode_conversation([{"role": "system", "content": "s" * 50}, {"role": "user", "content": "u" * 200}], max_length=100,
                                truncation="keep_system")
    assert len(enc["input_ids"]) == 100 and enc["roles"][0] == "system" and enc["roles"][-1] == "user"
    assert len(t.encode_batch(["a", "bb"] * 40)) == 80


# -- schedulers ---------------------------------------------------------------------------------------------------
def test_lr_schedules():
    for kind in ("cosine", "linear", "onecycle", "constant"):
        s = LRSchedule(kind, 1e-3, 100, warmup_ratio=0.1, min_lr=1e-5)
        lrs = [s.step() for _ in range(100)]
        assert all(0 < x <= 1e-3 + 1e-12 for x in lrs)
        if kind in ("cosine", "linear"):
            assert lrs[-1] == pytest.approx(1e-5, rel=1e-3) and max(lrs) == pytest.approx(1e-3, rel=0.02)
    s = LRSchedule("cosine", 1e-3, 100)
    s.scale_base(0.1)
    assert s.lr_at(0) == pytest.approx(1e-4)
    # the vendored scheduler package's shapes: steps at milestones, polynomial decay, flat then cosine
    ms = LRSchedule("multistep", 1e-3, 100, milestones=[0.5, 0.75], gamma=0.1)
    assert [ms.lr_at(t) for t in (0, 49, 50, 74, 75, 99)] == pytest.approx([1e-3, 1e-3, 1e-4, 1e-4, 1e-5, 1e-5])
    assert LRSchedule("multistep", 1e-3, 100, milestones=[30, 60]).lr_at(45) == pytest.approx(1e-4)      # absolute steps
    po = LRSchedule("poly", 1e-3, 100, min_lr=1e-5, power=2.0)
    assert po.lr_at(0) == pytest.approx(1e-3) and po.lr_at(50) == pytest.approx(1e-5 + (1e-3 - 1e-5) * 0.25) and po.lr_at(100) == pytest.approx(1e-5)
    fa = LRSchedule("flat_anneal", 1e-3, 100, warmup_ratio=0.1, min_lr=0.0, flat_fraction=0.5)
    assert fa.lr_at(5) < 1e-3 and fa.lr_at(30) == pytest.approx(1e-3) and 0 < fa.lr_at(80) < 1e-3 and fa.lr_at(100) == pytest.approx(0.0, abs=1e-12)
    restored = LRSchedule("cosine", 1.0, 1)
    restored.load_state_dict(ms.state_dict())
    assert restored.lr_at(60) == ms.lr_at(60)
    assert Config(lr_scheduler="poly", lr_power=2.0).lr_power == 2.0


# -- orchestrator ---------------------------------------------------------------------------------------------------
def _tm(step, loss, gn=1.0, util=None):
    return TrainingMetrics(epoch=0, step=step, loss=loss, grad_norm=gn, learning_rate=1e-3, expert_utilization=util or {})


def test_anomaly_detection():
    a = RealTimeAnalytics(min_samples=50)
    for i in range(80):
        assert not a.detect_training_anomalies(_tm(i, 2.0 + 0.01 * math.sin(i)))
    kinds = set()
    for i in range(12):
        kinds |= {x["type"] for x in a.detect_training_anomalies(_tm(80 + i, 4.0))}
    assert "loss_spike" in kinds
    assert {x["type"] for x in a.detect_training_anomalies(_tm(100, 2.0, gn=500.0))} >= {"gradient_explosion"}
    assert a.detect_training_anomalies(_tm(101, float("nan")))[0]["type"] == "divergence"
    util = {f"layer_0_expert_{j}": v for j, v in enumerate([0.5, 60.0, 20.0, 19.5])}
    assert "expert_collapse" in {x["type"] for x in a.detect_training_anomalies(_tm(102, 2.0, util=util))}


def test_orchestrator_decisions_drive_the_trainer(tmp_dir):
    cfg = Config(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32,
                 batch_size=4, micro_batch_size=4, gradient_accumulation_steps=1, num_epochs=1, precision="fp32", use_moe=True,
                 num_experts=4, output_dir=tmp_dir, experiment_name="o", log_every_n_steps=1, num_workers=0, gradient_checkpointing=False)
    torch.manual_seed(0)
    model = DeepSeekTransformer(cfg.to_model_config())
    orch = AdaptiveTrainingOrchestrator(cfg, model=model)
    tr = orch.initialize_training()
    lr0 = tr.engine.get_lr()
    orch._handle_training_anomaly({"type": "gradient_explosion", "severity": "critical", "detail": "test"}, _tm(1, 2.0, 500.0))
    assert tr.engine.get_lr() < lr0 / 5 and orch.decisions[-1].applied
    orch._decide("add_expert", {"layer_idx": 0}, 0.8, "test")
    assert tr.model.get_moe_layers()[0].num_experts == 5
    orch._decide("prune_expert", {"layer_idx": 0, "expert_idx": 4}, 0.8, "test")
    assert tr.model.get_moe_layers()[0].num_experts == 4
    orch._decide("expert_rebalance", {"temperature_factor": 1.5, "capacity_factor": 1.2}, 0.8, "test")
    assert tr.model.get_moe_layers()[0].routing_temperature == pytest.approx(1.5)
    from adaptivetrainingsystem_b200.data import SyntheticTokenDataset as S
    summary = orch.run_adaptive_training(S(512, 32, 16, seed=0))
    assert summary["global_step"] == 4 and summary["adaptive"]["decisions_total"] >= 4
    assert os.path.exists(os.path.join(tmp_dir, "o", "adaptive_learning_summary.json"))
    assert os.path.exists(os.path.join(tmp_dir, "o", "meta_learning_state.pkl"))
    # a decision posted from another thread is applied at the next step boundary, not concurrently
    import threading
    t = threading.Thread(target=lambda: tr.adjust_learning_rate(3.3e-6))
    t.start(); t.join()
    assert tr.engine.get_lr() != pytest.approx(3.3e-6) and len(tr._pending) == 1
    batch = next(iter(tr._make_loader(S(512, 32, 4, seed=0), False)))
    tr.train_step(batch); tr.optimizer_step()
    assert tr.engine.get_lr() == pytest.approx(3.3e-6)
    # documented helper: which post-training quantisation fits the serving memory
    assert orch.suggest_quantization_adjustment(serving_memory_gb=180.0)["suggested"] is None
    tight = orch.suggest_quantization_adjustment(serving_memory_gb=1e-4)
    assert tight["suggested"] == "fp8" and tight["fraction_of_memory"] > 1      # a MoE model: the experts need the e4m3 path
    orch.cleanup()


def test_meta_learning_and_architecture_policy(tmp_dir):
    p = os.path.join(tmp_dir, "m.pkl")
    m = MetaLearningEngine(p)
    m.record_run({"parameters": 1e9, "learning_rate": 2e-4}, 2.5, True)
    m.save()
    m2 = MetaLearningEngine(p)
    assert m2.suggest_hyperparameters({"parameters": 2e9})["learning_rate"] == 2e-4
    traj = m2.predict_training_trajectory([5.0 / (i + 1) ** 0.3 for i in range(100)])
    assert traj["slope"] < 0
    with open(p, "wb") as f:
        f.write(b"garbage")
    assert MetaLearningEngine(p).training_history == []  # a corrupt state file is survivable
    props = ArchitectureEvolution().propose({"layer_3": {"expert_usage": [0.9, 0.05, 0.03, 0.02, 0.0]}})
    assert props[0]["action"] == "add_expert" and props[0]["layer_idx"] == 3
    props = ArchitectureEvolution().propose({"layer_1": {"expert_usage": [0.3, 0.3, 0.3, 0.099, 0.001]}})
    assert props[0]["action"] == "prune_expert" and props[0]["expert_idx"] == 4


# -- chinchilla / monitoring ------------------------------------------------------------------------------------------
def test_chinchilla_planner(tmp_dir):
    cfg = Config(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, vocab_size=512, use_moe=True, num_experts=8, seq_length=32)
    sc = EnhancedChinchillaScaler(cfg, dataset_tokens=10_000)
    assert sc.active_params < sc.total_params
    assert sc.get_optimal_epochs() == max(1, min(50, math.ceil(20 * sc.active_params / 10_000)))
    for i in range(600):
        sc.update_metrics(i, 3.0, 1000.0, 1.0)
    assert sc.convergence.status()["state"] in ("plateau", "slowing") and sc.should_stop_early()
    sc.save_state(os.path.join(tmp_dir, "s.json"))
    det = ConvergenceDetector(window=20)
    for i in range(100):
        det.update(5.0 - 0.03 * i)
    assert det.status()["state"] == "improving"


def test_monitoring():
    c = MetricsCollector()
    for i in range(30):
        c.add_many({"loss": 2.0 - 0.01 * i, "grad_norm": 1.0}, i)
    assert c.trend("loss") < 0 and c.health_score() > 0.9
    assert any(a.message == "loss spike" for a in c.add("loss", 9.0, 31))
    assert c.add("grad_norm", 1e4, 32)[0].level == "critical"
    h = TrainingHealthMonitor(check_interval=10)
    for i in range(120):
        h.update(i, 3.0 * math.exp(-i / 40), 1.0, 1e-3, 1000.0)
    assert h.phase in ("rapid_learning", "steady_learning") and h.get_report()["checks"]


# -- inference sampling / security ---------------------------------------------------------------------------------------
def test_sampling_rules():
    torch.manual_seed(0)
    logits = torch.tensor([[0.0, 5.0, 4.0, -1.0, 3.0]])
    assert sample_next(logits, SamplingParams(temperature=0.0)).item() == 1
    hist = torch.tensor([[1, 1]])
    assert sample_next(logits, SamplingParams(temperature=0.0, repetition_penalty=2.0), hist).item() == 2
    picks = {sample_next(logits, SamplingParams(temperature=1.0, top_k=2, top_p=1.0, repetition_penalty=1.0)).item() for _ in range(50)}
    assert picks <= {1, 2}
    picks = {sample_next(logits, SamplingParams(temperature=1.0, top_k=0, top_p=0.5, repetition_penalty=1.0)).item() for _ in range(50)}
    assert picks == {1}
    s = KVSlotManager(8)
    a = s.alloc(3)
    assert s.alloc_contiguous(6) is None and s.alloc_contiguous(5).tolist() == [3, 4, 5, 6, 7]
    s.free(a)
    assert s.available == 3


def test_security_primitives():
    a = AuthManager(iterations=1000, max_attempts=2, lockout_s=60)
    a.create_user("alice", "correct horse")
    tok = a.authenticate("alice", "correct horse")
    assert a.verify(tok)["sub"] == "alice" and a.verify(tok + "x") is None
    assert a.authenticate("alice", "bad") is None and a.authenticate("alice", "bad") is None
    assert a.authenticate("alice", "correct horse") is None  # locked out
    a.logout(tok)
    assert a.verify(tok) is None
    now = [0.0]
    r = RateLimiter(2, 10.0, clock=lambda: now[0])
    assert r.allow("k")[0] and r.allow("k")[0] and not r.allow("k")[0]
    now[0] = 11.0
    assert r.allow("k")[0]
    v = InputValidator(max_length=50)
    assert v.validate("hello")[0] and not v.validate("<script>alert(1)</script>")[0] and not v.validate("x" * 51)[0]


def test_quantization_manager_methods_and_refusals():
    """bits=8 without a method selects the native fp8 path and bits=4 the native 4-bit one; GPTQ refuses to run uncalibrated;
    external backends that are not installed are refused."""
    from types import SimpleNamespace
    from adaptivetrainingsystem_b200.training import QuantizationManager
    qm = QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=8))
    st = qm.status()
    assert st["method"] == "fp8" and not st["applied"] and "bitsandbytes" in st["backends"]
    assert QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=None)).quantize_model("m") == "m"
    assert QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=4)).status()["method"] == "int4"
    with pytest.raises(RuntimeError):
        QuantizationManager(SimpleNamespace(quantization_method="gptq", quantization_bits=4)).quantize_model(None)
    with pytest.raises(RuntimeError):
        QuantizationManager(SimpleNamespace(quantization_method="bnb", quantization_bits=4)).quantize_model(None)
    info = qm.get_quantization_info()                       # the reference manager's names
    assert info["is_quantized"] is False and info["method"] == "fp8" and info["available_methods"]["gptq"] and not qm.is_quantized
    assert qm.create_quantized_optimizer(None) is None


def test_swiglu_backward_gemm_reference_matches_autograd():
    """CPU definition of the fused dh GEMM + SwiGLU backward against autograd through silu(gate) * up."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(0)
    M, H, I = 12, 16, 24
    dy, w2 = torch.randn(M, H), torch.randn(H, I)
    pre = torch.randn(M, 2 * I, requires_grad=True)
    g, u = pre.chunk(2, dim=-1)
    h_ref = torch.nn.functional.silu(g) * u
    h_ref.backward(dy @ w2)
    dgu, h = G.gemm_nn_swiglu_bwd(dy, w2, pre.detach())
    assert torch.allclose(h, h_ref.detach(), atol=1e-5) and torch.allclose(dgu, pre.grad, atol=1e-5)
    counts = torch.tensor([M], dtype=torch.int32)
    dgu_g, h_g = G.grouped_nn_swiglu_bwd(dy.view(1, M, H), w2.view(1, H, I), counts, pre.detach().view(1, M, 2 * I))
    assert torch.allclose(dgu_g[0], pre.grad, atol=1e-5) and torch.allclose(h_g[0], h_ref.detach(), atol=1e-5)


def test_skinny_product_split_rule_and_weight_packing():
    """Host-side rules of the serving GEMM paths: when the reduction is split, and the tile-packed weight layout."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    assert G._skinny_splits(64, 4096, 14336) == 8      # 16 output tiles: spread over 8 x 16 CTAs
    assert G._skinny_splits(64, 6144, 4096) == 4
    assert G._skinny_splits(64, 28672, 4096) == 1      # 112 tiles already fill the GPU
    assert G._skinny_splits(256, 4096, 14336) == 1     # not skinny
    assert G._skinny_splits(64, 4096, 1024) == 1       # reduction too short to split
    for m, n, k in ((1, 256, 2048), (128, 512, 8192), (64, 4096, 4096)):
        s = G._skinny_splits(m, n, k)
        assert k % (s * 64) == 0 and k // s >= 512 and s * ((n + 255) // 256) <= 160
    w = torch.arange(2 * 256 * 128, dtype=torch.float32).view(2, 256, 128)
    p = G.pack_kmajor(w)
    assert p.shape == w.shape and torch.equal(G.unpack_kmajor(p), w)
    # box (weight 1, row block 1, k block 1) is one contiguous run of 128 x 64 elements
    off = ((1 * 2 + 1) * 2 + 1) * 128 * 64
    assert torch.equal(p.reshape(-1)[off:off + 128 * 64].view(128, 64), w[1, 128:256, 64:128])
    with pytest.raises(ValueError):
        G.pack_kmajor(torch.zeros(100, 64))
    x = torch.randn(2, 128, 128)
    counts = torch.tensor([128, 7], dtype=torch.int32)
    assert torch.allclose(G.grouped_nt(x, w * 1e-4, counts), G.grouped_nt(x, G.pack_kmajor(w * 1e-4), counts, packed=True))


def test_weight_gradient_split_model_and_fp8_weight_copies():
    """Pure host logic: the wave model that decides reduction slices for weight-gradient products, and the per-input-channel
    e4m3 copy of a weight used by the fp8 input-gradient product (PyTorch definitions on CPU)."""
    from adaptivetrainingsystem_b200.ops import fp8
    from adaptivetrainingsystem_b200.ops import gemm as G
    assert G._tn_splits(2560, 2048, 16384) > 1          # 80 tiles on 74 CTA pairs: two waves at 0.54 utilisation
    assert G._tn_splits(2048, 2048, 16384) == 1         # 64 tiles: one wave
    assert G._tn_splits(32000, 2048, 16384) == 1        # many waves: the last partial one is noise
    assert G._tn_splits(2560, 2048, 4096) == 1          # short reduction: the fold would cost more than it saves
    torch.manual_seed(0)
    w = torch.randn(48, 32) * torch.logspace(-2, 1, 32)[None, :]     # input channels of very different magnitude
    fp8.clear_weight_cache()
    q, s = fp8.quantized_weight_t(w)
    assert q.shape == (32, 48) and s.shape == (32,)
    back = (q.float() * s[:, None]).t()
    assert ((back - w).abs() / w.abs().amax(0, keepdim=True)).max() < 0.07      # every channel resolved on its own scale
    q2, s2 = fp8.quantized_weight_t(w)
    assert q2 is q                                        # cached until the weights change
    fp8.weights_changed()
    assert fp8.quantized_weight_t(w)[0] is not q
    stacked = torch.randn(3, 16, 32)
    qe, se = fp8.quantized_weight_t(stacked)
    assert qe.shape == (3 * 32, 16) and se.shape == (96,)


def test_int8_and_smoothquant_post_training_quantisation_cpu():
    """W8A8 int8 through the manager (PyTorch definitions on CPU): close to the unquantised logits; SmoothQuant refuses to run
    uncalibrated and, on activations with outlier channels, beats plain int8."""
    from adaptivetrainingsystem_b200.ops import int8
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager

    class _C:
        quantization_bits = 8

        def __init__(self, method):
            self.quantization_method = method

    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=256, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=32)
    ids = torch.randint(0, 256, (2, 32))
    try:
        model = DeepSeekTransformer(cfg)
        with torch.no_grad():
            ref = model(ids, return_aux_loss=False)
        with pytest.raises(RuntimeError):
            QuantizationManager(_C("smoothquant")).quantize_model(model)
        qm = QuantizationManager(_C("int8"))
        qm.quantize_model(model)
        with torch.no_grad():
            out = model(ids, return_aux_loss=False)
        assert qm.status()["applied"] and qm.status()["tensors"] >= 7
        assert ((out - ref).norm() / ref.norm()).item() < 3e-2
        # outlier channels: a few input channels 50 x larger than the rest
        int8.clear()
        x = torch.randn(64, 128)
        x[:, :4] *= 50.0
        w = torch.randn(96, 128) * 0.05
        exact = x @ w.t()
        int8.set_enabled(True)
        with torch.no_grad():
            plain = int8.linear_int8(x, w)
        int8.record(x, w)
        int8.finish_calibration(0.5)
        with torch.no_grad():
            smooth = int8.linear_int8(x, w)
        e_plain = ((plain - exact).norm() / exact.norm()).item()
        e_smooth = ((smooth - exact).norm() / exact.norm()).item()
        assert e_smooth < 0.6 * e_plain and e_smooth < 2e-2, (e_plain, e_smooth)
    finally:
        int8.set_enabled(False)
        int8.clear()


def test_continuous_batcher_needs_a_gpu_and_validates_requests():
    from adaptivetrainingsystem_b200.inference import ContinuousBatcher, GenerationEngine
    model = DeepSeekTransformer(ModelConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, num_kv_heads=2, intermediate_size=64,
                                            seq_length=32)).eval()
    with pytest.raises(RuntimeError, match="CUDA"):
        ContinuousBatcher(GenerationEngine(model), max_batch=2, max_len=16)

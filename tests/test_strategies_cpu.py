"""Tensor, sequence and pipeline parallelism selected through ``Config`` and applied by the trainer, on Gloo ranks, against the
same training steps in one process."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_dist  # noqa: E402

from adaptivetrainingsystem_b200.config import Config  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402

pytestmark = pytest.mark.dist


def _config(tmp, **kw):
    base = dict(vocab_size=256, hidden_size=64, num_layers=4, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=16,
                use_moe=False, precision="fp32", gradient_checkpointing=False, tie_word_embeddings=False, learning_rate=1e-2,
                batch_size=2, micro_batch_size=2, gradient_accumulation_steps=2, zero_stage=1, output_dir=tmp, experiment_name="s",
                num_workers=0, heartbeat_interval_s=0.0, use_lr_scheduler=False, weight_decay=0.0)
    base.update(kw)
    return Config(**base)


def _data():
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 256, (4, 17), generator=g)
    return [{"input_ids": ids[2 * i:2 * i + 2, :-1], "labels": ids[2 * i:2 * i + 2, 1:]} for i in range(2)]


def _train(trainer, steps=2):
    losses = []
    for _ in range(steps):
        for mb in _data():
            out = trainer.train_step(mb)
            losses.append(out["loss"])
        trainer.optimizer_step()
    return losses


def _reference(tmp):
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer
    cfg = _config(tmp)
    torch.manual_seed(0)
    model = DeepSeekTransformer(cfg.to_model_config())
    init = {k: v.clone() for k, v in model.state_dict().items()}
    tr = EnhancedConversationTrainer(model, None, cfg)
    _train(tr)
    return init, {k: v.clone() for k, v in model.state_dict().items()}


def _worker(rank, world, kind, path, tmp):
    from adaptivetrainingsystem_b200.parallel import ProcessMesh
    from adaptivetrainingsystem_b200.parallel.strategy import gather_tensor_parallel_state
    from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer
    ref = torch.load(path)
    extra = {"tp": dict(tensor_parallel_size=2), "sp": dict(sequence_parallel_size=2), "pp": dict(pipeline_parallel_size=2),
             "pp_interleaved": dict(pipeline_parallel_size=2, pipeline_chunks=2)}[kind]
    cfg = _config(os.path.join(tmp, f"r{rank}"), **extra)
    mesh = ProcessMesh.from_config(cfg, world, rank)
    assert mesh.describe().startswith({"tp": "tp2", "sp": "sp2", "pp": "pp2", "pp_interleaved": "pp2"}[kind]), mesh.describe()
    model = DeepSeekTransformer(cfg.to_model_config())
    model.load_state_dict(ref["init"])
    tr = EnhancedConversationTrainer(model, None, cfg, mesh=mesh)
    if kind == "tp":
        assert model.layers[0].self_attn.n_q == 2 and model.layers[0].ffn.down_proj.shape == (64, 64)
    if kind.startswith("pp"):
        assert sum(p.numel() for p in model.parameters()) < sum(v.numel() for v in ref["init"].values())  # foreign stages are gone
    _train(tr)
    got = gather_tensor_parallel_state(model, mesh) if kind == "tp" else model.state_dict()
    checked = 0
    for k, v in ref["final"].items():
        if k not in got or got[k].numel() == 0:
            continue
        assert got[k].shape == v.shape and torch.allclose(got[k], v, atol=3e-5, rtol=1e-4), (kind, k, (got[k] - v).abs().max())
        checked += 1
    assert checked >= (len(ref["final"]) if kind in ("tp", "sp") else 8), (kind, checked)
    if kind.startswith("pp"):
        m = tr._flush_metrics()
        assert m is not None and m["loss"] > 0  # the last stage's loss reached every stage
    tr.shutdown()


@pytest.mark.parametrize("kind", ["tp", "sp", "pp", "pp_interleaved"])
def test_strategy_from_config_matches_single_process(kind, tmp_path):
    init, final = _reference(str(tmp_path / "ref"))
    path = str(tmp_path / "ref.pt")
    torch.save({"init": init, "final": final}, path)
    run_dist(_worker, 2, (kind, path, str(tmp_path)))

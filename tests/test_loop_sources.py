"""Stand-alone training loop, corpus file formats, diagnostics report (CPU)."""
import json

import torch

from adaptivetrainingsystem_b200.config import ConfigPresets
from adaptivetrainingsystem_b200.data import sources
from adaptivetrainingsystem_b200.data.dataset import SyntheticTokenDataset
from adaptivetrainingsystem_b200.models.transformer import DeepSeekTransformer
from adaptivetrainingsystem_b200.training.checkpoint import CheckpointManager
from adaptivetrainingsystem_b200.training.trainer import EnhancedConversationTrainer
from adaptivetrainingsystem_b200.training.training_loop import TrainingLoop
from adaptivetrainingsystem_b200.utils import diagnostics


def test_training_loop_runs_evaluates_and_saves(tmp_path):
    torch.manual_seed(0)
    cfg = ConfigPresets.tiny_cpu()
    cfg.num_epochs, cfg.gradient_accumulation_steps, cfg.batch_size = 2, 1, 2
    cfg.output_dir = str(tmp_path)
    model = DeepSeekTransformer(cfg.to_model_config())
    trainer = EnhancedConversationTrainer(model, None, cfg)
    ckpt = CheckpointManager(cfg, directory=str(tmp_path / "ckpt"))
    loop = TrainingLoop(trainer, ckpt, eval_every_n_steps=3, save_every_n_steps=4, max_steps=8)
    train = SyntheticTokenDataset(cfg.vocab_size, cfg.seq_length, 16, seed=1)
    ev = SyntheticTokenDataset(cfg.vocab_size, cfg.seq_length, 4, seed=2)
    out = loop.train(train, ev)
    assert out["global_step"] == 8 and loop.should_stop
    assert len(loop.metrics["train_losses"]) == 8 and len(loop.metrics["eval_losses"]) >= 2
    assert all(v > 0 for v in loop.metrics["throughput"])
    assert out["best_eval_loss"] < float("inf")


def test_corpus_formats_roundtrip(tmp_path):
    docs = [{"source": "wikipedia", "text": "Alpha line one.\nAlpha line two."}, {"source": "arxiv", "text": "Beta abstract."}]
    p = tmp_path / "corpus.txt"
    assert sources.write_text_corpus(docs, str(p)) == 2
    back = list(sources.iter_text_documents(str(p)))
    assert back == docs
    stats = sources.corpus_statistics([str(p)])
    assert stats["wikipedia"]["documents"] == 1 and stats["arxiv"]["characters"] == len("Beta abstract.")
    msgs = [{"message_id": "a", "parent_id": None, "role": "prompter", "text": "Hi", "lang": "en"},
            {"message_id": "b", "parent_id": "a", "role": "assistant", "text": "Hello!", "lang": "en"}]
    mp = tmp_path / "oasst.jsonl"
    mp.write_text("\n".join(json.dumps(m) for m in msgs))
    n = sources.convert_oasst_export(str(mp), str(tmp_path / "conv.jsonl"))
    convs = list(sources.iter_conversations(str(tmp_path / "conv.jsonl")))
    assert n == len(convs) == 1 and [m["role"] for m in convs[0]["messages"]] == ["user", "assistant"]


def test_diagnostics_report_without_gpu():
    rep = diagnostics.collect()
    assert "torch" in rep and isinstance(rep["devices"], list)
    assert diagnostics.main(["--json"]) == 0 or torch.cuda.is_available()

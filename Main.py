#!/usr/bin/env python
"""Training entry point.

    python Main.py --preset b1 [--override key=value ...] [--synthetic N] [--resume latest]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 Main.py --preset b7 --synthetic 100000

Pipeline (reference ``Main.py:1506-3145``): diagnostics -> preset + overrides -> precision / environment validation ->
tokenizer -> datasets -> time estimate -> model -> engine (DDP / ZeRO / expert parallel) -> orchestrator -> Chinchilla
epoch plan -> optional resume -> scheduler -> experiment directory -> training with OOM protection -> reports.
The reference edits in-file dictionaries; the same keys are accepted here as ``--override`` pairs or a YAML/JSON file."""
from __future__ import annotations

import argparse
import ast
import logging
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from adaptivetrainingsystem_b200.config import Config, ConfigManager, ConfigPresets  # noqa: E402
from adaptivetrainingsystem_b200.data import SyntheticTokenDataset, setup_datasets  # noqa: E402
from adaptivetrainingsystem_b200.data.tokenizer import ConversationTokenizer  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.monitoring.logger import ProductionLogger  # noqa: E402
from adaptivetrainingsystem_b200.parallel import ProcessMesh, init_distributed, shutdown  # noqa: E402
from adaptivetrainingsystem_b200.training import EnhancedConversationTrainer  # noqa: E402
from adaptivetrainingsystem_b200.training.chinchilla import auto_adjust_epochs_chinchilla  # noqa: E402
from adaptivetrainingsystem_b200.training.orchestrator import AdaptiveTrainingOrchestrator  # noqa: E402
from adaptivetrainingsystem_b200.utils import estimate_training_time, get_system_info, print_system_diagnostics, validate_environment  # noqa: E402
from adaptivetrainingsystem_b200.utils.reporting import create_html_report, create_training_summary, save_experiment_metadata  # noqa: E402


def parse_overrides(pairs):
    out = {}
    for p in pairs or []:
        k, _, v = p.partition("=")
        try:
            out[k] = ast.literal_eval(v)
        except Exception:
            out[k] = v
    return out


def validate_precision_support(precision: str, device: torch.device) -> str:
    if device.type != "cuda" and precision not in ("fp32", "fp64"):
        return "fp32"
    return precision


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="debug", choices=ConfigPresets.names())
    ap.add_argument("--config", default=None, help="YAML / JSON file saved by Config.save (wins over --preset)")
    ap.add_argument("--override", nargs="*", default=[])
    ap.add_argument("--synthetic", type=int, default=0, help="train on N synthetic sequences instead of files")
    ap.add_argument("--resume", default=None, help="checkpoint path, 'latest' or 'best'")
    ap.add_argument("--no-orchestrator", action="store_true")
    args = ap.parse_args(argv)

    rank, local_rank, world = init_distributed()
    over = parse_overrides(args.override)
    cfg = Config.load(args.config) if args.config else ConfigManager.create_config(args.preset, over)
    if args.config:
        for k, v in over.items():
            setattr(cfg, k, v)
    cfg.world_size = world
    logger = ProductionLogger(cfg.log_level, cfg.experiment_name, os.path.join(cfg.output_dir, cfg.experiment_name, "logs"), rank)
    if rank == 0:
        print_system_diagnostics()
        for w in ConfigManager.validate_config(cfg):
            logger.warning("config: %s", w)
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    cfg.precision = validate_precision_support(cfg.precision, device)
    problems = [p for p in validate_environment(None) if "no CUDA" not in p]
    for p in problems:
        logger.warning("environment: %s", p)

    tokenizer = ConversationTokenizer()
    if args.synthetic:
        train_ds = SyntheticTokenDataset(cfg.vocab_size, cfg.seq_length, args.synthetic, cfg.seed)
        eval_ds = SyntheticTokenDataset(cfg.vocab_size, cfg.seq_length, max(args.synthetic // 20, cfg.micro_batch_size), cfg.seed + 1)
    else:
        cfg.vocab_size = max(cfg.vocab_size, tokenizer.vocab_size)
        train_ds, eval_ds = setup_datasets(cfg, tokenizer)
        if train_ds is None:
            logger.error("no training data found (train_data_path=%s); use --synthetic N for a dry run", cfg.train_data_path)
            return 2

    ep = 1
    if cfg.use_moe and world > 1:
        import math
        ep = math.gcd(cfg.num_experts, world) if not cfg.expert_parallel_size else min(cfg.expert_parallel_size, world)
    mesh = ProcessMesh(world, rank, ep_size=ep)
    dtype = torch.bfloat16 if device.type == "cuda" and cfg.precision not in ("fp32", "fp64") else torch.float32
    torch.manual_seed(cfg.seed)
    model = DeepSeekTransformer(cfg.to_model_config(), ep_size=ep, ep_rank=mesh.coord.ep).to(device, dtype)
    fused = None
    if world > 1 and device.type == "cuda":
        from adaptivetrainingsystem_b200.parallel.expert_parallel import attach_expert_parallel
        fused = attach_expert_parallel(model, mesh, cfg, use_fused=cfg.fused_comm)
    trainer = EnhancedConversationTrainer(model, tokenizer if not args.synthetic else None, cfg, logger, mesh=mesh, fused_comm=fused)
    scaler = auto_adjust_epochs_chinchilla(cfg, model, train_ds)
    trainer.chinchilla_scaler = scaler
    if rank == 0:
        est = estimate_training_time(cfg, getattr(train_ds, "total_tokens", lambda: 0)(), world)
        logger.info("model %.2f B parameters (%.2f B active); planned epochs %d; estimated %.2f h at %.0f tok/s",
                    cfg.num_parameters() / 1e9, cfg.num_parameters(True) / 1e9, cfg.num_epochs, est["hours"], est["tokens_per_second"])
        save_experiment_metadata(cfg, os.path.join(cfg.output_dir, cfg.experiment_name), get_system_info())
    resume = args.resume
    if not resume and getattr(cfg, "auto_resume", False):
        # ``auto_resume``: an experiment directory that already holds checkpoints (same experiment name) continues from its latest
        ck_dir = trainer.checkpoint_manager.directory
        if os.path.isdir(ck_dir) and any(f.startswith("checkpoint_") and (f.endswith(".pt") or os.path.isdir(os.path.join(ck_dir, f)))
                                         for f in os.listdir(ck_dir)):
            resume = "latest"
    if resume:
        info = trainer.load_checkpoint(resume)
        logger.info("resumed from %s at step %d", info["path"], info["global_step"])

    if args.no_orchestrator:
        summary = trainer.train_with_oom_fallback(train_ds, eval_ds)
    else:
        orch = AdaptiveTrainingOrchestrator(cfg, model, tokenizer, trainer, mesh, install_signal_handlers=True)
        orch.initialize_training(train_ds, eval_ds)
        summary = orch.run_adaptive_training(train_ds, eval_ds)
        orch.cleanup()
    if rank == 0:
        exp = os.path.join(cfg.output_dir, cfg.experiment_name)
        import json
        with open(os.path.join(exp, "training_summary.json"), "w") as f:
            json.dump(create_training_summary(trainer, {"epochs_detail": summary.get("epochs")}), f, indent=2, default=str)
        create_html_report(trainer, os.path.join(exp, "reports", "training_report.html"))
        scaler.save_state(os.path.join(exp, "chinchilla_scaler_final_state.json"))
        logger.info("done: %d steps, final checkpoint %s", trainer.global_step, summary.get("final_checkpoint"))
    shutdown()
    return 0


if __name__ == "__main__":
    logging.basicConfig(level=logging.INFO)
    sys.exit(main())

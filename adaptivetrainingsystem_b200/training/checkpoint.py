"""Checkpoint manager: single-file interchange format with the reference's schema and names, gathered from ZeRO / EP
shards on save and re-sharded on load, plus history, retention, best link, backup and emergency save.

File layout (reference ``training/checkpoint.py:51-70`` and ``training/trainer.py:3395-3422``)::

    {model_state_dict, optimizer_state_dict, scheduler_state_dict | None, global_step, epoch | current_epoch,
     metrics, config (dict), model_config {vocab_size, hidden_size, num_layers, num_heads, num_kv_heads, seq_length,
     intermediate_size, ...}, save_time, pytorch_version, rng_state}

``model_state_dict`` uses the reference parameter names (``layers.N.self_attn.q_proj.weight`` ...).  The RNG state is
saved (the reference README promises it, its code does not).  Loading accepts the key aliases
``module | model_state_dict | state_dict | model`` (reference ``Chat.py:150``).
"""
from __future__ import annotations

import json
import os
import shutil
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

MODEL_KEYS = ("model_state_dict", "module", "state_dict", "model")
ARCH_KEYS = ("vocab_size", "hidden_size", "num_layers", "num_heads")


class CheckpointError(RuntimeError):
    pass


class CheckpointManager:
    def __init__(self, config, directory: str = "checkpoints"):
        self.config = config
        self.directory = directory
        self.history_file = os.path.join(directory, "checkpoint_history.json")
        self.history: List[Dict[str, Any]] = []
        self.best_metric = float("inf")
        if os.path.exists(self.history_file):
            try:
                with open(self.history_file) as f:
                    self.history = json.load(f)
            except Exception:
                self.history = []

    # -- gather helpers -------------------------------------------------------------------------------------
    @staticmethod
    def _gather_model_state(model, mesh) -> Dict[str, torch.Tensor]:
        """Full model state on every rank: expert-parallel ranks contribute their own experts."""
        sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        if mesh is not None and mesh.ep_size > 1 and dist.is_initialized():
            mine = {k: v for k, v in sd.items() if ".ffn.experts." in k}
            parts: List[Optional[Dict[str, torch.Tensor]]] = [None] * mesh.ep_size
            dist.all_gather_object(parts, mine, group=mesh.group("ep"))
            for p in parts:
                sd.update(p or {})
        return sd

    def save_checkpoint(self, model, engine=None, scheduler=None, global_step: int = 0, epoch: int = 0,
                        metrics: Optional[Dict[str, Any]] = None, suffix: Optional[str] = None, mesh=None,
                        is_best: bool = False, eval_loss: Optional[float] = None) -> Optional[str]:
        rank = dist.get_rank() if dist.is_initialized() else 0
        if engine is not None and hasattr(engine, "gather_full_parameters"):
            engine.gather_full_parameters()  # ZeRO-3: materialise every block for the state dict
        model_sd = self._gather_model_state(model, mesh)
        if engine is not None and hasattr(engine, "release_parameters"):
            engine.release_parameters()
        opt_sd = engine.state_dict() if (engine is not None and getattr(self.config, "save_optimizer_states", True)) else None
        if opt_sd is not None and mesh is not None and mesh.ep_size > 1 and dist.is_initialized():
            mine = {k: v for k, v in opt_sd["state"].items() if "experts_w" in k}
            parts: List[Optional[Dict[str, Any]]] = [None] * mesh.ep_size
            dist.all_gather_object(parts, {f"ep{mesh.coord.ep}:{k}": v for k, v in mine.items()}, group=mesh.group("ep"))
            for p in parts:
                opt_sd["state"].update(p or {})
        if rank != 0:
            if dist.is_initialized():
                dist.barrier()
            return None
        os.makedirs(self.directory, exist_ok=True)
        name = f"checkpoint_{suffix}.pt" if suffix else f"checkpoint_epoch_{epoch:03d}_step_{global_step:06d}.pt"
        path = os.path.join(self.directory, name)
        mc = model.config.to_dict() if hasattr(model, "config") else {}
        payload = {
            "model_state_dict": model_sd, "optimizer_state_dict": opt_sd,
            "scheduler_state_dict": scheduler.state_dict() if scheduler is not None else None,
            "global_step": global_step, "epoch": epoch, "current_epoch": epoch,
            "metrics": {k: list(v)[-1000:] for k, v in (metrics or {}).items()},
            "config": self.config.to_dict() if hasattr(self.config, "to_dict") else dict(vars(self.config)),
            "model_config": mc, "save_time": time.time(), "pytorch_version": torch.__version__,
            "rng_state": {"torch": torch.get_rng_state(),
                          "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None},
        }
        tmp = path + ".tmp"
        torch.save(payload, tmp)
        os.replace(tmp, path)
        entry = {"path": path, "global_step": global_step, "epoch": epoch, "save_time": payload["save_time"],
                 "eval_loss": eval_loss, "suffix": suffix}
        self.history.append(entry)
        if is_best or (eval_loss is not None and eval_loss < self.best_metric):
            self.best_metric = eval_loss if eval_loss is not None else self.best_metric
            self._link_best(path)
        self._enforce_retention()
        self._write_history()
        if dist.is_initialized():
            dist.barrier()
        return path

    def _link_best(self, path: str) -> None:
        best = os.path.join(self.directory, "best_checkpoint.pt")
        try:
            if os.path.lexists(best):
                os.remove(best)
            os.symlink(os.path.basename(path), best)
        except OSError:
            shutil.copyfile(path, best)

    def _enforce_retention(self) -> None:
        limit = getattr(self.config, "save_total_limit", None)
        if not limit or limit <= 0:
            return
        best = os.path.join(self.directory, "best_checkpoint.pt")
        best_target = os.path.realpath(best) if os.path.lexists(best) else None
        regular = [e for e in self.history if not e.get("suffix")]
        while len(regular) > limit:
            victim = regular.pop(0)
            if best_target and os.path.realpath(victim["path"]) == best_target:
                continue
            try:
                os.remove(victim["path"])
            except OSError:
                pass
            self.history.remove(victim)

    def _write_history(self) -> None:
        with open(self.history_file, "w") as f:
            json.dump(self.history, f, indent=2)

    # -- load -----------------------------------------------------------------------------------------------
    def resolve(self, path: str) -> str:
        if path == "latest":
            cands = [e["path"] for e in self.history if os.path.exists(e["path"])]
            if not cands:
                cands = sorted((os.path.join(self.directory, f) for f in os.listdir(self.directory) if f.endswith(".pt")),
                               key=os.path.getmtime) if os.path.isdir(self.directory) else []
            if not cands:
                raise CheckpointError(f"no checkpoint in {self.directory}")
            return cands[-1]
        if path == "best":
            p = os.path.join(self.directory, "best_checkpoint.pt")
            if not os.path.exists(p):
                raise CheckpointError("no best checkpoint recorded")
            return p
        return path

    @staticmethod
    def read(path: str) -> Dict[str, Any]:
        try:
            return torch.load(path, map_location="cpu", weights_only=False)
        except Exception as e:
            raise CheckpointError(f"cannot read checkpoint {path}: {e}") from e

    def load_checkpoint(self, path: str, model, engine=None, scheduler=None, strict: bool = True,
                        restore_rng: bool = False) -> Dict[str, Any]:
        path = self.resolve(path)
        ckpt = self.read(path)
        sd = next((ckpt[k] for k in MODEL_KEYS if k in ckpt), None)
        if sd is None:
            raise CheckpointError(f"{path}: no model state under any of {MODEL_KEYS}")
        mc = ckpt.get("model_config") or {}
        if hasattr(model, "config") and mc:
            for k in ARCH_KEYS:
                if k in mc and getattr(model.config, k, mc[k]) != mc[k]:
                    raise CheckpointError(f"architecture mismatch on {k}: checkpoint {mc[k]} vs model {getattr(model.config, k)}")
        if engine is not None and hasattr(engine, "gather_full_parameters"):
            engine.gather_full_parameters()
        target = next(p for p in model.parameters() if p.numel() > 0)
        res = model.load_state_dict({k: v.to(target.dtype) if v.is_floating_point() else v for k, v in sd.items()}, strict=strict)
        if engine is not None:
            osd = ckpt.get("optimizer_state_dict")
            if osd:
                ep = getattr(getattr(engine, "mesh", None), "coord", None)
                if ep is not None and engine.mesh.ep_size > 1:
                    pre = f"ep{ep.ep}:"
                    osd = dict(osd)
                    osd["state"] = {**osd["state"], **{k[len(pre):]: v for k, v in osd["state"].items() if k.startswith(pre)}}
                engine.load_state_dict(osd)
            else:
                engine.resync_master_from_params()
        if scheduler is not None and ckpt.get("scheduler_state_dict"):
            scheduler.load_state_dict(ckpt["scheduler_state_dict"])
        if restore_rng and ckpt.get("rng_state"):
            torch.set_rng_state(ckpt["rng_state"]["torch"])
        return {"path": path, "global_step": ckpt.get("global_step", 0), "epoch": ckpt.get("epoch", ckpt.get("current_epoch", 0)),
                "metrics": ckpt.get("metrics", {}), "missing_keys": list(getattr(res, "missing_keys", [])),
                "unexpected_keys": list(getattr(res, "unexpected_keys", []))}

    def emergency_save(self, model, engine=None, global_step: int = 0, epoch: int = 0) -> Optional[str]:
        try:
            return self.save_checkpoint(model, engine, None, global_step, epoch, suffix=f"emergency_{int(time.time())}")
        except Exception:
            return None

    def create_backup(self, path: str) -> Optional[str]:
        src = self.resolve(path)
        dst_dir = os.path.join(self.directory, "backups")
        os.makedirs(dst_dir, exist_ok=True)
        dst = os.path.join(dst_dir, time.strftime("%Y%m%d_%H%M%S_") + os.path.basename(src))
        shutil.copyfile(src, dst)
        return dst

    def list_checkpoints(self) -> List[Dict[str, Any]]:
        return [e for e in self.history if os.path.exists(e["path"])]

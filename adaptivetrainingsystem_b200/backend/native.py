from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch

from ..parallel.bootstrap import ProcessMesh, get_rank, init_distributed, world_size
from ..parallel.zero import ShardedEngine
from ..training.checkpoint import CheckpointManager
from ..training.schedulers import build_scheduler

FSDP_TO_STAGE = {"NO_SHARD": 0, "SHARD_GRAD_OP": 2, "FULL_SHARD": 3, "HYBRID_SHARD": 3}


class NativeBackend:
    def __init__(self, model, config, zero_stage: Optional[int] = None, mesh: Optional[ProcessMesh] = None, name: str = "native"):
        self.name, self.config = name, config
        init_distributed()
        self._model = model
        self.mesh = mesh or ProcessMesh(ep_size=1)
        stage = config.zero_stage if zero_stage is None else zero_stage
        fused = None
        if self.mesh.world > 1 and getattr(config, "fused_comm", True) and torch.cuda.is_available():
            from ..parallel.expert_parallel import attach_expert_parallel
            fused = attach_expert_parallel(model, self.mesh, config, use_fused=True)
        self.engine = ShardedEngine(model, lr=config.learning_rate, betas=(config.adam_beta1, config.adam_beta2), eps=config.adam_eps,
                                    weight_decay=config.weight_decay, max_grad_norm=config.max_grad_norm, zero_stage=min(stage, 2),
                                    mesh=self.mesh, fused_comm=fused, grad_accumulation_steps=config.gradient_accumulation_steps)
        self.scheduler = None
        self.checkpoints = CheckpointManager(config, os.path.join(config.output_dir, config.experiment_name or "run", "checkpoints"))
        self.global_step = 0

    # -- reference wrapper surface --------------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        return self._model(*args, **kwargs)

    def backward(self, loss: torch.Tensor) -> None:
        loss.backward()

    def step(self) -> Dict[str, Any]:
        out = self.engine.step()
        self.global_step += 1
        if self.scheduler is not None:
            self.engine.set_lr(self.scheduler.step())
        return out

    def zero_grad(self) -> None:
        self.engine.zero_grad()

    def train(self):
        self._model.train()
        return self

    def eval(self):
        self._model.eval()
        return self

    def setup_scheduler(self, total_steps: int) -> None:
        self.scheduler = build_scheduler(self.config, total_steps)
        self.engine.set_lr(self.scheduler.current_lr())

    def state_dict(self):
        return self._model.state_dict()

    def load_state_dict(self, sd, strict: bool = True):
        res = self._model.load_state_dict(sd, strict=strict)
        self.engine.resync_master_from_params()
        return res

    def get_lr(self) -> float:
        return self.engine.get_lr()

    def get_global_grad_norm(self) -> float:
        return self.engine.get_global_grad_norm()

    def save_checkpoint(self, directory: Optional[str] = None, tag: Optional[str] = None, epoch: int = 0):
        if directory:
            self.checkpoints.directory = directory
            self.checkpoints.history_file = os.path.join(directory, "checkpoint_history.json")
        return self.checkpoints.save_checkpoint(self._model, self.engine, self.scheduler, self.global_step, epoch, suffix=tag, mesh=self.mesh)

    def load_checkpoint(self, path: str = "latest", strict: bool = True):
        info = self.checkpoints.load_checkpoint(path, self._model, self.engine, self.scheduler, strict=strict)
        self.global_step = info["global_step"]
        return info

    @property
    def module(self):
        return self._model

    @property
    def world_size(self) -> int:
        return world_size()

    @property
    def local_rank(self) -> int:
        return int(os.environ.get("LOCAL_RANK", "0"))

    def is_main_process(self) -> bool:
        return get_rank() == 0

    def get_memory_stats(self) -> Dict[str, float]:
        out = {k + "_gb": v / 2 ** 30 for k, v in self.engine.memory_bytes().items()}
        if torch.cuda.is_available():
            out["allocated_gb"] = torch.cuda.memory_allocated() / 2 ** 30
            out["peak_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
        return out


def create_fsdp_backend(model, config) -> NativeBackend:
    return NativeBackend(model, config, FSDP_TO_STAGE.get(getattr(config, "fsdp_sharding_strategy", "FULL_SHARD"), 3), name="fsdp")


def create_deepspeed_backend(model, config) -> NativeBackend:
    return NativeBackend(model, config, config.zero_stage, name="deepspeed")


def create_colossalai_backend(model, config, plugin: str = "low_level_zero") -> NativeBackend:
    return NativeBackend(model, config, 3 if plugin == "gemini" else max(config.zero_stage, 1), name="colossalai")


def create_backend(model, config) -> NativeBackend:
    kind = getattr(config, "backend", "native")
    return {"fsdp": create_fsdp_backend, "deepspeed": create_deepspeed_backend, "colossalai": create_colossalai_backend}.get(
        kind, lambda m, c: NativeBackend(m, c))(model, config)

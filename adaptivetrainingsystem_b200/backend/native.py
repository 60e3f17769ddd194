"""Uniform backend wrapper (reference ``backend/backend_fsdp.py:311-616``, ``backend_deepspeed.py:211-467``,
``backend_colossalai.py:79-141``): ``__call__ / backward / step / zero_grad / train / eval / state_dict / load_state_dict /
get_lr / get_global_grad_norm / save_checkpoint / load_checkpoint / module / world_size / local_rank / is_main_process /
get_memory_stats``.  The three factory names of the reference select a sharding stage of the native engines:

* FSDP ``FULL_SHARD`` / ``HYBRID_SHARD``, DeepSpeed ``zero_stage=3`` and the ColossalAI ``gemini`` plugin build
  :class:`~adaptivetrainingsystem_b200.parallel.zero3.ZeRO3Engine` (parameters, gradients and optimiser state sharded);
* ``SHARD_GRAD_OP`` / stage 1-2 / ``low_level_zero`` build :class:`~adaptivetrainingsystem_b200.parallel.zero.ShardedEngine`
  (replicated bf16 parameters, sharded fp32 master weights and moments, fused peer-memory step);
* ``NO_SHARD`` / stage 0 is bucketed data parallelism.

Expert-parallel models keep their experts partitioned by expert parallelism and run the dense part at stage <= 2 (a stage-3
request is downgraded with a warning, never silently).
"""
from __future__ import annotations

import logging
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
        opt = dict(lr=config.learning_rate, betas=(config.adam_beta1, config.adam_beta2), eps=config.adam_eps,
                   weight_decay=config.weight_decay, max_grad_norm=config.max_grad_norm, mesh=self.mesh,
                   grad_accumulation_steps=config.gradient_accumulation_steps)
        self.requested_stage = stage
        if stage >= 3 and self.mesh.ep_size == 1 and self.mesh.world > 1:
            from ..parallel.zero3 import ZeRO3Engine
            self.engine = ZeRO3Engine(model, fused_comm=fused, **opt)
        else:
            if stage >= 3:
                why = "one process" if self.mesh.world == 1 else f"expert parallelism (ep={self.mesh.ep_size}) partitions the experts"
                logging.getLogger(__name__).warning("%s backend: stage 3 requested, running stage 2 (%s)", name, why)
            self.engine = ShardedEngine(model, zero_stage=min(stage, 2), fused_comm=fused, **opt)
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

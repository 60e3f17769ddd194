"""Process-group bootstrap and the rank mesh.

One process per GPU; ``torch.distributed`` (NCCL on CUDA, Gloo on CPU) provides rendezvous, barriers and the
baseline collectives.  The mesh factors the world into pipeline x data x expert axes and hands out cached
process groups per axis (the role of ``ProcessGroupMesh`` / ``DistCoordinator`` in the reference's vendored
tree, ``colossalai/cluster/process_group_mesh.py:24-260``, ``dist_coordinator.py:40-201``; first-party bootstrap
``backend/backend_fsdp.py:102-116``).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


def env_rank_info() -> Tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> Tuple[int, int, int]:
    """Initialise the default process group from the launcher's environment (``env://``).  Returns
    ``(rank, local_rank, world_size)``; a single process without launcher variables needs no group."""
    rank, local_rank, world = env_rank_info()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, init_method="env://", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, local_rank, world


def shutdown() -> None:
    if dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()


def world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def get_rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def is_main_process() -> bool:
    return get_rank() == 0


def barrier(group=None) -> None:
    if dist.is_initialized():
        dist.barrier(group)


@dataclass
class MeshCoord:
    pp: int
    dp: int
    ep: int
    tp: int = 0
    sp: int = 0


class ProcessMesh:
    """World = pp x dp_outer x ep x sp x tp (tp fastest).  Expert parallelism lives inside data parallelism: the ``ep`` ranks
    of one group hold different experts and the same dense weights.  Sequence-parallel ranks hold the same weights and
    different parts of every sequence, so for gradient averaging they count as data parallelism too.  Groups:

    ``tp``   tensor-parallel ranks (sharded attention heads / FFN columns; activations all-reduced)
    ``sp``   sequence-parallel ranks (head-scatter all-to-all around attention)
    ``ep``   expert-parallel ranks
    ``edp``  ranks that hold the same experts (gradient averaging of expert weights): dp_outer x sp
    ``dp``   ranks that hold the same dense weights (gradient averaging / ZeRO sharding): dp_outer x ep x sp
    ``pp``   pipeline stages

    (the role of ``ProcessGroupMesh`` in the reference's vendored tree, ``colossalai/cluster/process_group_mesh.py:24-260``)."""

    AXES = ("dp", "ep", "edp", "pp", "tp", "sp")

    def __init__(self, world: Optional[int] = None, rank: Optional[int] = None, pp_size: int = 1, ep_size: int = 1,
                 create_groups: bool = True, tp_size: int = 1, sp_size: int = 1):
        self.world = world if world is not None else world_size()
        self.rank = rank if rank is not None else get_rank()
        inner = pp_size * ep_size * tp_size * sp_size
        if self.world % inner:
            raise ValueError(f"world size {self.world} not divisible by pp*ep*sp*tp = {inner}")
        self.pp_size, self.ep_size, self.tp_size, self.sp_size = pp_size, ep_size, tp_size, sp_size
        self.dp_outer = self.world // inner
        self.dp_size = self.dp_outer * ep_size * sp_size
        self.coord = self.coord_of(self.rank)
        self._groups: Dict[str, Optional[dist.ProcessGroup]] = {a: None for a in self.AXES}
        self._ranks: Dict[str, List[int]] = {}
        if create_groups:
            self._build_groups()

    def coord_of(self, rank: int) -> MeshCoord:
        tp = rank % self.tp_size
        rank //= self.tp_size
        sp = rank % self.sp_size
        rank //= self.sp_size
        ep = rank % self.ep_size
        rank //= self.ep_size
        dp = rank % self.dp_outer
        pp = rank // self.dp_outer
        return MeshCoord(pp, dp, ep, tp, sp)

    def rank_of(self, pp: int, dp: int, ep: int, tp: int = 0, sp: int = 0) -> int:
        return (((pp * self.dp_outer + dp) * self.ep_size + ep) * self.sp_size + sp) * self.tp_size + tp

    def ranks_along(self, axis: str, rank: Optional[int] = None) -> List[int]:
        c = self.coord_of(self.rank if rank is None else rank)
        if axis == "tp":
            return [self.rank_of(c.pp, c.dp, c.ep, t, c.sp) for t in range(self.tp_size)]
        if axis == "sp":
            return [self.rank_of(c.pp, c.dp, c.ep, c.tp, s) for s in range(self.sp_size)]
        if axis == "ep":
            return [self.rank_of(c.pp, c.dp, e, c.tp, c.sp) for e in range(self.ep_size)]
        if axis == "edp":
            return [self.rank_of(c.pp, d, c.ep, c.tp, s) for d in range(self.dp_outer) for s in range(self.sp_size)]
        if axis == "dp":
            return [self.rank_of(c.pp, d, e, c.tp, s) for d in range(self.dp_outer) for e in range(self.ep_size) for s in range(self.sp_size)]
        if axis == "pp":
            return [self.rank_of(p, c.dp, c.ep, c.tp, c.sp) for p in range(self.pp_size)]
        raise KeyError(axis)

    def _build_groups(self) -> None:
        for axis in self.AXES:
            self._ranks[axis] = self.ranks_along(axis)
            if not dist.is_initialized() or self.world == 1:
                continue
            seen = set()
            for r in range(self.world):  # every rank must create every group, in the same order
                ranks = tuple(self.ranks_along(axis, r))
                if ranks in seen:
                    continue
                seen.add(ranks)
                if sorted(ranks) == list(range(self.world)):
                    g = dist.group.WORLD
                elif len(ranks) == 1:
                    g = None
                else:
                    g = dist.new_group(list(ranks))
                if self.rank in ranks:
                    self._groups[axis] = g

    def group(self, axis: str):
        return self._groups[axis]

    def size(self, axis: str) -> int:
        return {"dp": self.dp_size, "ep": self.ep_size, "edp": self.dp_outer * self.sp_size, "pp": self.pp_size, "tp": self.tp_size,
                "sp": self.sp_size}[axis]

    def index(self, axis: str) -> int:
        return self.ranks_along(axis).index(self.rank)

    @property
    def is_first_stage(self) -> bool:
        return self.coord.pp == 0

    @property
    def is_last_stage(self) -> bool:
        return self.coord.pp == self.pp_size - 1

    def describe(self) -> str:
        parts = []
        if self.pp_size > 1:
            parts.append(f"pp{self.pp_size}")
        if self.tp_size > 1:
            parts.append(f"tp{self.tp_size}")
        if self.sp_size > 1:
            parts.append(f"sp{self.sp_size}")
        if self.ep_size > 1:
            parts.append(f"ep{self.ep_size}")
        parts.append(f"dp{self.dp_size}")
        return "+".join(parts)

    @classmethod
    def from_config(cls, config, world: Optional[int] = None, rank: Optional[int] = None, create_groups: bool = True) -> "ProcessMesh":
        """The mesh that ``Config.pipeline_parallel_size / tensor_parallel_size / sequence_parallel_size / expert_parallel_size``
        ask for (the reference reaches these through one plugin object, ``colossalai/booster/plugin/hybrid_parallel_plugin.py:880-1110``)."""
        w = world if world is not None else world_size()
        pp = max(int(getattr(config, "pipeline_parallel_size", 1) or 1), 1)
        tp = max(int(getattr(config, "tensor_parallel_size", 1) or 1), 1)
        sp = max(int(getattr(config, "sequence_parallel_size", 1) or 1), 1)
        ep = int(getattr(config, "expert_parallel_size", 1) or 1) if getattr(config, "use_moe", False) else 1
        rest = max(w // (pp * tp * sp), 1)
        import math
        ep = math.gcd(max(ep, 1), rest)
        return cls(w, rank, pp_size=pp, ep_size=ep, create_groups=create_groups, tp_size=tp, sp_size=sp)

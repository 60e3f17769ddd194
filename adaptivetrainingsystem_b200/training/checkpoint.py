"""Checkpoint manager: a single-file interchange format with the reference's schema and names, and a sharded format
for models whose state does not fit one host; history, retention, best link, backup and emergency save.

Single file (reference ``training/checkpoint.py:51-70`` and ``training/trainer.py:3395-3422``)::

    {model_state_dict, optimizer_state_dict, scheduler_state_dict | None, global_step, epoch | current_epoch,
     metrics, config (dict), model_config {vocab_size, hidden_size, num_layers, num_heads, num_kv_heads, seq_length,
     intermediate_size, ...}, save_time, pytorch_version, rng_state}

``model_state_dict`` uses the reference parameter names (``layers.N.self_attn.q_proj.weight`` ...).  The RNG state is
saved (the reference README promises it, its code does not).  Loading accepts the key aliases
``module | model_state_dict | state_dict | model`` (reference ``Chat.py:150``).  Only rank 0 ever holds the gathered
state: every rank sends the optimiser state it owns (its ZeRO shard, its experts) to rank 0 and nothing else moves.

Sharded directory (the role of the reference's vendored ``colossalai/checkpoint_io/hybrid_parallel_checkpoint_io.py`` and
``colossalai/moe/checkpoint.py:163-275``: per-rank shards plus an index)::

    <name>/index.json              what is where: files, the experts each file holds, every optimiser piece
    <name>/model_dense.pt          non-expert weights, reference names (rank 0)
    <name>/model_experts_epK.pt    the experts of expert-parallel coordinate K, reference names
    <name>/optim_rankR.pt          the optimiser state that rank R owns (fp32 master / moments of its shard)
    <name>/meta.pt                 scheduler, counters, metrics, configs, RNG (rank 0)

Optimiser state is addressed in both formats by *global pieces*: ``(key, first element, length)`` with ``key`` the
parameter name, or ``name#E`` for the slice of a stacked expert parameter that belongs to global expert ``E``.  A load
therefore re-shards for any data-parallel and expert-parallel layout: every rank asks for the stretches it owns now.
"""
from __future__ import annotations

import json
import os
import shutil
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

MODEL_KEYS = ("model_state_dict", "module", "state_dict", "model")
ARCH_KEYS = ("vocab_size", "hidden_size", "num_layers", "num_heads")
STATE_KEYS = ("master", "exp_avg", "exp_avg_sq")
SHARDED_FORMAT = "ats-sharded-v1"


class CheckpointError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------------------------------
# global pieces
# ------------------------------------------------------------------------------------------------------------------
def _ep_layout(engine) -> Tuple[int, int]:
    mesh = getattr(engine, "mesh", None)
    if mesh is None or getattr(mesh, "ep_size", 1) <= 1:
        return 1, 0
    return mesh.ep_size, mesh.coord.ep


def _split_global(piece: Dict[str, Any], ep_rank: int) -> List[Tuple[str, Tuple[int, ...], int, int, int]]:
    """A stretch of a (local) parameter -> [(global key, shape of that key's tensor, first element inside it, length,
    offset of this part inside the stretch)].  Stacked expert parameters are cut at expert boundaries and named by the
    GLOBAL expert index, so the naming does not depend on the expert-parallel layout that wrote it."""
    name, shape, start, length = piece["name"], tuple(piece["shape"]), piece["start"], piece["length"]
    if not piece.get("expert"):
        return [(name, shape, start, length, 0)]
    e_local = shape[0]
    per = 1
    for d in shape[1:]:
        per *= d
    out, pos, end = [], start, start + length
    while pos < end:
        e = pos // per
        stop = min(end, (e + 1) * per)
        out.append((f"{name}#{ep_rank * e_local + e}", shape[1:], pos - e * per, stop - pos, pos - start))
        pos = stop
    return out


def collect_pieces(engine) -> List[Dict[str, Any]]:
    """The optimiser state this rank owns as CPU pieces ``{key, shape, start, length, master, exp_avg, exp_avg_sq}``."""
    _, ep_rank = _ep_layout(engine)
    out = []
    for piece in engine.owned_pieces(unique=True):
        for key, shape, first, length, off in _split_global(piece, ep_rank):
            rec = {"key": key, "shape": tuple(shape), "start": first, "length": length}
            for k in STATE_KEYS:
                rec[k] = piece["tensors"][k][off:off + length].detach().to("cpu", copy=True)
            out.append(rec)
    return out


class _PieceIndex:
    """Look-up of saved pieces by key and range, over one or several sources that are read on demand."""

    def __init__(self):
        self.by_key: Dict[str, List[Tuple[int, int, Callable[[], Dict[str, torch.Tensor]]]]] = {}

    def add(self, key: str, start: int, length: int, getter: Callable[[], Dict[str, torch.Tensor]]) -> None:
        self.by_key.setdefault(key, []).append((start, length, getter))

    def fetch(self, key: str, start: int, length: int) -> Optional[Dict[str, torch.Tensor]]:
        """The three state vectors of [start, start + length) of ``key`` assembled from the saved pieces that overlap it;
        ``None`` unless the range is covered completely."""
        entries = self.by_key.get(key)
        if not entries:
            return None
        out = {k: torch.empty(length, dtype=torch.float32) for k in STATE_KEYS}
        covered = 0
        for s, n, getter in entries:
            a, b = max(s, start), min(s + n, start + length)
            if b <= a:
                continue
            src = getter()
            for k in STATE_KEYS:
                out[k][a - start:b - start] = src[k].reshape(-1)[a - s:b - s].float()
            covered += b - a
        return out if covered == length else None


def _fetcher(index: _PieceIndex, ep_rank: int, legacy_state: Optional[Dict[str, Any]] = None):
    """``fetch(piece)`` for :meth:`load_pieces` of the engines."""
    def fetch(piece: Dict[str, Any]) -> Optional[Dict[str, torch.Tensor]]:
        parts = _split_global(piece, ep_rank)
        out = {k: torch.empty(piece["length"], dtype=torch.float32) for k in STATE_KEYS}
        for key, _shape, first, length, off in parts:
            got = index.fetch(key, first, length)
            if got is None:
                break
            for k in STATE_KEYS:
                out[k][off:off + length] = got[k]
        else:
            return out
        if legacy_state is not None:  # files written before pieces existed: whole local tensors under the parameter name
            st = legacy_state.get(f"ep{ep_rank}:{piece['name']}") or legacy_state.get(piece["name"])
            if st is not None and st["master"].numel() >= piece["start"] + piece["length"]:
                return {k: st[k].reshape(-1)[piece["start"]:piece["start"] + piece["length"]] for k in STATE_KEYS}
        return None
    return fetch


def _assemble(pieces: List[Dict[str, Any]]) -> Dict[str, Dict[str, torch.Tensor]]:
    """Pieces of all ranks -> ``{key: {master, exp_avg, exp_avg_sq}}`` in full shapes (rank 0 of a single-file save)."""
    state: Dict[str, Dict[str, torch.Tensor]] = {}
    for rec in pieces:
        shape = tuple(rec["shape"])
        n = 1
        for d in shape:
            n *= d
        st = state.get(rec["key"])
        if st is None:
            st = {k: torch.zeros(n, dtype=torch.float32) for k in STATE_KEYS}
            state[rec["key"]] = st
        for k in STATE_KEYS:
            st[k][rec["start"]:rec["start"] + rec["length"]] = rec[k].float()
    for key, st in state.items():
        shape = next(tuple(r["shape"]) for r in pieces if r["key"] == key)
        for k in STATE_KEYS:
            st[k] = st[k].view(shape)
    return state


def _all_ok(ok: bool, err: str = "") -> None:
    """Every rank learns whether the writer succeeded; nobody is left waiting in a barrier for a rank that raised."""
    if dist.is_initialized():
        box = [(ok, err)] if dist.get_rank() == 0 else [None]
        dist.broadcast_object_list(box, src=0)
        ok, err = box[0]
    if not ok:
        raise CheckpointError(f"checkpoint write failed on rank 0: {err}")


class CheckpointManager:
    def __init__(self, config, directory: str = "checkpoints"):
        self.config = config
        self.directory = directory
        self.history_file = os.path.join(directory, "checkpoint_history.json")
        self.history: List[Dict[str, Any]] = []
        self.best_metric = float("inf")
        # further metadata of the owner, merged into every checkpoint (the trainer adds ``precision_info`` and
        # ``quantization_info``, the keys of the reference's live format, ``training/trainer.py:3395-3422``)
        self.extra_meta = None
        if os.path.exists(self.history_file):
            try:
                with open(self.history_file) as f:
                    self.history = json.load(f)
            except Exception:
                self.history = []
        losses = [e["eval_loss"] for e in self.history if e.get("eval_loss") is not None]
        if losses:  # resume: "best so far" continues from the recorded history instead of starting at infinity
            self.best_metric = min(losses)

    # -- gather helpers -------------------------------------------------------------------------------------
    @staticmethod
    def _gather_model_state(model, mesh, dst_only: bool = False) -> Optional[Dict[str, torch.Tensor]]:
        """The full model state: expert-parallel ranks contribute their own experts.  With ``dst_only`` just global rank 0
        receives the experts of the other ranks of its expert-parallel group (the others return ``None``)."""
        sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        if mesh is not None and mesh.ep_size > 1 and dist.is_initialized():
            mine = {k: v for k, v in sd.items() if ".ffn.experts." in k}
            if dst_only:
                ranks = mesh.ranks_along("ep")
                if 0 in ranks:  # the expert-parallel group that contains the writer
                    parts: Optional[List[Any]] = [None] * mesh.ep_size if dist.get_rank() == 0 else None
                    dist.gather_object(mine, parts, dst=0, group=mesh.group("ep"))
                    for p in parts or []:
                        sd.update(p or {})
                return sd if dist.get_rank() == 0 else None
            parts = [None] * mesh.ep_size
            dist.all_gather_object(parts, mine, group=mesh.group("ep"))
            for p in parts:
                sd.update(p or {})
        return sd

    def _use_sharded(self, model, sharded: Optional[bool]) -> bool:
        if sharded is not None:
            return bool(sharded)
        cfg = getattr(self.config, "sharded_checkpoint", None)
        if cfg is not None:
            return bool(cfg)
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return False
        # fp32 master + two moments of every parameter on one host: beyond ~2 B parameters write shards
        n = sum(p.numel() for p in model.parameters()) if hasattr(model, "parameters") else 0
        return n * (dist.get_world_size() if getattr(model, "ep_size", 1) > 1 else 1) > 2_000_000_000

    def _meta(self, model, scheduler, global_step, epoch, metrics) -> Dict[str, Any]:
        extra = self.extra_meta() if callable(self.extra_meta) else {}
        return {
            **extra,
            "scheduler_state_dict": scheduler.state_dict() if scheduler is not None else None,
            "global_step": global_step, "epoch": epoch, "current_epoch": epoch,
            "metrics": {k: list(v)[-1000:] for k, v in (metrics or {}).items()},
            "config": self.config.to_dict() if hasattr(self.config, "to_dict") else dict(vars(self.config)),
            "model_config": model.config.to_dict() if hasattr(model, "config") else {},
            "save_time": time.time(), "pytorch_version": torch.__version__,
            "rng_state": {"torch": torch.get_rng_state(),
                          "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None},
        }

    def save_checkpoint(self, model, engine=None, scheduler=None, global_step: int = 0, epoch: int = 0,
                        metrics: Optional[Dict[str, Any]] = None, suffix: Optional[str] = None, mesh=None,
                        is_best: bool = False, eval_loss: Optional[float] = None, sharded: Optional[bool] = None) -> Optional[str]:
        if self._use_sharded(model, sharded):
            return self.save_sharded(model, engine, scheduler, global_step, epoch, metrics, suffix, mesh, is_best, eval_loss)
        rank = dist.get_rank() if dist.is_initialized() else 0
        multi = dist.is_initialized() and dist.get_world_size() > 1
        if engine is not None and hasattr(engine, "gather_full_parameters"):
            engine.gather_full_parameters()  # ZeRO-3: materialise every block for the state dict
        model_sd = self._gather_model_state(model, mesh, dst_only=True)
        if engine is not None and hasattr(engine, "release_parameters"):
            engine.release_parameters()
        opt_sd = None
        if engine is not None and getattr(self.config, "save_optimizer_states", True):
            mine = collect_pieces(engine)  # this rank's shard only; nothing is all-gathered
            if multi:
                parts: Optional[List[Any]] = [None] * dist.get_world_size() if rank == 0 else None
                dist.gather_object(mine, parts, dst=0)
                mine = [rec for p in (parts or []) for rec in (p or [])]
            if rank == 0:
                opt_sd = {"state": _assemble(mine), "step": engine.step_count, "hyper": list(engine._hyper_host),
                          "zero_stage": engine.zero_stage, "format": "pieces"}
        path, ok, err = None, True, ""
        if rank == 0:
            try:
                os.makedirs(self.directory, exist_ok=True)
                name = f"checkpoint_{suffix}.pt" if suffix else f"checkpoint_epoch_{epoch:03d}_step_{global_step:06d}.pt"
                path = os.path.join(self.directory, name)
                payload = {"model_state_dict": model_sd, "optimizer_state_dict": opt_sd,
                           **self._meta(model, scheduler, global_step, epoch, metrics)}
                tmp = path + ".tmp"
                torch.save(payload, tmp)
                os.replace(tmp, path)
                self._record(path, global_step, epoch, payload["save_time"], eval_loss, suffix, is_best)
            except Exception as e:  # the other ranks must not wait for a writer that raised
                ok, err = False, repr(e)
        if multi:
            _all_ok(ok, err)
        elif not ok:
            raise CheckpointError(f"checkpoint write failed: {err}")
        return path

    # -- sharded format ------------------------------------------------------------------------------------------
    def save_sharded(self, model, engine=None, scheduler=None, global_step: int = 0, epoch: int = 0,
                     metrics: Optional[Dict[str, Any]] = None, suffix: Optional[str] = None, mesh=None,
                     is_best: bool = False, eval_loss: Optional[float] = None) -> Optional[str]:
        """Every rank writes what it owns; rank 0 adds the dense weights, the bookkeeping and the index.  No rank ever holds
        more than its own shard, so a 47 B-parameter expert-parallel model saves without a gather."""
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        multi = world > 1
        name = f"checkpoint_{suffix}" if suffix else f"checkpoint_epoch_{epoch:03d}_step_{global_step:06d}"
        path = os.path.join(self.directory, name)
        ok, err = True, ""
        if rank == 0:
            try:
                if os.path.isdir(path):
                    shutil.rmtree(path)
                os.makedirs(path, exist_ok=True)
            except Exception as e:
                ok, err = False, repr(e)
        if multi:
            _all_ok(ok, err)
        elif not ok:
            raise CheckpointError(err)
        ep_size = mesh.ep_size if mesh is not None else 1
        ep_rank = mesh.coord.ep if mesh is not None else 0
        first_replica = mesh is None or mesh.coord.dp == 0  # one writer per expert-parallel coordinate
        if engine is not None and hasattr(engine, "gather_full_parameters"):
            engine.gather_full_parameters()
        sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        if engine is not None and hasattr(engine, "release_parameters"):
            engine.release_parameters()
        experts = {k: v for k, v in sd.items() if ".ffn.experts." in k} if ep_size > 1 else {}
        local = {"rank": rank, "pieces": [], "expert_file": None, "expert_ids": []}
        try:
            if experts and first_replica:
                fn = f"model_experts_ep{ep_rank}.pt"
                torch.save(experts, os.path.join(path, fn))
                ids = sorted({int(k.split(".ffn.experts.")[1].split(".")[0]) for k in experts})
                local["expert_file"], local["expert_ids"] = fn, ids
            if engine is not None and getattr(self.config, "save_optimizer_states", True):
                mine = collect_pieces(engine)
                fn = f"optim_rank{rank:05d}.pt"
                torch.save(mine, os.path.join(path, fn))
                local["pieces"] = [[r["key"], list(r["shape"]), r["start"], r["length"], fn, i] for i, r in enumerate(mine)]
            if rank == 0:
                dense = {k: v for k, v in sd.items() if k not in experts}
                torch.save(dense, os.path.join(path, "model_dense.pt"))
                torch.save(self._meta(model, scheduler, global_step, epoch, metrics), os.path.join(path, "meta.pt"))
        except Exception as e:
            local["error"] = repr(e)
        infos: List[Any] = [local]
        if multi:
            infos = [None] * world if rank == 0 else None
            dist.gather_object(local, infos, dst=0)
        if rank == 0:
            try:
                bad = [i for i in infos if i and i.get("error")]
                if bad:
                    raise CheckpointError(f"rank {bad[0]['rank']}: {bad[0]['error']}")
                index = {"format": SHARDED_FORMAT, "world_size": world, "ep_size": ep_size, "global_step": global_step, "epoch": epoch,
                         "step": getattr(engine, "step_count", 0) if engine is not None else 0,
                         "hyper": list(getattr(engine, "_hyper_host", [])) if engine is not None else [],
                         "zero_stage": getattr(engine, "zero_stage", 0) if engine is not None else 0,
                         "dense_file": "model_dense.pt", "meta_file": "meta.pt",
                         "expert_files": {i["expert_file"]: i["expert_ids"] for i in infos if i and i["expert_file"]},
                         "pieces": [p for i in infos if i for p in i["pieces"]]}
                with open(os.path.join(path, "index.json.tmp"), "w") as f:
                    json.dump(index, f)
                os.replace(os.path.join(path, "index.json.tmp"), os.path.join(path, "index.json"))
                self._record(path, global_step, epoch, time.time(), eval_loss, suffix, is_best)
            except Exception as e:
                ok, err = False, repr(e)
        if multi:
            _all_ok(ok, err)
        elif not ok:
            raise CheckpointError(err)
        return path if rank == 0 else None

    def _load_sharded(self, path: str, model, engine, scheduler, strict: bool, restore_rng: bool) -> Dict[str, Any]:
        try:
            with open(os.path.join(path, "index.json")) as f:
                index = json.load(f)
        except Exception as e:
            raise CheckpointError(f"cannot read checkpoint index in {path}: {e}") from e
        if index.get("format") != SHARDED_FORMAT:
            raise CheckpointError(f"{path}: unknown sharded format {index.get('format')!r}")
        meta = self.read(os.path.join(path, index["meta_file"]))
        self._check_arch(model, meta.get("model_config") or {})
        sd = self.read(os.path.join(path, index["dense_file"]))
        ep_size, ep_rank = getattr(model, "ep_size", 1), getattr(model, "ep_rank", 0)
        want = set()
        for layer in (model.get_moe_layers() if hasattr(model, "get_moe_layers") else []):
            e_local = layer.experts_w1.shape[0]
            want.update(range(ep_rank * e_local, (ep_rank + 1) * e_local))
        for fn, ids in index.get("expert_files", {}).items():
            if want & set(ids):
                part = self.read(os.path.join(path, fn))
                sd.update({k: v for k, v in part.items() if int(k.split(".ffn.experts.")[1].split(".")[0]) in want})
        res = self._load_model(model, engine, sd, strict)
        if engine is not None:
            if index.get("pieces"):
                cache: Dict[str, Any] = {}
                pidx = _PieceIndex()

                def getter(fn: str, i: int):
                    def get():
                        if fn not in cache:
                            cache.clear()  # one shard file in memory at a time
                            cache[fn] = self.read(os.path.join(path, fn))
                        return cache[fn][i]
                    return get
                for key, _shape, start, length, fn, i in sorted(index["pieces"], key=lambda p: (p[4], p[5])):
                    pidx.add(key, start, length, getter(fn, i))
                n = engine.load_pieces(_fetcher(pidx, ep_rank), step=index.get("step"), hyper=index.get("hyper") or None)
                if n == 0:
                    engine.resync_master_from_params()
                elif hasattr(engine, "release_parameters"):
                    engine.release_parameters()
            else:
                engine.resync_master_from_params()
        if scheduler is not None and meta.get("scheduler_state_dict"):
            scheduler.load_state_dict(meta["scheduler_state_dict"])
        if restore_rng and meta.get("rng_state"):
            torch.set_rng_state(meta["rng_state"]["torch"])
        return {"path": path, "global_step": meta.get("global_step", 0), "epoch": meta.get("epoch", 0), "metrics": meta.get("metrics", {}),
                "missing_keys": list(getattr(res, "missing_keys", [])), "unexpected_keys": list(getattr(res, "unexpected_keys", [])),
                "sharded": True}

    # -- bookkeeping ------------------------------------------------------------------------------------------------
    def _record(self, path, global_step, epoch, save_time, eval_loss, suffix, is_best) -> None:
        entry = {"path": path, "global_step": global_step, "epoch": epoch, "save_time": save_time,
                 "eval_loss": eval_loss, "suffix": suffix}
        self.history.append(entry)
        if is_best or (eval_loss is not None and eval_loss < self.best_metric):
            self.best_metric = eval_loss if eval_loss is not None else self.best_metric
            self._link_best(path)
        self._enforce_retention()
        self._write_history()

    def _link_best(self, path: str) -> None:
        best = os.path.join(self.directory, "best_checkpoint.pt")
        try:
            if os.path.lexists(best):
                os.remove(best)
            os.symlink(os.path.basename(path), best)
        except OSError:
            if os.path.isdir(path):
                shutil.copytree(path, best)
            else:
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
                if os.path.isdir(victim["path"]):
                    shutil.rmtree(victim["path"])
                else:
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
            if not cands and os.path.isdir(self.directory):
                def is_ckpt(f):
                    full = os.path.join(self.directory, f)
                    return f.startswith("checkpoint_") and (f.endswith(".pt") or os.path.exists(os.path.join(full, "index.json")))
                cands = sorted((os.path.join(self.directory, f) for f in os.listdir(self.directory) if is_ckpt(f)), key=os.path.getmtime)
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

    @staticmethod
    def _check_arch(model, mc: Dict[str, Any]) -> None:
        if hasattr(model, "config") and mc:
            for k in ARCH_KEYS:
                if k in mc and getattr(model.config, k, mc[k]) != mc[k]:
                    raise CheckpointError(f"architecture mismatch on {k}: checkpoint {mc[k]} vs model {getattr(model.config, k)}")

    @staticmethod
    def _load_model(model, engine, sd: Dict[str, torch.Tensor], strict: bool):
        if engine is not None and hasattr(engine, "gather_full_parameters"):
            engine.gather_full_parameters()
        target = next(p for p in model.parameters() if p.numel() > 0)
        return model.load_state_dict({k: v.to(target.dtype) if v.is_floating_point() else v for k, v in sd.items()}, strict=strict)

    def load_checkpoint(self, path: str, model, engine=None, scheduler=None, strict: bool = True,
                        restore_rng: bool = False) -> Dict[str, Any]:
        path = self.resolve(path)
        if os.path.isdir(path):
            return self._load_sharded(path, model, engine, scheduler, strict, restore_rng)
        ckpt = self.read(path)
        sd = next((ckpt[k] for k in MODEL_KEYS if k in ckpt), None)
        if sd is None:
            raise CheckpointError(f"{path}: no model state under any of {MODEL_KEYS}")
        self._check_arch(model, ckpt.get("model_config") or {})
        res = self._load_model(model, engine, sd, strict)
        if engine is not None:
            osd = ckpt.get("optimizer_state_dict")
            if osd and osd.get("state"):
                _, ep_rank = _ep_layout(engine)
                pidx = _PieceIndex()
                for key, st in osd["state"].items():
                    if "master" in st:
                        pidx.add(key, 0, st["master"].numel(), lambda st=st: st)
                n = engine.load_pieces(_fetcher(pidx, ep_rank, legacy_state=osd["state"]), step=osd.get("step", 0), hyper=osd.get("hyper"))
                if n == 0:
                    engine.resync_master_from_params()
                elif hasattr(engine, "release_parameters"):
                    engine.release_parameters()
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
        if os.path.isdir(src):
            shutil.copytree(src, dst)
        else:
            shutil.copyfile(src, dst)
        return dst

    def list_checkpoints(self) -> List[Dict[str, Any]]:
        return [e for e in self.history if os.path.exists(e["path"])]

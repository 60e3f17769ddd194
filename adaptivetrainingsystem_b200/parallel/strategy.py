"""Parallel strategies as properties of a run, not of a code path: the mesh that ``Config`` asks for, and the in-place
conversions that make one ``DeepSeekTransformer`` tensor-parallel, sequence-parallel or a pipeline stage.

The reference reaches these through one plugin object of its vendored tree (``colossalai/booster/plugin/hybrid_parallel_plugin.py:880-1110``;
sharded layers ``shardformer/layer/linear.py:190-442``, head-scatter sequence parallelism ``shardformer/modeling/llama.py:503-540``,
stage partition ``pipeline/stage_manager.py:11-239``).  Here:

* ``apply_tensor_parallel``: attention heads and FFN columns are split over the ``tp`` group.  ``qkv_proj`` keeps this rank's query
  and KV heads, ``o_proj`` / ``down_proj`` their input columns, ``gate_up_proj`` its gate and up rows; the block input enters
  through an identity whose backward all-reduces, the row-parallel outputs are all-reduced before the residual is added.
* ``apply_sequence_parallel``: every rank of the ``sp`` group holds ``L / W`` tokens of every sequence; attention exchanges heads
  for tokens with an all-to-all on both sides (positions of the rotary embedding are global).
* ``PipelineStage`` / ``InterleavedStages`` (``parallel/pipeline.py``) own a slice of the layers and free the rest.

``EnhancedConversationTrainer`` applies them from the mesh it is given (``ProcessMesh.from_config``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def _shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].clone()


def _shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n].clone()


@torch.no_grad()
def apply_tensor_parallel(model, mesh) -> None:
    """Shard every attention module and every dense SwiGLU FFN of ``model`` over ``mesh.group('tp')`` in place.  MoE and MoD
    FFNs stay replicated inside a tensor-parallel group (every rank computes the same tokens)."""
    W, r, group = mesh.tp_size, mesh.coord.tp, mesh.group("tp")
    if W <= 1:
        return
    cfg = model.config
    if cfg.num_heads % W or cfg.num_kv_heads % W or cfg.intermediate_size % W:
        raise ValueError(f"tensor_parallel_size {W} must divide num_heads ({cfg.num_heads}), num_kv_heads ({cfg.num_kv_heads}) and "
                         f"intermediate_size ({cfg.intermediate_size})")
    d = cfg.head_dim
    for blk in model.layers:
        att = blk.self_attn
        if getattr(att, "tp_group", None) is None:
            nq, nk = att.n_q * d, att.n_kv * d
            qkv = att.qkv_proj.data
            parts = [_shard_rows(qkv[:nq], r, W), _shard_rows(qkv[nq:nq + nk], r, W), _shard_rows(qkv[nq + nk:], r, W)]
            att.qkv_proj = nn.Parameter(torch.cat(parts, dim=0))
            att.o_proj = nn.Parameter(_shard_cols(att.o_proj.data, r, W))
            att.n_q, att.n_kv = att.n_q // W, att.n_kv // W
            att.tp_group, att.tp_size, att.tp_rank = group, W, r
            att.qkv_proj._ats_tp = ("qkv", W, r)
            att.o_proj._ats_tp = ("col", W, r)
        ffn = blk.ffn
        if blk.ffn_kind == "dense" and getattr(ffn, "tp_group", None) is None:
            inter = ffn.gate_up_proj.shape[0] // 2
            gu = ffn.gate_up_proj.data
            ffn.gate_up_proj = nn.Parameter(torch.cat([_shard_rows(gu[:inter], r, W), _shard_rows(gu[inter:], r, W)], dim=0))
            ffn.down_proj = nn.Parameter(_shard_cols(ffn.down_proj.data, r, W))
            ffn.tp_group, ffn.tp_size, ffn.tp_rank = group, W, r
            ffn.gate_up_proj._ats_tp = ("gate_up", W, r)
            ffn.down_proj._ats_tp = ("col", W, r)
    model.tp_size, model.tp_rank = W, r


def gather_tensor_parallel_state(model, mesh) -> dict:
    """Full (un-sharded) state dict of a tensor-parallel model, on every rank of the ``tp`` group (checkpoint interchange)."""
    W, group = mesh.tp_size, mesh.group("tp")
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    if W <= 1:
        return sd

    def gather(t: torch.Tensor, dim: int) -> torch.Tensor:
        parts = [torch.empty_like(t) for _ in range(W)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts, dim=dim)
    for i, blk in enumerate(model.layers):
        base = f"layers.{i}."
        if getattr(blk.self_attn, "tp_group", None) is not None:
            for n in ("q_proj", "k_proj", "v_proj"):
                sd[base + f"self_attn.{n}.weight"] = gather(sd[base + f"self_attn.{n}.weight"], 0)
            sd[base + "self_attn.o_proj.weight"] = gather(sd[base + "self_attn.o_proj.weight"], 1)
        if blk.ffn_kind == "dense" and getattr(blk.ffn, "tp_group", None) is not None:
            gu = sd[base + "ffn.gate_up_proj.weight"]
            half = gu.shape[0] // 2
            sd[base + "ffn.gate_up_proj.weight"] = torch.cat([gather(gu[:half], 0), gather(gu[half:], 0)], dim=0)
            sd[base + "ffn.down_proj.weight"] = gather(sd[base + "ffn.down_proj.weight"], 1)
    return sd


def apply_sequence_parallel(model, mesh) -> None:
    """Head-scatter sequence parallelism over ``mesh.group('sp')``: every rank feeds its ``L / W`` tokens of each sequence."""
    W, r, group = mesh.sp_size, mesh.coord.sp, mesh.group("sp")
    if W <= 1:
        return
    cfg = model.config
    tp = getattr(model, "tp_size", 1)
    if (cfg.num_heads // tp) % W or (cfg.num_kv_heads // tp) % W:
        raise ValueError(f"sequence_parallel_size {W} must divide the attention heads of a rank ({cfg.num_heads // tp} query, "
                         f"{cfg.num_kv_heads // tp} KV)")
    for blk in model.layers:
        blk.self_attn.sp_group, blk.self_attn.sp_size, blk.self_attn.sp_rank = group, W, r
    model.sp_size, model.sp_rank = W, r


def shard_sequence(batch: dict, mesh) -> dict:
    """This rank's ``L / W`` tokens of every tensor of the batch that has a sequence dimension."""
    W, r = mesh.sp_size, mesh.coord.sp
    if W <= 1:
        return batch
    out = {}
    for k, v in batch.items():
        if torch.is_tensor(v) and v.dim() >= 2:
            L = v.shape[1]
            if L % W:
                raise ValueError(f"sequence length {L} is not divisible by sequence_parallel_size {W}")
            out[k] = v[:, r * (L // W):(r + 1) * (L // W)].contiguous()
        else:
            out[k] = v
    return out

"""All-gather fused into the GEMM: linear layers whose weight is row-sharded over the data-parallel group (ZeRO-3 style)
and never gathered by a collective in the forward pass.

One kernel launch (``csrc/gemm_tcgen05.cu``, ``ats_gemm_bf16_gathered``): a few CTAs of the persistent GEMM grid are copy
engines that pull the remote shards over NVLink (bulk copies staged through shared memory, each remote byte crosses the
link once) into a staging buffer on this GPU and publish 128-row chunks through flags; the other CTAs run the tcgen05
GEMM, beginning with the output columns that belong to this rank's own shard and waiting (bounded) only for the chunks
a tile actually reads.  The weight shards live in CUDA-IPC symmetric memory so that peers can read them.

The reference reaches the same state with a library all-gather followed by a library GEMM (DeepSpeed ZeRO-3 / FSDP
``FULL_SHARD``, reference ``backend/backend_fsdp.py``; vendored Gemini chunk gather, colossalai ``zero/gemini/chunk/chunk.py:508``).
The backward pass here re-gathers with NCCL (input gradient) and reduce-scatters the weight gradient.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as G
from .peer import SymmetricBuffer

_vp, _ci, _cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_sig = False


def _fn():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_gemm_bf16_gathered.restype = _ci
        lib.ats_gemm_bf16_gathered.argtypes = [_vp, _cll, _vp, _vp, _cll, _vp, _ci, _ci, _ci, _vp, _ci, _vp, _ci, _vp, _ci, _vp, _ci,
                                               _ci, _ci, _ci, _ci, _ci, _vp, _vp]
        _sig = True
    return lib.ats_gemm_bf16_gathered


class GatherContext:
    """Per-group resources shared by all sharded linears: the staging buffer the remote shards are pulled into."""
    READY_ROWS = 128

    def __init__(self, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.staging: Optional[torch.Tensor] = None

    def reserve(self, rows: int, cols: int) -> None:
        need = rows * cols
        if self.staging is None or self.staging.numel() < need:
            self.staging = torch.empty(need, dtype=torch.bfloat16, device=self.device)


class ShardedWeight:
    """A [N, K] weight whose rows are split evenly over the group; this rank's rows live in symmetric memory."""

    def __init__(self, full: torch.Tensor, ctx: GatherContext):
        N, K = full.shape
        W = ctx.world
        if N % (W * GatherContext.READY_ROWS):
            raise ValueError(f"rows ({N}) must be a multiple of group size x {GatherContext.READY_ROWS}")
        self.ctx, self.N, self.K = ctx, N, K
        self.shard_rows = N // W
        self.buf = SymmetricBuffer(self.shard_rows * K * 2, ctx.group, ctx.device)
        self.shard = self.buf.tensor(torch.bfloat16, self.shard_rows * K).view(self.shard_rows, K)
        self.shard.copy_(full[ctx.rank * self.shard_rows:(ctx.rank + 1) * self.shard_rows].to(torch.bfloat16))
        self.src_table = torch.tensor(self.buf.ptrs, dtype=torch.int64, device=ctx.device)  # device array of shard addresses
        self.grad_shard: Optional[torch.Tensor] = None
        # per-chunk piece counters (they only grow) and the number of gathers done with them
        self.flags = torch.zeros(N // GatherContext.READY_ROWS, dtype=torch.int32, device=ctx.device)
        self.calls = 0
        ctx.reserve(N, K)
        if W > 1:
            dist.barrier(ctx.group)  # every shard is written and mapped before the first remote read

    def gather_nccl(self) -> torch.Tensor:
        """Library path (baseline twin and backward pass): the full [N, K] weight in a fresh tensor."""
        full = torch.empty(self.N, self.K, dtype=torch.bfloat16, device=self.ctx.device)
        if self.ctx.world > 1:
            dist.all_gather_into_tensor(full.view(-1), self.shard.reshape(-1), group=self.ctx.group)
        else:
            full.copy_(self.shard)
        return full


def gathered_gemm(x2: torch.Tensor, w: ShardedWeight, out: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None,
                  swiglu: bool = False, pre_act: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x2 [M, K] @ W^T with W gathered inside the kernel.  ``swiglu``: W = [gate; up], out = silu(gate) * up."""
    ctx = w.ctx
    M, K = x2.shape
    n_out = w.N // 2 if swiglu else w.N
    if out is None:
        out = torch.empty(M, n_out, dtype=x2.dtype, device=x2.device)
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    ctx.reserve(w.N, K)
    w.calls += 1
    if w.calls >= 1 << 18:  # counters are int32: start over long before they wrap
        w.flags.zero_()
        w.calls = 1
    epi = G.EPI_SWIGLU if swiglu else (G.EPI_ADDC if add is not None else G.EPI_STORE)
    st = _lib.status_tensor(x2.device)
    err = _fn()(_lib.ptr(x2), x2.stride(0), _lib.ptr(ctx.staging), _lib.ptr(w.shard), w.N, _lib.ptr(w.src_table), ctx.world, ctx.rank,
                getattr(w, "ready_rows", GatherContext.READY_ROWS),
                _lib.ptr(w.flags), w.calls, _lib.ptr(out), out.stride(0), _lib.ptr(add), add.stride(0) if add is not None else 0,
                _lib.ptr(pre_act), pre_act.stride(0) if pre_act is not None else 0, M, n_out, K, epi, w.N // 2 if swiglu else 0,
                _lib.ptr(st), _lib.stream_ptr(x2.device))
    _lib.check(err, "ats_gemm_bf16_gathered")
    return out


class _AGLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, w: ShardedWeight, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, w.N) if residual is not None else None
        y = torch.empty(*shape[:-1], w.N, dtype=x.dtype, device=x.device)
        gathered_gemm(x2, w, out=y.view(-1, w.N), add=r2)
        ctx.save_for_backward(x2)
        ctx.w, ctx.shape, ctx.has_res = w, shape, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        w: ShardedWeight = ctx.w
        dy2 = dy.reshape(-1, w.N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        full = w.gather_nccl()
        dx = G.gemm_nn(dy2, full).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw_full = G.gemm_tn(dy2, x2)  # [N, K]
        g = torch.empty(w.shard_rows, w.K, dtype=dw_full.dtype, device=dw_full.device)
        if w.ctx.world > 1:
            dist.reduce_scatter_tensor(g.view(-1), dw_full.view(-1), group=w.ctx.group)
        else:
            g.copy_(dw_full)
        w.grad_shard = g if w.grad_shard is None else w.grad_shard + g
        return dx, None, None, (dy if ctx.has_res else None)


class AllGatherLinear(torch.nn.Module):
    """``y = x W^T (+ residual)`` with W row-sharded over ``ctx.group``.  ``weight_shard`` is this rank's slice (a view of
    the symmetric buffer); its gradient arrives in ``weight.grad_shard`` already summed over the group."""

    def __init__(self, full_weight: torch.Tensor, ctx: GatherContext):
        super().__init__()
        self.weight = ShardedWeight(full_weight, ctx)
        self._anchor = torch.nn.Parameter(torch.zeros((), device=ctx.device))  # keeps the Function in the autograd graph

    @property
    def weight_shard(self) -> torch.Tensor:
        return self.weight.shard

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return _AGLinearFn.apply(x, self._anchor, self.weight, residual)

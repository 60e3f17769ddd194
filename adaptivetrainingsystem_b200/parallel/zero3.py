"""ZeRO stage 3: parameters, gradients and optimiser state are all partitioned; a transformer block's weights exist in
full only while that block runs.

Layout.  Every weight matrix of a block is sharded by ROWS over the data-parallel group (rank ``r`` keeps rows
``[r N / W, (r + 1) N / W)`` as a bf16 shard plus fp32 master / moments / gradient shard); a block is one *unit* (the FSDP
wrapping unit / Gemini chunk of the reference's backends, ``backend/backend_fsdp.py:151-198``,
``colossalai/zero/gemini/chunk/chunk.py:58-650``, ``gemini_ddp.py:343-401``).  Everything else (embedding, output head, norm
weights) forms a *root* unit that stays gathered, like FSDP's root, with a flat ZeRO shard of its optimiser state.

With peer memory (one process per GPU on NVLink) no collective library call is on the training path:

* forward: every linear layer of a block runs the GEMM that gathers its weight itself (``ats_gemm_bf16_gathered``: copy warps
  of the GEMM launch pull the remote row shards over NVLink while the tensor cores already work on the local ones), so no
  all-gather precedes the forward pass and no gathered copy outlives the product;
* backward: the unit below the running one is re-gathered by a pull kernel on a side stream (``BACKWARD_PRE`` prefetch) into
  one of two rotating buffers; every weight-gradient GEMM does its own reduce-scatter: its epilogue adds each output row
  straight into the fp32 gradient shard of the rank that owns the row (vector ``red.add`` over NVLink for rows owned by
  peers), while the main loop of the next tile is running.  No gradient buffer of full size exists, no reduction kernel or
  collective follows the backward pass, and gradients of several micro-batches accumulate in fp32 in the same place;
* step: squared norm of the gradient shards -> scalar exchange on a flag barrier -> clip coefficient on the device -> one
  AdamW launch over the whole shard arena that writes the bf16 row shards in place -> flag barrier.  Nothing is gathered
  after the step; the next forward reads the peers' shards directly.

Without peer memory (CPU / Gloo, or ``fused_comm=None``) the same engine runs on ``all_gather_into_tensor`` /
``reduce_scatter_tensor`` per matrix: the baseline twin, and what the CPU tests exercise.
"""
from __future__ import annotations

import ctypes
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import _lib
from .bootstrap import ProcessMesh
from .zero import NO_DECAY_KEYS, _pad_to

STATE_KEYS = ("master", "exp_avg", "exp_avg_sq")
_vp = ctypes.c_void_p


class Matrix:
    """One row-sharded weight of a block.  Duck-types ``fused_linear.ShardedWeight`` (``ctx, N, K, shard, src_table, flags,
    calls, ready_rows``) so that the gathering GEMM takes it as its B operand."""

    def __init__(self, name: str, param: nn.Parameter, W: int, r: int):
        self.name, self.param = name, param
        self.shape = tuple(param.shape)
        self.N = self.shape[0]
        self.K = param.numel() // self.N
        self.W, self.r = W, r
        self.rows = self.N // W
        self.shard_numel = self.rows * self.K
        self.numel = self.N * self.K
        self.full: Optional[torch.Tensor] = None   # [N, K] view into a gather slot while the unit is gathered
        self.full_off = 0                          # element offset inside the unit's full buffers
        self.arena_off = 0                         # element offset of this rank's shard inside the shard arenas
        # set by the engine
        self.shard = self.master = self.exp_avg = self.exp_avg_sq = self.grad32 = None
        self.ctx = None
        self.src_table = self.flags = None
        self.calls = 0
        self.ready_rows = 128 if self.rows % 128 == 0 else 64
        self.gather_in_gemm = False

    @staticmethod
    def eligible(param: nn.Parameter, W: int) -> bool:
        return (param.ndim == 2 and param.shape[0] % W == 0 and ((param.shape[0] // W) * param.shape[1]) % 8 == 0
                and param.shape[1] % 8 == 0)

    def fused_forward_ok(self) -> bool:
        # shards of whole 64-row chunks; when a shard begins or ends inside one of the 128-row boxes the GEMM reads, the kernel
        # stages that edge chunk of the own shard next to the remote ones
        return self.rows % 64 == 0 and self.K % 32 == 0 and self.N >= 128


class BlockUnit:
    def __init__(self, index: int, module: nn.Module, matrices: List[Matrix]):
        self.index, self.module, self.matrices = index, module, matrices
        off = 0
        for m in matrices:
            m.full_off = off
            off += _pad_to(m.numel, 8)
        self.full_numel = off
        self.gathered = False
        self.ready_event = None
        self.slot = index % 2
        self.grads_open = False
        self.in_backward = False


class RootUnit:
    """Flat ZeRO shard of every parameter that is not a block matrix; the full copy stays resident."""

    def __init__(self, params: List[Tuple[str, nn.Parameter]], group, W: int, r: int, dtype, device, alloc):
        self.group, self.W, self.r = group, W, r
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.shapes = [p.shape for p in self.params]
        offs, total = [], 0
        for p in self.params:
            offs.append(total)
            total += _pad_to(p.numel(), 8)
        self.offsets, self.padded = offs, _pad_to(max(total, 8), W * 8)
        self.shard = self.padded // W
        self.full = alloc(self.padded, dtype)
        self.full_grad = alloc(self.padded, dtype)
        for p, o in zip(self.params, offs):
            self.full[o:o + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.full[o:o + p.numel()].view(p.shape)
        lo, hi = r * self.shard, (r + 1) * self.shard
        self.master = self.full[lo:hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad32 = torch.zeros_like(self.master)
        wd = torch.zeros(self.padded, dtype=torch.float32, device=device)
        for n, p, o in zip(self.names, self.params, offs):
            if not (p.ndim < 2 or any(k in n.lower() for k in NO_DECAY_KEYS)):
                wd[o:o + p.numel()] = 1.0
        self.wd_mask = wd[lo:hi].clone()
        self.open_grads()

    def open_grads(self) -> None:
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            p._ats_grad = self.full_grad[o:o + shp.numel()]
            p._ats_grad_fresh = True
            ops.functional.register_grad_sink(p)
            p.grad = None

    def fold_autograd_grads(self) -> None:
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            sink = self.full_grad[o:o + shp.numel()]
            if p.grad is not None:
                if getattr(p, "_ats_grad_fresh", True):
                    sink.copy_(p.grad.reshape(-1))
                else:
                    sink.add_(p.grad.reshape(-1).to(sink.dtype))
                p.grad = None
                p._ats_grad_fresh = False
            elif getattr(p, "_ats_grad_fresh", True):
                sink.zero_()


class ZeRO3Engine:
    """Same surface as :class:`~adaptivetrainingsystem_b200.parallel.zero.ShardedEngine` (``step``, ``zero_grad``,
    ``set_lr`` ...), for models whose blocks hold plain weight matrices (dense decoders)."""

    def __init__(self, model: nn.Module, lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, mesh: Optional[ProcessMesh] = None, grad_accumulation_steps: int = 1, prefetch: bool = True,
                 fused_comm=None, copy_blocks: int = 64):
        self.model = model
        self.mesh = mesh or ProcessMesh(create_groups=False)
        self.zero_stage = 3
        self.max_grad_norm, self.grad_accumulation_steps = max_grad_norm, max(grad_accumulation_steps, 1)
        p0 = next(model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        self.group, self.W, self.r = self.mesh.group("dp"), self.mesh.size("dp"), self.mesh.index("dp")
        W, r = self.W, self.r
        # fused_comm: True / a peer-memory communicator -> kernels move everything over NVLink; None / False -> library collectives
        self.fused = bool(fused_comm) and self.device.type == "cuda" and W > 1 and self.dtype == torch.bfloat16 \
            and dist.is_initialized() and W == self.mesh.world
        import os as _os
        self.copy_blocks = int(_os.environ.get("ATS_Z3_COPY_BLOCKS", copy_blocks))  # CTAs of the side-stream pull kernels (they share the GPU with the GEMMs)
        self._sym: List[Any] = []

        # -- units -----------------------------------------------------------------------------------------------
        self.units: List[BlockUnit] = []
        in_block = set()
        for i, blk in enumerate(model.layers):
            mats = []
            for n, p in blk.named_parameters():
                if p.requires_grad and Matrix.eligible(p, W) and not getattr(p, "_ats_expert", False):
                    mats.append(Matrix(f"layers.{i}.{n}", p, W, r))
                    in_block.add(id(p))
            self.units.append(BlockUnit(i, blk, mats))
        self.matrices: List[Matrix] = [m for u in self.units for m in u.matrices]

        # -- shard arenas (bf16 row shards peer-readable when fused; fp32 state private) ---------------------------------
        off = 0
        for m in self.matrices:
            m.arena_off = off
            off += m.shard_numel
        self.arena_numel = _pad_to(max(off, 8), 8)
        self.shard_arena = self._alloc(self.arena_numel, self.dtype, symmetric=True)
        for m in self.matrices:
            lo = r * m.shard_numel
            m.shard = self.shard_arena[m.arena_off:m.arena_off + m.shard_numel].view(m.rows, m.K)
            m.shard.copy_(m.param.data.reshape(-1)[lo:lo + m.shard_numel].view(m.rows, m.K))
        self.master = self.shard_arena.float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        # with peer memory the gradient shards are written by every rank's weight-gradient GEMMs: peer-mapped, zeroed once per step
        self.grad32 = self._alloc(self.arena_numel, torch.float32, symmetric=True)
        for m in self.matrices:
            sl = slice(m.arena_off, m.arena_off + m.shard_numel)
            m.master, m.exp_avg, m.exp_avg_sq, m.grad32 = self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], self.grad32[sl]
            m.scatter = None
            m.param.data = torch.empty(0, dtype=self.dtype, device=self.device)
            m.param._ats_z3 = m

        # -- gather / gradient slots (two of each, rotating over the units) -------------------------------------------------
        slot_numel = max([u.full_numel for u in self.units] + [8])
        self.full_slots = [torch.empty(slot_numel, dtype=self.dtype, device=self.device) for _ in range(2)]
        # library path only: full-size gradient buffers that are reduce-scattered per matrix
        self.grad_slots = [] if self.fused else [torch.zeros(slot_numel, dtype=self.dtype, device=self.device) for _ in range(2)]

        # -- root --------------------------------------------------------------------------------------------------------
        root = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in in_block]
        self.root = RootUnit(root, self.group, W, r, self.dtype, self.device, lambda n, dt: self._alloc(n, dt, symmetric=True))

        self.hyper = torch.tensor([lr, betas[0], betas[1], eps, weight_decay, 0.0], dtype=torch.float32, device=self.device)
        self._hyper_host = [lr, betas[0], betas[1], eps, weight_decay, 0.0]
        self.clip_state = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step_count = 0
        self.last_grad_norm = None
        self.prefetch = prefetch and self.device.type == "cuda"
        self._pending: List[int] = []
        self.grad_fresh_units = [True] * len(self.units)

        if self.fused:
            from .fused_linear import GatherContext
            from .peer import PeerBarrier
            self.ctx = GatherContext(self.group, self.device)
            self.ctx.reserve(1, max([m.numel for m in self.matrices] + [8]))
            from ..ops.gemm import ScatterTarget
            arena_ptrs = list(self.shard_arena._ats_sym.ptrs)
            grad_ptrs = list(self.grad32._ats_sym.ptrs)
            for m in self.matrices:
                # where the rows of this matrix's gradient live: rank q owns rows [q * rows, (q + 1) * rows) in its own fp32 shard
                m.scatter = ScatterTarget(torch.tensor([p + m.arena_off * 4 for p in grad_ptrs], dtype=torch.int64, device=self.device),
                                          m.rows, (m.N, m.K))
                m.ctx = self.ctx
                m.peer_ptrs = [p + m.arena_off * 2 for p in arena_ptrs]
                m.peer_table = (_vp * W)(*[_vp(p) for p in m.peer_ptrs])
                m.src_table = torch.tensor(m.peer_ptrs, dtype=torch.int64, device=self.device)
                m.gather_in_gemm = m.fused_forward_ok()
                if m.gather_in_gemm:
                    m.flags = torch.zeros(m.N // m.ready_rows, dtype=torch.int32, device=self.device)
            self.root_grad_table = self.root.full_grad._ats_sym.table(0)
            self.root_param_table = self.root.full._ats_sym.table(0)
            self.step_barrier = PeerBarrier(self.group, self.device)
            self.gather_stream = torch.cuda.Stream(device=self.device)
            self.slot_free = [None, None]      # event: the gather slot's last user has finished with it
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self.params_ready = torch.cuda.Event()  # recorded after the barrier that ends a step: every rank's shards are current
            self.params_ready.record(torch.cuda.current_stream(self.device))
        self._install_hooks()

    # -- memory ------------------------------------------------------------------------------------------------------
    def _alloc(self, n: int, dtype, symmetric: bool) -> torch.Tensor:
        n = max(int(n), 8)
        if symmetric and self.fused:
            from .peer import SymmetricBuffer
            es = torch.empty((), dtype=dtype).element_size()
            buf = SymmetricBuffer(n * es, self.group, self.device)
            self._sym.append(buf)
            t = buf.tensor(dtype, n)
            t._ats_sym = buf
            return t
        return torch.zeros(n, dtype=dtype, device=self.device)

    def close(self) -> None:
        """Give the peer-mapped buffers back (they live outside PyTorch's allocator).  The engine is unusable afterwards."""
        for b in self._sym:
            b.close()
        self._sym = []
        if self.fused:
            self.step_barrier.buf.close()

    # -- gather / release of one unit ------------------------------------------------------------------------------------
    def _attach(self, u: BlockUnit, buf: torch.Tensor) -> None:
        for m in u.matrices:
            m.full = buf[m.full_off:m.full_off + m.numel].view(m.N, m.K)
            m.param.data = m.full.view(m.shape)
        u.gathered = True

    def _release(self, u: BlockUnit) -> None:
        if not u.gathered:
            return
        if self.fused:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.slot_free[u.slot] = ev
        for m in u.matrices:
            m.full = None
            m.param.data = torch.empty(0, dtype=self.dtype, device=self.device)
        u.gathered = False
        u.ready_event = None

    def _gather_matrix_twin(self, m: Matrix, dst: torch.Tensor) -> None:
        if self.W == 1 or not dist.is_initialized():
            dst.copy_(m.shard.reshape(-1))
        elif dist.get_backend(self.group) == "gloo":
            parts = [torch.empty(m.shard_numel, dtype=self.dtype, device=self.device) for _ in range(self.W)]
            dist.all_gather(parts, m.shard.reshape(-1).contiguous(), group=self.group)
            torch.cat(parts, out=dst)
        else:
            dist.all_gather_into_tensor(dst, m.shard.reshape(-1).contiguous(), group=self.group)

    def _ensure_gathered(self, u: BlockUnit, prefetching: bool = False) -> None:
        """Unit ``u`` is (or will be, once its ready event has fired) in its slot with the parameters pointing there."""
        if u.gathered:
            return
        buf = self.full_slots[u.slot]
        if not self.fused:
            # library path: one all-gather per matrix (rank-major concatenation = row order)
            for m in u.matrices:
                self._gather_matrix_twin(m, buf[m.full_off:m.full_off + m.numel])
            self._attach(u, buf)
            return
        from .peer import _L
        cur = torch.cuda.current_stream(self.device)
        gs = self.gather_stream
        gs.wait_event(self.params_ready)  # never read a shard that the last optimiser step has not finished writing
        ev = self.slot_free[u.slot]
        if ev is not None:
            gs.wait_event(ev)        # the slot's previous user has finished with it
        st = _lib.status_tensor(self.device)
        sp = _vp(gs.cuda_stream)
        for m in u.matrices:   # pull every row shard from its owner, on the side stream, with a bounded number of CTAs
            dst = buf[m.full_off:m.full_off + m.numel]
            _lib.check(_L().ats_peer_gather(m.peer_table, self.W, _lib.ptr(dst), m.shard_numel * 2, self.copy_blocks, _lib.ptr(st), sp),
                       "peer_gather")
        u.ready_event = torch.cuda.Event()
        u.ready_event.record(gs)
        self._attach(u, buf)
        if not prefetching:
            cur.wait_event(u.ready_event)

    # -- gradients -----------------------------------------------------------------------------------------------------------
    def _open_grads(self, u: BlockUnit) -> None:
        if self.fused:
            for m in u.matrices:  # the weight-gradient GEMM adds its rows into the owners' shards: nothing to buffer, always accumulating
                m.param._ats_grad = m.scatter
                m.param._ats_grad_fresh = False
                ops.functional.register_grad_sink(m.param)
                m.param.grad = None
            u.grads_open = True
            return
        slot = self.grad_slots[u.slot]
        for m in u.matrices:
            m.param._ats_grad = slot[m.full_off:m.full_off + m.numel]
            m.param._ats_grad_fresh = True
            ops.functional.register_grad_sink(m.param)
            m.param.grad = None
        u.grads_open = True

    def _reduce_unit(self, u: BlockUnit) -> None:
        """The unit's backward is complete on this rank.  Library path: fold what autograd delivered, reduce-scatter every
        matrix, accumulate into the fp32 shards.  With peer memory the GEMM epilogues have already done all of it."""
        if not u.grads_open:
            return
        u.grads_open = False
        if self.fused:
            for m in u.matrices:
                if m.param.grad is not None:
                    raise RuntimeError(f"{m.name}: a gradient arrived through plain autograd; with peer memory the weight-gradient "
                                       "products of row-sharded matrices must go through ops.linear / ops.swiglu_mlp")
            self.grad_fresh_units[u.index] = False
            return
        slot = self.grad_slots[u.slot]
        acc = not self.grad_fresh_units[u.index]
        for m in u.matrices:
            sink = slot[m.full_off:m.full_off + m.numel]
            p = m.param
            if p.grad is not None:
                if getattr(p, "_ats_grad_fresh", True):
                    sink.copy_(p.grad.reshape(-1))
                else:
                    sink.add_(p.grad.reshape(-1).to(sink.dtype))
                p.grad = None
            elif getattr(p, "_ats_grad_fresh", True):
                sink.zero_()  # the matrix took no part in this backward
            lo = self.r * m.shard_numel
            if self.W > 1 and dist.is_initialized():
                if dist.get_backend(self.group) == "gloo":
                    dist.all_reduce(sink, group=self.group)
                    red = sink[lo:lo + m.shard_numel]
                else:
                    red = torch.empty(m.shard_numel, dtype=self.dtype, device=self.device)
                    dist.reduce_scatter_tensor(red, sink, group=self.group)
            else:
                red = sink[lo:lo + m.shard_numel]
            if acc:
                m.grad32.add_(red.float())
            else:
                m.grad32.copy_(red.float())
        self.grad_fresh_units[u.index] = False

    # -- hooks ---------------------------------------------------------------------------------------------------------------
    def _install_hooks(self) -> None:
        n = len(self.units)
        for u in self.units:
            if not u.matrices:
                continue

            def pre_fwd(mod, args, i=u.index):
                uu = self.units[i]
                if self.fused and not uu.gathered and all(m.gather_in_gemm for m in uu.matrices):
                    return  # every linear of the block gathers its weight inside its own GEMM
                self._ensure_gathered(uu)

            def post_fwd(mod, args, out, i=u.index):
                uu = self.units[i]
                if uu.in_backward or (torch.is_grad_enabled() and i == n - 1):
                    return  # a recomputed forward inside the backward pass, or the last block whose backward comes next
                self._release(uu)

            def pre_bwd(mod, gout, i=u.index):
                self._flush_pending()  # the unit above has finished: its reduce goes out now and overlaps this unit's backward
                uu = self.units[i]
                uu.in_backward = True
                self._ensure_gathered(uu)
                if self.fused and uu.ready_event is not None:
                    torch.cuda.current_stream(self.device).wait_event(uu.ready_event)
                self._open_grads(uu)
                if self.prefetch and self.fused and i - 1 >= 0 and self.units[i - 1].matrices:
                    self._ensure_gathered(self.units[i - 1], prefetching=True)

            def post_bwd(mod, gin, gout, i=u.index):
                self._pending.append(i)

            u.module.register_forward_pre_hook(pre_fwd)
            u.module.register_forward_hook(post_fwd)
            u.module.register_full_backward_pre_hook(pre_bwd)
            u.module.register_full_backward_hook(post_bwd)

    def _flush_pending(self) -> None:
        for i in self._pending:
            u = self.units[i]
            self._reduce_unit(u)
            u.in_backward = False
            self._release(u)
        self._pending = []

    # -- optimiser API ----------------------------------------------------------------------------------------
    def set_lr(self, lr: float) -> None:
        self._hyper_host[0] = float(lr)
        self.hyper[0] = float(lr)

    def get_lr(self) -> float:
        return self._hyper_host[0]

    def set_weight_decay(self, wd: float) -> None:
        self._hyper_host[4] = float(wd)
        self.hyper[4] = float(wd)

    def zero_grad(self) -> None:
        self.grad_fresh_units = [True] * len(self.units)
        self.root.open_grads()

    def _reduce_root(self) -> None:
        root = self.root
        root.fold_autograd_grads()
        lo = self.r * root.shard
        if self.fused:
            from .peer import _L
            st = _lib.status_tensor(self.device)
            _lib.check(_L().ats_peer_reduce_rows(self.root_grad_table, self.W, self.r, lo, root.shard, _lib.ptr(root.grad32), 0, _lib.ptr(st),
                                                 0, _lib.stream_ptr(self.device)), "peer_reduce_rows(root)")
            return
        if self.W > 1 and dist.is_initialized():
            if dist.get_backend(self.group) == "gloo":
                dist.all_reduce(root.full_grad, group=self.group)
                red = root.full_grad[lo:lo + root.shard]
            else:
                red = torch.empty(root.shard, dtype=self.dtype, device=self.device)
                dist.reduce_scatter_tensor(red, root.full_grad, group=self.group)
        else:
            red = root.full_grad[lo:lo + root.shard]
        root.grad32.copy_(red.float())

    def step(self) -> Dict[str, Any]:
        self.step_count += 1
        self._hyper_host[5] = float(self.step_count)
        self.hyper[5] = float(self.step_count)
        ops.fp8.weights_changed()  # cached quantised weights are stale after this step
        self._flush_pending()
        for u in self.units:  # a unit that is still gathered goes back to shards
            self._release(u)
        root = self.root
        if self.fused:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_stream(self.gather_stream)
            root.fold_autograd_grads()
            # every rank has finished its backward: all rows that peers added to this rank's gradient shards have landed and the
            # root gradients are final everywhere
            self.step_barrier()
        self._reduce_root()
        if not self.fused:
            for i, fresh in enumerate(self.grad_fresh_units):
                if fresh:
                    for m in self.units[i].matrices:  # the unit took no part in this step
                        m.grad32.zero_()
        ops.sumsq(self.grad32, self.sumsq, accumulate=False)
        ops.sumsq(root.grad32, self.sumsq, accumulate=True)
        scale = 1.0 / (self.mesh.dp_size * self.grad_accumulation_steps)
        if self.fused:
            from .peer import _L
            self.step_barrier(self.sumsq)         # carries every rank's squared norm to every rank
            _lib.check(_L().ats_clip_coef_slots(_lib.ptr(self.step_barrier.slots), self.W, scale, float(self.max_grad_norm),
                                                _lib.ptr(self.clip_state), _lib.stream_ptr(self.device)), "clip_coef_slots")
        else:
            if dist.is_initialized() and self.mesh.world > 1:
                dist.all_reduce(self.sumsq)
            ops.clip_coef(self.sumsq, self.clip_state, scale, self.max_grad_norm)
        self._adamw()
        if self.fused:
            self.grad32.zero_()                   # the next step's weight-gradient GEMMs add into zeros
            self.step_barrier()                   # every shard is updated (and every gradient shard cleared) before anyone goes on
            self.params_ready = torch.cuda.Event()
            self.params_ready.record(torch.cuda.current_stream(self.device))
        self.zero_grad()
        self.last_grad_norm = self.clip_state[1]
        return {"grad_norm": self.clip_state[1], "skipped": self.clip_state[2]}

    def _adamw(self) -> None:
        root = self.root
        lr, wd = self._hyper_host[0], self._hyper_host[4]
        if wd != 0.0:  # the root mixes decayed and non-decayed elements: decay applied through a mask, the kernel runs without
            root.master.mul_(1.0 - (lr * wd) * root.wd_mask * (1.0 - self.clip_state[2]))
        lo = self.r * root.shard
        if self.device.type == "cuda" and self.dtype == torch.bfloat16:
            from .peer import _L
            st = _lib.status_tensor(self.device)
            stream = _lib.stream_ptr(self.device)
            if self.matrices:
                table = (_vp * 1)(_vp(self.shard_arena.data_ptr()))
                _lib.check(_L().ats_adamw_push(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq), _lib.ptr(self.grad32),
                                               table, 1, 0, 0, self.arena_numel, _lib.ptr(self.hyper), _lib.ptr(self.clip_state), 1.0,
                                               _lib.ptr(st), stream), "adamw(arena)")
            # root: with peer memory the updated shard goes straight into every rank's resident copy (the all-gather is the store)
            if self.fused:
                table, world, rank = self.root_param_table, self.W, self.r
            else:
                table, world, rank = (_vp * 1)(_vp(root.full.data_ptr())), 1, 0
            _lib.check(_L().ats_adamw_push(_lib.ptr(root.master), _lib.ptr(root.exp_avg), _lib.ptr(root.exp_avg_sq), _lib.ptr(root.grad32),
                                           table, world, rank, lo, root.shard, _lib.ptr(self.hyper), _lib.ptr(self.clip_state), 0.0,
                                           _lib.ptr(st), stream), "adamw(root)")
            if not self.fused:
                self._gather_root()
            return
        if self.matrices:
            ops.adamw_step(self.master, self.exp_avg, self.exp_avg_sq, self.grad32, self.shard_arena, self.hyper, self.clip_state, 1.0)
        ops.adamw_step(root.master, root.exp_avg, root.exp_avg_sq, root.grad32, root.full[lo:lo + root.shard], self.hyper, self.clip_state, 0.0)
        self._gather_root()

    def _gather_root(self) -> None:
        root = self.root
        if self.W == 1 or not dist.is_initialized():
            return
        lo = self.r * root.shard
        mine = root.full[lo:lo + root.shard].clone()
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(mine) for _ in range(self.W)]
            dist.all_gather(parts, mine, group=self.group)
            torch.cat(parts, out=root.full)
        else:
            dist.all_gather_into_tensor(root.full, mine, group=self.group)

    def get_global_grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    def gather_full_parameters(self) -> None:
        """Materialise every block (checkpoint save / evaluation without hooks): private full copies, not the rotating slots."""
        for u in self.units:
            if not u.matrices:
                continue
            self._release(u)
            buf = torch.empty(u.full_numel, dtype=self.dtype, device=self.device)
            for m in u.matrices:
                self._gather_matrix_twin(m, buf[m.full_off:m.full_off + m.numel])
            self._attach(u, buf)

    def release_parameters(self) -> None:
        for u in self.units:
            self._release(u)

    def memory_bytes(self) -> Dict[str, int]:
        es = self.shard_arena.element_size()
        return {"params": (self.arena_numel + self.root.padded) * es,
                "grads": (self.arena_numel + self.root.shard) * 4 + sum(t.numel() for t in self.grad_slots) * es + self.root.padded * es,
                "optimizer": 3 * (self.arena_numel + self.root.shard) * 4}

    # -- state: every stretch of a parameter whose optimiser state this rank holds -----------------------------------------------
    def owned_pieces(self, unique: bool = True) -> List[Dict[str, Any]]:
        """Same contract as :meth:`ShardedEngine.owned_pieces`."""
        out = []
        for m in self.matrices:
            out.append({"name": m.name, "shape": m.shape, "expert": False, "start": self.r * m.shard_numel, "length": m.shard_numel,
                        "tensors": {k: getattr(m, k) for k in STATE_KEYS}})
        root = self.root
        lo, hi = self.r * root.shard, (self.r + 1) * root.shard
        for name, o, shp in zip(root.names, root.offsets, root.shapes):
            a, e = max(o, lo), min(o + shp.numel(), hi)
            if e > a:
                out.append({"name": name, "shape": tuple(shp), "expert": False, "start": a - o, "length": e - a,
                            "tensors": {k: getattr(root, k)[a - lo:e - lo] for k in STATE_KEYS}})
        return out

    def load_pieces(self, fetch, step: Optional[int] = None, hyper: Optional[List[float]] = None) -> int:
        if step is not None:
            self.step_count = int(step)
        if hyper:
            self._hyper_host = list(hyper)
            self.hyper.copy_(torch.tensor(self._hyper_host, dtype=torch.float32))
        n = 0
        for piece in self.owned_pieces():
            got = fetch(piece)
            if got is None:
                continue
            for k, t in piece["tensors"].items():
                t.copy_(got[k].reshape(-1).to(t.device, t.dtype))
            n += 1
        if n:
            self._params_from_masters()
        return n

    def _params_from_masters(self) -> None:
        self.release_parameters()
        self.shard_arena.copy_(self.master.to(self.dtype))
        root = self.root
        lo = self.r * root.shard
        root.full[lo:lo + root.shard].copy_(root.master.to(self.dtype))
        self._gather_root()
        if self.fused:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)

    def state_dict(self) -> Dict[str, Any]:
        """Per-parameter optimiser state in full shapes (gathers: small models / tests; checkpoints use ``owned_pieces``)."""
        state: Dict[str, Any] = {}

        def gather(t: torch.Tensor) -> torch.Tensor:
            if self.W == 1 or not dist.is_initialized():
                return t
            parts = [torch.empty_like(t) for _ in range(self.W)]
            dist.all_gather(parts, t.contiguous(), group=self.group)
            return torch.cat(parts)
        for m in self.matrices:
            state[m.name] = {k: gather(getattr(m, k)).view(m.shape).cpu() for k in STATE_KEYS}
        root = self.root
        full = {k: gather(getattr(root, k)) for k in STATE_KEYS}
        for name, shp, o in zip(root.names, root.shapes, root.offsets):
            state[name] = {k: v[o:o + shp.numel()].view(shp).cpu() for k, v in full.items()}
        return {"state": state, "step": self.step_count, "hyper": list(self._hyper_host), "zero_stage": 3}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        st = sd["state"]

        def fetch(piece):
            e = st.get(piece["name"])
            if e is None:
                return None
            a, n = piece["start"], piece["length"]
            return {k: e[k].reshape(-1)[a:a + n] for k in STATE_KEYS}
        self.load_pieces(fetch, step=sd.get("step", 0), hyper=sd.get("hyper"))

    def resync_master_from_params(self) -> None:
        """Parameters were overwritten while gathered (checkpoint load): refresh shards and masters from them."""
        for u in self.units:
            if not u.gathered:
                continue
            for m in u.matrices:
                lo = self.r * m.shard_numel
                m.shard.copy_(m.param.data.reshape(-1)[lo:lo + m.shard_numel].view(m.rows, m.K))
        self.master.copy_(self.shard_arena.float())
        root = self.root
        lo = self.r * root.shard
        root.master.copy_(root.full[lo:lo + root.shard].float())
        self.release_parameters()
        if self.fused:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)

    @property
    def param_groups(self) -> List[Dict[str, Any]]:
        lr, wd = self._hyper_host[0], self._hyper_host[4]
        return [{"lr": lr, "weight_decay": wd, "name": f"layers.{u.index}", "params": [m.param for m in u.matrices]} for u in self.units] + \
               [{"lr": lr, "weight_decay": wd, "name": "root", "params": self.root.params}]

"""Expert parallelism: every rank of the ``ep`` group owns ``E / W`` experts of each MoE layer and all ranks exchange
routed tokens.

Layout.  Source rank ``s`` routes its ``T`` tokens, ranks the (token, k) slots per expert in token order and keeps at
most ``C`` of them per expert (per-source capacity, as DeepSpeed-MoE / the reference's vendored routers do,
``colossalai/moe/routers.py:47-58``).  The owner of expert ``e`` holds a receive buffer ``[E_local, W, C, H]``: block
``(e_local, s)`` is filled by source ``s``.  The grouped GEMM then runs over ``E_local * W`` row groups with one weight
per ``W`` groups; outputs go back to the sources' ``[E, C, H]`` return buffers, where the combine kernel forms the
weighted sum.

Two transports with identical numerics:

* **fused** (default on NVLink): the dispatch kernel writes token rows, pad rows and row counts straight into the
  owner's receive buffer on the peer GPU; the down-projection GEMM's epilogue writes its output tiles straight into the
  source rank's return buffer on the peer GPU; flag barriers (one warp, bounded wait) separate the phases.  Routing,
  permutation, the grouped SwiGLU GEMMs and the all-to-all traffic are the same kernels -- no collective library call.
* **nccl** (baseline, also what runs on CPU/Gloo): ``all_to_all_single`` on the capacity layout plus the same grouped
  GEMMs -- what ColossalAI's ``SparseMLP`` does (``colossalai/moe/layers.py:221-249``, ``moe/_operation.py:132-135``).
"""
from __future__ import annotations

import os

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as G
from ..ops import moe as M
from ..ops.functional import _L, _P, _S, _CK, _deliver_grad


# Decode-sized steps: the owners' "results are ready" flags can travel with the fold of the down projection and be awaited inside the
# combine kernel (1) instead of a flag-barrier launch between the two (0, default).  Measured on 2 GPUs the flag form is slower
# (8 Mixtral layers 3.16 -> 3.25 ms per step, the 22-layer model 3.75 -> 3.88 ms): a system-scope fence in every CTA of the fold
# and 64 polling CTAs cost more than the one-warp barrier launch they replace.
FLAG_SYNC = os.environ.get("ATS_EP_FLAG_SYNC", "0") == "1"


class _LayerBuffers:
    """Per-layer exchange buffers (symmetric when fused)."""

    def __init__(self, comm: "ExpertParallelComm", E: int, C: int, H: int, dtype: torch.dtype, device):
        W, r = comm.W, comm.rank
        El = E // W
        self.E, self.El, self.C, self.H = E, El, C, H
        n_recv = El * W * C * H
        n_ret = E * C * H
        es = torch.empty((), dtype=dtype).element_size()
        if comm.fused:
            from .peer import SymmetricBuffer
            # one symmetric allocation: recv_x | ret_y | recv_g | ret_dx | counts | own_y | own_dx
            off = [0]
            for n in (n_recv * es, n_ret * es, n_recv * es, n_ret * es, El * W * 4, n_recv * es, n_recv * es):
                off.append(off[-1] + (n + 255) // 256 * 256)
            self.sym = SymmetricBuffer(off[-1], comm.group, device)
            s = self.sym
            self.recv_x = s.tensor(dtype, n_recv, off[0]).view(El * W, C, H)
            self.ret_y = s.tensor(dtype, n_ret, off[1]).view(E, C, H)
            self.recv_g = s.tensor(dtype, n_recv, off[2]).view(El * W, C, H)
            self.ret_dx = s.tensor(dtype, n_ret, off[3]).view(E, C, H)
            self.counts = s.tensor(torch.int32, El * W, off[4])
            # expert outputs (forward) and input gradients (backward) stay on the GPU that computed them; the source ranks
            # pull their rows in the combine kernel (coalesced 4 KB row reads instead of scattered remote stores)
            self.own_y = s.tensor(dtype, n_recv, off[5]).view(El * W, C, H)
            self.own_dx = s.tensor(dtype, n_recv, off[6]).view(El * W, C, H)
            e = torch.arange(E, dtype=torch.int64)
            owner, el = e // El, e % El
            base = torch.tensor(s.ptrs, dtype=torch.int64)
            block = (el * W + r) * C * H * es
            # where this rank's rows for expert e go (forward activations / backward gradients) and its count
            self.t_disp_x = (base[owner] + off[0] + block).to(device)
            self.t_disp_g = (base[owner] + off[2] + block).to(device)
            self.t_count = (base[owner] + off[4] + (el * W + r) * 4).to(device)
            # ... and where the results for this rank's rows of expert e can be read from
            self.t_pull_y = (base[owner] + off[5] + block).to(device)
            self.t_pull_dx = (base[owner] + off[6] + block).to(device)
            # where the output of local group g = e_local * W + src goes on rank src
            g = torch.arange(El * W, dtype=torch.int64)
            gel, src = g // W, g % W
            back = ((r * El + gel) * C * H) * es
            self.t_ret_y = (base[src] + off[1] + back).to(device)
            self.t_ret_dx = (base[src] + off[3] + back).to(device)
        else:
            self.sym = None
            self.recv_x = torch.zeros(El * W, C, H, dtype=dtype, device=device)
            self.ret_y = torch.zeros(E, C, H, dtype=dtype, device=device)
            self.recv_g = torch.zeros(El * W, C, H, dtype=dtype, device=device)
            self.ret_dx = torch.zeros(E, C, H, dtype=dtype, device=device)
            self.counts = torch.zeros(El * W, dtype=torch.int32, device=device)


class _ServingBuffers:
    """Exchange buffers of a decode-sized step (no autograd): every source rank owns ``Cs`` rows of each expert's ONE row
    block ``[W * Cs, H]`` (``W * Cs`` a multiple of 128), so the expert GEMMs see one group per local expert and stream each
    weight once, however many ranks sent rows.  ``Cs >= T`` tokens per rank: nothing is ever dropped."""

    def __init__(self, comm: "ExpertParallelComm", E: int, Cs: int, H: int, dtype: torch.dtype, device):
        from .peer import SymmetricBuffer
        W, r = comm.W, comm.rank
        El = E // W
        self.E, self.El, self.Cs, self.H, self.rows = E, El, Cs, H, W * Cs
        es = torch.empty((), dtype=dtype).element_size()
        n = El * W * Cs * H
        off = [0, (n * es + 255) // 256 * 256]
        self.sym = SymmetricBuffer(off[1] * 2, comm.group, device)
        self.recv_x = self.sym.tensor(dtype, n, off[0]).view(El, W * Cs, H)
        self.own_y = self.sym.tensor(dtype, n, off[1]).view(El, W * Cs, H)
        e = torch.arange(E, dtype=torch.int64)
        owner, el = e // El, e % El
        base = torch.tensor(self.sym.ptrs, dtype=torch.int64)
        block = (el * W + r) * Cs * H * es  # this rank's rows inside expert e's block on the owner
        self.t_disp_x = (base[owner] + off[0] + block).to(device)
        self.t_pull_y = (base[owner] + off[1] + block).to(device)
        # every row of a block takes part in the products: rows that no token uses hold zeros or an earlier step's (finite)
        # values, their results are never read, so no row counts need to travel
        # "my down projection of this call is folded" flags: rank q raises entry q of every peer's array from the launch that folds
        # its down projection; the combine kernels wait on the entries of the owners they pull from (no barrier launch in between)
        self.flag_buf = SymmetricBuffer(256, comm.group, device)
        self.ready_flags = self.flag_buf.tensor(torch.int32, 64)
        self.ready_flags.zero_()
        self.flag_table = self.flag_buf.table(0)
        self.sync_state = torch.zeros(2, dtype=torch.int32, device=device)   # [calls so far (the epoch), CTAs done in the current fold]
        self.counts = torch.full((El,), W * Cs, dtype=torch.int32, device=device)
        self.local_counts = torch.zeros(E, dtype=torch.int32, device=device)
        self.shape_probe = torch.empty(1, dtype=dtype, device=device).expand(E, Cs, H)


class ExpertParallelComm:
    def __init__(self, mesh, fused: bool = True):
        self.mesh = mesh
        self.group = mesh.group("ep")
        self.W = mesh.ep_size
        self.rank = mesh.coord.ep
        self.fused = bool(fused) and torch.cuda.is_available()
        # results travel back by pull (the combine kernel reads the owners' buffers) or by push (GEMM epilogue stores)
        self.pull_results = os.environ.get("ATS_EP_RETURN", "pull") == "pull"
        self.barrier = None
        if self.fused:
            from .peer import PeerBarrier
            self.barrier = PeerBarrier(self.group)
        self._layers: Dict[Tuple[int, int, int, int], _LayerBuffers] = {}
        self.bytes_dispatched = 0

    def serving_rows(self, tokens: int) -> int:
        """Rows per (source rank, expert) of a decode-sized step, or 0 when the step is too large for the one-block layout:
        the smallest ``Cs >= tokens`` with ``W * Cs`` a multiple of 128, as long as a block stays within 256 rows."""
        W = self.W
        if not self.fused or W > 128 or 128 % W:
            return 0
        unit = 128 // W
        cs = (max(tokens, 1) + unit - 1) // unit * unit
        return cs if W * cs <= 256 else 0

    def serving_buffers(self, E: int, Cs: int, H: int, dtype, device) -> _ServingBuffers:
        key = ("serve", E, Cs, H)
        b = self._layers.get(key)
        if b is None:
            b = _ServingBuffers(self, E, Cs, H, dtype, device)
            self._layers[key] = b
            dist.barrier(self.group)  # all peers have mapped the new buffers
        return b

    def close(self) -> None:
        """Give the exchange buffers (device memory outside PyTorch's allocator) back."""
        for b in self._layers.values():
            if getattr(b, "sym", None) is not None:
                b.sym.close()
            if getattr(b, "flag_buf", None) is not None:
                b.flag_buf.close()
        self._layers.clear()
        if self.barrier is not None:
            self.barrier.buf.close()
            self.barrier = None

    def buffers(self, layer_idx: int, E: int, C: int, H: int, dtype, device) -> _LayerBuffers:
        key = (layer_idx, E, C, H)
        b = self._layers.get(key)
        if b is None:
            for k in [k for k in self._layers if k[0] == layer_idx]:
                del self._layers[k]
            b = _LayerBuffers(self, E, C, H, dtype, device)
            self._layers[key] = b
            if self.fused:
                dist.barrier(self.group)  # all peers have mapped the new buffers
        return b

    # -- transports -----------------------------------------------------------------------------------------
    def exchange_to_owners(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        """send [E, C, H] (by global expert = [W_owner, El, C, H]) -> recv [El * W_src, C, H]."""
        W = self.W
        El = send.shape[0] // W
        tmp = torch.empty_like(send)
        dist.all_to_all_single(tmp, send.contiguous(), group=self.group)  # tmp = [W_src, El, C, H]
        recv.copy_(tmp.view(W, El, *send.shape[1:]).transpose(0, 1).reshape(recv.shape))

    def exchange_to_sources(self, out: torch.Tensor, ret: torch.Tensor) -> None:
        """out [El * W_src, C, H] -> ret [E, C, H] on every source."""
        W = self.W
        El = out.shape[0] // W
        send = out.view(El, W, *out.shape[1:]).transpose(0, 1).contiguous()  # [W_src, El, C, H]
        dist.all_to_all_single(ret.view(W, El, *out.shape[1:]), send, group=self.group)

    def exchange_counts(self, counts: torch.Tensor, recv_counts: torch.Tensor) -> None:
        W = self.W
        El = counts.numel() // W
        tmp = torch.empty_like(counts)
        dist.all_to_all_single(tmp, counts.contiguous(), group=self.group)  # [W_src, El]
        recv_counts.copy_(tmp.view(W, El).t().reshape(-1))


class _EPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w1, w2, capacity, residual, comm: ExpertParallelComm, buf: _LayerBuffers):
        T, H = x.shape
        E, W, C = buf.E, comm.W, capacity
        slot_pos, counts, totals = M.plan_slots(topk_idx, E, C)
        if comm.fused:
            M.dispatch(x, topk_idx, slot_pos, counts, E, C, table=buf.t_disp_x, count_table=buf.t_count)
            comm.barrier()
        else:
            send = M.dispatch(x, topk_idx, slot_pos, counts, E, C)
            comm.exchange_to_owners(send, buf.recv_x)
            comm.exchange_counts(counts, buf.counts)
        need_bwd = any(ctx.needs_input_grad)
        pre = torch.empty(buf.El * W, C, w1.shape[1], dtype=x.dtype, device=x.device) if need_bwd else None
        packed = bool(getattr(w1, "_ats_packed", False))  # serving: expert weights stored tile by tile
        if packed and need_bwd:
            raise RuntimeError("expert weights are packed for serving; the backward pass needs the plain layout")
        from ..ops import fp8  # with the fp8 recipe on, the expert products (and the input gradient below) run in e4m3
        h = fp8.grouped_nt(buf.recv_x, w1, buf.counts, swiglu=True, pre_act=pre, b_div=W)
        if comm.fused and comm.pull_results:
            fp8.grouped_nt(h, w2, buf.counts, b_div=W, out=buf.own_y)
            comm.barrier()
            out = M.combine(buf.ret_y, topk_idx, slot_pos, topk_w, T, residual, table=buf.t_pull_y, keep_copy=True)
        else:
            if comm.fused:
                G.grouped_nt(h, w2, buf.counts, b_div=W, d_table=buf.t_ret_y, packed=packed)
                comm.barrier()
            else:
                ye = G.grouped_nt(h, w2, buf.counts, b_div=W, packed=packed)
                comm.exchange_to_sources(ye, buf.ret_y)
            out = M.combine(buf.ret_y, topk_idx, slot_pos, topk_w, T, residual)
        ctx.save_for_backward(topk_idx, slot_pos, counts, topk_w, w1, w2, pre)
        ctx.comm, ctx.buf, ctx.capacity, ctx.has_res = comm, buf, capacity, residual is not None
        ctx.mark_non_differentiable(totals)
        return out, totals

    @staticmethod
    def backward(ctx, dout, _dt=None):
        topk_idx, slot_pos, counts, topk_w, w1, w2, pre = ctx.saved_tensors
        comm, buf, C = ctx.comm, ctx.buf, ctx.capacity
        E, W = buf.E, comm.W
        T = dout.shape[0]
        inter = w2.shape[2]
        dout = dout.contiguous()
        dw_topk = M.slot_dot(buf.ret_y, topk_idx, slot_pos, dout) if ctx.needs_input_grad[2] else None
        scale = topk_w.contiguous().float()
        if comm.fused:
            M.dispatch(dout, topk_idx, slot_pos, counts, E, C, slot_scale=scale, table=buf.t_disp_g)
            comm.barrier()
        else:
            send = M.dispatch(dout, topk_idx, slot_pos, counts, E, C, slot_scale=scale)
            comm.exchange_to_owners(send, buf.recv_g)
        if M.FUSED_SWIGLU_BWD or not _lib.use_cuda_kernels(pre):
            dgu, h = G.grouped_nn_swiglu_bwd(buf.recv_g, w2, buf.counts, pre, b_div=W)  # dh and the SwiGLU backward in one kernel
        else:
            dh = G.grouped_nn(buf.recv_g, w2, buf.counts, b_div=W)
            dgu = torch.empty_like(pre)
            h = torch.empty(buf.El * W, C, inter, dtype=pre.dtype, device=pre.device)
            _CK(_L().ats_swiglu_bwd_grouped(_P(pre), _P(dh), _P(dgu), _P(h), buf.El * W, C, _P(buf.counts), inter, _S(pre.device)),
                "swiglu_bwd")
        dw2 = _deliver_grad(w2, lambda out, acc: G.grouped_tn(buf.recv_g, h, buf.counts, out=out, accumulate=acc, k_segs=W))
        dw1 = _deliver_grad(w1, lambda out, acc: G.grouped_tn(dgu, buf.recv_x, buf.counts, out=out, accumulate=acc, k_segs=W))
        if comm.fused and comm.pull_results:
            from ..ops import fp8
            fp8.grouped_nn(dgu, w1, buf.counts, b_div=W, out=buf.own_dx)
            comm.barrier()
            dx = M.combine(buf.ret_dx, topk_idx, slot_pos, None, T, None, table=buf.t_pull_dx)
        else:
            if comm.fused:
                G.grouped_nn(dgu, w1, buf.counts, b_div=W, d_table=buf.t_ret_dx)
                comm.barrier()
            else:
                dxe = G.grouped_nn(dgu, w1, buf.counts, b_div=W)
                comm.exchange_to_sources(dxe, buf.ret_dx)
            dx = M.combine(buf.ret_dx, topk_idx, slot_pos, None, T, None)
        return dx, None, dw_topk, dw1, dw2, None, (dout if ctx.has_res else None), None, None


def _down_proj_slices(n_groups: int, N: int, K: int) -> int:
    """Reduction slices for a skinny grouped product with few output tiles: enough (group, slice) work items for all SMs."""
    tiles = n_groups * ((N + 255) // 256)
    s = 1
    while s * 2 * tiles <= 160 and K % (s * 2 * 64) == 0 and K // (s * 2) >= 512 and s < 16:
        s *= 2
    return s


@torch.no_grad()
def ep_moe_serving(x, wg, top_k, temperature, w1, w2, residual, comm: "ExpertParallelComm", buf: _ServingBuffers, next_norm=None):
    """One MoE layer of a decode step across the expert-parallel ranks, six launches between two flag barriers:

    gate + route -> slot plan + dispatch (token rows go straight into the owners' row blocks over NVLink) -> barrier ->
    grouped SwiGLU up-projection over one 128/256-row block per local expert -> down-projection with the reduction cut into
    slices so that every SM streams part of the weight (+ fold) -> barrier -> combine (the source ranks pull their rows from
    the owners).

    Each rank brings its OWN sequences (the batch is split over the ranks, each keeps the KV cache of its sequences); the
    experts see the rows of all ranks.  Nothing is dropped and no row counts are exchanged."""
    T, H = x.shape
    E, Cs = buf.E, buf.Cs
    idx, w = M.serve_gate_route(x, wg, top_k, temperature)
    slot_pos, _, _ = M.serve_plan_dispatch(x, idx, E, Cs, table=buf.t_disp_x, want_counts=False)
    comm.barrier()
    packed = bool(getattr(w1, "_ats_packed", False))
    h = G.grouped_nt(buf.recv_x, w1, buf.counts, swiglu=True, packed=packed)
    ks = _down_proj_slices(buf.El, w2.shape[1], w2.shape[2])
    if ks > 1 and FLAG_SYNC:
        # the launch that folds the slices of the down projection raises this rank's flag on every peer, and the combine kernels
        # wait for the owners they read from: the second barrier launch of the layer is gone
        def fold(part, splits, n_inner, n_outer, out_rows):
            from .peer import _L as _PL
            _lib.check(_PL().ats_splitk_reduce_signal(_lib.ptr(part), splits, n_inner, n_outer, _lib.ptr(out_rows), _lib.ptr(buf.sync_state[1:]),
                                                      _lib.ptr(buf.sync_state), buf.flag_table, comm.rank, comm.W,
                                                      _lib.stream_ptr(x.device)), "splitk_reduce_signal")
        G.grouped_nt(h, w2, buf.counts, out=buf.own_y, packed=packed, k_split=ks, fold=fold)
        out = M.serve_combine(idx, slot_pos, w, T, H, x.dtype, x.device, table=buf.t_pull_y, residual=residual, next_norm=next_norm,
                              wait=(buf.ready_flags, buf.sync_state, buf.El))
        return out, None
    G.grouped_nt(h, w2, buf.counts, out=buf.own_y, packed=packed, k_split=ks)
    comm.barrier()
    out = M.serve_combine(idx, slot_pos, w, T, H, x.dtype, x.device, table=buf.t_pull_y, residual=residual, next_norm=next_norm)
    return out, None   # with next_norm, out is the pair (output, normalised output)


class EPLayer:
    """Bound to one MoE layer as ``layer.ep``; ``moe_ffn`` has the signature of the local MoE function."""

    def __init__(self, comm: ExpertParallelComm, layer_idx: int, num_experts: int):
        self.comm, self.layer_idx, self.num_experts = comm, layer_idx, num_experts

    def moe_serving(self, x, wg, top_k, temperature, w1, w2, residual=None, next_norm=None):
        """Decode-sized step (no autograd): one row block per expert, all layers share one set of buffers.  Returns ``None``
        when the step does not fit that layout (the caller then takes the general path)."""
        cs = self.comm.serving_rows(x.shape[0])
        if not cs:
            return None
        buf = self.comm.serving_buffers(self.num_experts, cs, x.shape[1], x.dtype, x.device)
        return ep_moe_serving(x, wg, top_k, temperature, w1, w2, residual, self.comm, buf, next_norm)

    def moe_ffn(self, x, topk_idx, topk_w, w1, w2, capacity, residual=None):
        # Training keeps one set of exchange buffers per layer (the backward pass reads what the forward pass received).
        # Without autograd nothing outlives the layer call, and the barriers inside it order every reuse, so all layers share
        # one set: a 64 x 1024-token prefill needs 12 GiB of buffers once instead of once per layer.
        key = self.layer_idx if torch.is_grad_enabled() else -1
        buf = self.comm.buffers(key, self.num_experts, capacity, x.shape[1], x.dtype, x.device)
        return _EPMoEFn.apply(x, topk_idx, topk_w, w1, w2, capacity, residual, self.comm, buf)


def attach_expert_parallel(model, mesh, cfg=None, use_fused: bool = True):
    """Wire every MoE layer of ``model`` to the expert-parallel transport of ``mesh``.  Returns the peer-memory
    communicator for the optimiser step (``None`` on the NCCL/Gloo baseline path)."""
    fused_ok = bool(use_fused) and torch.cuda.is_available()
    if fused_ok:
        from .peer import peers_available
        fused_ok = peers_available(None)
    if mesh.ep_size > 1:
        comm = ExpertParallelComm(mesh, fused=fused_ok)
        for layer in model.get_moe_layers():
            layer.ep = EPLayer(comm, layer.layer_idx, layer.num_experts)
        model._ep_comm = comm
    if fused_ok and mesh.world > 1:
        from .fused import FusedComm
        return FusedComm(mesh)
    return None

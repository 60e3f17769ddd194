"""Mixture-of-Experts operators: gate projection, routing, and the dispatch -> grouped SwiGLU FFN -> combine
block as one autograd function.

Routing semantics (documented behaviour of the reference, ``core/model.py:1169-1263``): gate logits (+ optional
Gaussian noise while training) / temperature -> softmax over ALL experts -> top-k -> the kept probabilities are
renormalised to sum to one.  Auxiliary loss ``E * sum_e f_e * P_e * weight`` with ``f_e`` the fraction of
(token, k) slots routed to expert ``e`` and ``P_e`` the mean softmax probability of the clean logits.

Capacity: every expert accepts at most ``C = ceil(capacity_factor * k * T / E)`` slots (rounded up to a
multiple of 128 rows so GEMM tiles are whole); slots are ranked in token order, later ones are dropped.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as G
from .functional import _L, _P, _S, _CK, _deliver_grad


# SwiGLU backward of the expert FFN inside the epilogue of the dh GEMM (default; measured 1 % faster per step once the epilogue
# reads and writes whole 32-byte sectors) or, with ATS_SWIGLU_BWD_FUSED=0, as a separate streaming kernel after the GEMM.
FUSED_SWIGLU_BWD = os.environ.get("ATS_SWIGLU_BWD_FUSED", "1") == "1"


def expert_capacity(tokens: int, num_experts: int, top_k: int, capacity_factor: float, drop_tokens: bool = True,
                    multiple: int = 128) -> int:
    if drop_tokens:
        c = int(math.ceil(capacity_factor * top_k * tokens / num_experts))
    else:
        c = tokens  # dropless: an expert can receive every token once
    c = max(c, 1)
    return ((c + multiple - 1) // multiple) * multiple


# ----------------------------------------------------------------------------------------------------------
# gate projection
# ----------------------------------------------------------------------------------------------------------
class _GateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wg):
        T, H = x.shape
        E = wg.shape[0]
        if T >= 256 and E % 8 == 0 and H % 64 == 0 and x.is_contiguous() and wg.is_contiguous():
            # tensor cores, fp32 logits: the 256-column tile is mostly padding (rows of wg beyond E read as zeros), yet the
            # product then costs about one pass over x, a third of the CUDA-core kernel's time
            logits = G.gemm_nt(x, wg, out_fp32=True)
        else:
            logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
            _CK(_L().ats_gate_fwd(_P(x), _P(wg), _P(logits), T, H, E, _S(x.device)), "gate_fwd")
        ctx.save_for_backward(x, wg)
        return logits

    @staticmethod
    def backward(ctx, dlogits):
        x, wg = ctx.saved_tensors
        T, H = x.shape
        E = wg.shape[0]
        dl = dlogits.contiguous().float()
        dx = torch.empty_like(x)
        _CK(_L().ats_gate_bwd_dx(_P(dl), _P(wg), _P(dx), T, H, E, 0, _S(x.device)), "gate_bwd_dx")
        nb = max(1, min(296, T // 16))
        partial = torch.empty(nb, E * H, dtype=torch.float32, device=x.device)
        _CK(_L().ats_gate_bwd_dw(_P(dl), _P(x), _P(partial), nb, T, H, E, _S(x.device)), "gate_bwd_dw")

        def compute(out, acc):
            if out is None:
                out = torch.empty_like(wg)
            _CK(_L().ats_colsum_partial(_P(partial), nb, E * H, _P(out), None, 1 if acc else 0, _S(x.device)), "gate_dw_reduce")
            return out
        return dx, _deliver_grad(wg, compute)


def gate_logits(x: torch.Tensor, wg: torch.Tensor) -> torch.Tensor:
    """fp32 router logits x[T,H] @ wg[E,H]^T."""
    if _lib.use_cuda_kernels(x) and wg.shape[0] <= 64 and x.shape[1] % 8 == 0:
        return _GateFn.apply(x.contiguous(), wg)
    return F.linear(x.float(), wg.float())


def route(logits: torch.Tensor, top_k: int, temperature: float = 1.0, noise_std: float = 0.0,
          training: bool = False, generator: Optional[torch.Generator] = None):
    """-> (topk_idx int32 [T,k], topk_w fp32 [T,k], clean_probs fp32 [T,E])."""
    clean_probs = torch.softmax(logits, dim=-1)
    z = logits
    if training and noise_std > 0:
        z = z + torch.randn(z.shape, device=z.device, dtype=z.dtype, generator=generator) * noise_std
    if not torch.is_grad_enabled() and logits.is_cuda and not (training and noise_std > 0) and logits.shape[1] <= 64 and top_k <= 8:
        T, E = logits.shape
        probs = torch.empty_like(logits)
        idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        _CK(_L().ats_topk_softmax(_P(logits.contiguous()), _P(probs), _P(idx), _P(w), T, E, top_k, float(temperature),
                                  _S(logits.device)), "topk_softmax")
        return idx, w, clean_probs
    probs = torch.softmax(z / temperature, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True).clamp(min=1e-20)
    return idx.to(torch.int32), w, clean_probs


class _RouteFn(torch.autograd.Function):
    """Soft-max, top-k, renormalised weights and the load-balancing loss in two launches (one more in the backward), instead
    of some thirty small tensor operations."""

    @staticmethod
    def forward(ctx, logits, top_k, temperature, weight):
        T, E = logits.shape
        lg = logits.contiguous()
        dev = lg.device
        probs = torch.empty_like(lg)
        clean = torch.empty_like(lg) if temperature != 1.0 else None
        idx = torch.empty(T, top_k, dtype=torch.int32, device=dev)
        w = torch.empty(T, top_k, dtype=torch.float32, device=dev)
        part = torch.empty((T + 255) // 256 * 2 * E, dtype=torch.float32, device=dev)
        stats = torch.empty(2 * E + 2, dtype=torch.float32, device=dev)
        _CK(_L().ats_route_fwd(_P(lg), _P(probs), _P(clean), _P(idx), _P(w), _P(part), _P(stats), T, E, top_k, float(temperature),
                               float(weight), _S(dev)), "route_fwd")
        ctx.save_for_backward(probs, clean, idx, w, stats) if clean is not None else ctx.save_for_backward(probs, idx, w, stats)
        ctx.args = (top_k, float(temperature), float(weight), clean is not None)
        ctx.mark_non_differentiable(idx)
        aux = stats[2 * E].clone()
        return idx, w, aux

    @staticmethod
    def backward(ctx, _didx, dw, daux):
        top_k, temperature, weight, has_clean = ctx.args
        if has_clean:
            probs, clean, idx, w, stats = ctx.saved_tensors
        else:
            probs, idx, w, stats = ctx.saved_tensors
            clean = None
        T, E = probs.shape
        dlogits = torch.empty_like(probs)
        dwc = dw.contiguous().float() if dw is not None else None
        dac = daux.reshape(1).float().contiguous() if daux is not None else None
        _CK(_L().ats_route_bwd(_P(probs), _P(clean), _P(idx), _P(w), _P(dwc), _P(dac), _P(stats), _P(dlogits), T, E, top_k,
                               temperature, weight, _S(probs.device)), "route_bwd")
        return dlogits, None, None, None


def route_and_balance(logits: torch.Tensor, top_k: int, temperature: float, weight: float):
    """-> (topk_idx int32 [T,k], topk_w fp32 [T,k], load-balancing loss) with one fused forward / backward on CUDA; elsewhere
    ``route`` + ``load_balancing_loss``."""
    if logits.is_cuda and logits.dtype == torch.float32 and logits.shape[1] <= 64 and top_k <= 8:
        return _RouteFn.apply(logits, top_k, temperature, weight)
    idx, w, clean = route(logits, top_k, temperature, 0.0, False)
    return idx, w, load_balancing_loss(clean, idx, logits.shape[1], weight)


def load_balancing_loss(clean_probs: torch.Tensor, topk_idx: torch.Tensor, num_experts: int, weight: float,
                        token_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """E * sum_e f_e * P_e * weight, clamped to <= 1 (reference ``core/model.py:1244-1263``)."""
    flat = topk_idx.reshape(-1).long()
    # scatter-add instead of bincount: no device-to-host synchronisation (bincount reads back the maximum), so the host keeps
    # running ahead of the GPU and the step can be captured in a CUDA graph
    counts = torch.zeros(num_experts, dtype=torch.float32, device=flat.device).scatter_add_(
        0, flat, torch.ones(flat.numel(), dtype=torch.float32, device=flat.device))
    f = counts / max(flat.numel(), 1)
    p = clean_probs.mean(0)
    return (num_experts * (f * p).sum() * weight).clamp(max=1.0)


# ----------------------------------------------------------------------------------------------------------
# slot planning (deterministic) -- shared by the CUDA and the PyTorch bodies
# ----------------------------------------------------------------------------------------------------------
def plan_slots(topk_idx: torch.Tensor, num_experts: int, capacity: int):
    """-> slot_pos int32 [T*k] (row inside the expert region or -1), counts int32 [E] (clamped), totals int32 [E]."""
    flat = topk_idx.reshape(-1).contiguous()
    if flat.is_cuda and num_experts <= 64:
        slot_pos = torch.empty(flat.numel(), dtype=torch.int32, device=flat.device)
        counts = torch.empty(num_experts, dtype=torch.int32, device=flat.device)
        totals = torch.empty(num_experts, dtype=torch.int32, device=flat.device)
        if flat.numel() > 4096:  # many slots: two multi-CTA passes instead of one CTA walking the whole list
            chunk_cnt = torch.empty((flat.numel() + 1023) // 1024 * num_experts, dtype=torch.int32, device=flat.device)
            _CK(_L().ats_plan_slots_chunked(_P(flat), _P(slot_pos), _P(counts), _P(totals), _P(chunk_cnt), flat.numel(), num_experts,
                                            capacity, _S(flat.device)), "plan_slots_chunked")
        else:
            _CK(_L().ats_plan_slots(_P(flat), _P(slot_pos), _P(counts), _P(totals), flat.numel(), num_experts, capacity,
                                    _S(flat.device)), "plan_slots")
        return slot_pos, counts, totals
    oh = F.one_hot(flat.long(), num_experts)
    rank = (oh.cumsum(0) - oh).gather(1, flat.long()[:, None]).squeeze(1)
    totals = oh.sum(0).to(torch.int32)
    slot_pos = torch.where(rank < capacity, rank, torch.full_like(rank, -1)).to(torch.int32)
    return slot_pos, totals.clamp(max=capacity), totals


def _ptr_table(t: torch.Tensor) -> torch.Tensor:
    """int64 device table with the base address of every expert region of t[E, C, H]."""
    E = t.shape[0]
    step = t.stride(0) * t.element_size()
    return torch.arange(E, dtype=torch.int64, device=t.device) * step + t.data_ptr()


def dispatch(x: torch.Tensor, topk_idx: torch.Tensor, slot_pos: torch.Tensor, counts: torch.Tensor,
             num_experts: int, capacity: int, slot_scale: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None,
             count_table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[T,H] -> buf[E, C, H] with row ``slot_pos`` of expert ``topk_idx`` holding (scaled) x[t]."""
    T, H = x.shape
    k = topk_idx.shape[1]
    if out is None and table is None:
        out = torch.empty(num_experts, capacity, H, dtype=x.dtype, device=x.device)
    if _lib.use_cuda_kernels(x):
        if table is None:
            table = _ptr_table(out)
        _CK(_L().ats_dispatch_rows(_P(x), _P(topk_idx), _P(slot_pos), _P(slot_scale), _P(table), _P(counts),
                                   _P(count_table), T * k, k, H, num_experts, capacity, 1, _S(x.device)), "dispatch_rows")
        return out
    out.zero_()
    flat_e = topk_idx.reshape(-1).long()
    pos = slot_pos.long()
    keep = pos >= 0
    tok = torch.arange(T * k, device=x.device) // k
    rows = x[tok[keep]]
    if slot_scale is not None:
        rows = (rows.float() * slot_scale.reshape(-1)[keep][:, None]).to(x.dtype)
    out[flat_e[keep], pos[keep]] = rows
    return out


def combine(buf: torch.Tensor, topk_idx: torch.Tensor, slot_pos: torch.Tensor, topk_w: Optional[torch.Tensor],
            tokens: int, residual: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None,
            keep_copy: bool = False) -> torch.Tensor:
    """out[t] = residual[t] + sum_j w[t,j] * buf[e_j, pos_j] over kept slots.  ``table`` (int64 [E]) replaces the base address
    of every expert's rows (e.g. buffers on the GPUs that own the experts: the rows are then pulled over NVLink);
    ``keep_copy`` stores the pulled rows into ``buf`` as well."""
    E, C, H = buf.shape
    k = topk_idx.shape[1]
    if _lib.use_cuda_kernels(buf):
        out = torch.empty(tokens, H, dtype=buf.dtype, device=buf.device)
        copy_table = _ptr_table(buf) if (keep_copy and table is not None) else None
        if table is None:
            table = _ptr_table(buf)
        w = topk_w.contiguous().float() if topk_w is not None else None
        _CK(_L().ats_combine_rows(_P(table), _P(copy_table), _P(topk_idx), _P(slot_pos), _P(w), _P(residual), _P(out), tokens, k, H,
                                  _S(buf.device)), "combine_rows")
        return out
    flat_e = topk_idx.reshape(-1).long()
    pos = slot_pos.long()
    keep = pos >= 0
    rows = torch.zeros(tokens * k, H, dtype=torch.float32, device=buf.device)
    rows[keep] = buf[flat_e[keep], pos[keep]].float()
    if topk_w is not None:
        rows = rows * topk_w.reshape(-1, 1).float()
    out = rows.view(tokens, k, H).sum(1)
    if residual is not None:
        out = out + residual.float()
    return out.to(buf.dtype)


def slot_dot(buf: torch.Tensor, topk_idx: torch.Tensor, slot_pos: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """<dout[t], buf[e_j, pos_j]> for every slot -> [T, k] fp32 (gradient of the combine weights)."""
    T, H = dout.shape
    k = topk_idx.shape[1]
    if _lib.use_cuda_kernels(buf):
        dw = torch.empty(T, k, dtype=torch.float32, device=buf.device)
        _CK(_L().ats_slot_dot(_P(_ptr_table(buf)), _P(topk_idx), _P(slot_pos), _P(dout.contiguous()), _P(dw), T * k, k, H,
                              _S(buf.device)), "slot_dot")
        return dw
    flat_e = topk_idx.reshape(-1).long()
    pos = slot_pos.long()
    keep = pos >= 0
    rows = torch.zeros(T * k, H, dtype=torch.float32, device=buf.device)
    rows[keep] = buf[flat_e[keep], pos[keep]].float()
    return (rows.view(T, k, H) * dout.float()[:, None, :]).sum(-1)


# ----------------------------------------------------------------------------------------------------------
# dispatch -> experts -> combine
# ----------------------------------------------------------------------------------------------------------
class _MoEFFNFn(torch.autograd.Function):
    """y[t] = residual[t] + sum_j w[t,j] * FFN_{e_j}(x[t]) under a capacity limit.

    ``w1``: [E, 2I, H] (gate rows then up rows), ``w2``: [E, H, I].  Saved for backward: the dispatched inputs,
    the SwiGLU pre-activations and the expert outputs (needed for the combine-weight gradient)."""

    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w1, w2, capacity, residual):
        T, H = x.shape
        E = w1.shape[0]
        slot_pos, counts, totals = plan_slots(topk_idx, E, capacity)
        xe = dispatch(x, topk_idx, slot_pos, counts, E, capacity)
        need_bwd = any(ctx.needs_input_grad)
        pre = torch.empty(E, capacity, w1.shape[1], dtype=x.dtype, device=x.device) if need_bwd else None
        packed = bool(getattr(w1, "_ats_packed", False))  # serving: expert weights stored tile by tile (GenerationEngine)
        if packed and need_bwd:
            raise RuntimeError("expert weights are packed for serving; the backward pass needs the plain layout")
        from . import fp8  # the fp8 recipe (when switched on) runs both expert products and the input gradient in e4m3
        h = fp8.grouped_nt(xe, w1, counts, swiglu=True, pre_act=pre)
        ye = fp8.grouped_nt(h, w2, counts)
        out = combine(ye, topk_idx, slot_pos, topk_w, T, residual)
        ctx.save_for_backward(topk_idx, slot_pos, counts, topk_w, w1, w2, xe, pre, ye)
        ctx.capacity = capacity
        ctx.has_res = residual is not None
        ctx.mark_non_differentiable(totals)
        return out, totals

    @staticmethod
    def backward(ctx, dout, _dtotals=None):
        topk_idx, slot_pos, counts, topk_w, w1, w2, xe, pre, ye = ctx.saved_tensors
        E, C, H = xe.shape
        inter = w2.shape[2]
        T = dout.shape[0]
        dout = dout.contiguous()
        dw_topk = slot_dot(ye, topk_idx, slot_pos, dout) if ctx.needs_input_grad[2] else None
        dye = dispatch(dout, topk_idx, slot_pos, counts, E, C, slot_scale=topk_w.contiguous().float())
        if FUSED_SWIGLU_BWD or not _lib.use_cuda_kernels(pre):
            dgu, h = G.grouped_nn_swiglu_bwd(dye, w2, counts, pre)  # dh = dye · w2 never leaves the GEMM: its epilogue does the SwiGLU backward
        else:
            dh = G.grouped_nn(dye, w2, counts)
            dgu = torch.empty_like(pre)
            h = torch.empty(E, C, inter, dtype=pre.dtype, device=pre.device)
            _CK(_L().ats_swiglu_bwd_grouped(_P(pre), _P(dh), _P(dgu), _P(h), E, C, _P(counts), inter, _S(pre.device)), "swiglu_bwd")
        dw2 = _deliver_grad(w2, lambda out, acc: G.grouped_tn(dye, h, counts, out=out, accumulate=acc))
        dw1 = _deliver_grad(w1, lambda out, acc: G.grouped_tn(dgu, xe, counts, out=out, accumulate=acc))
        from . import fp8
        dxe = fp8.grouped_nn(dgu, w1, counts)
        dx = combine(dxe, topk_idx, slot_pos, None, T, None)
        return dx, None, dw_topk, dw1, dw2, None, (dout if ctx.has_res else None)


# ----------------------------------------------------------------------------------------------------------
# decode-sized steps (serving): three small launches around the two grouped GEMMs
# ----------------------------------------------------------------------------------------------------------
SERVE_MAX_SLOTS = 1024


def serving_path_ok(x: torch.Tensor, num_experts: int, top_k: int) -> bool:
    """A step small enough for the serving kernels: no autograd, bf16 on the GPU, at most 1024 (token, k) slots."""
    return (not torch.is_grad_enabled() and _lib.use_cuda_kernels(x) and x.dim() == 2 and x.shape[0] * top_k <= SERVE_MAX_SLOTS
            and num_experts <= 64 and top_k <= 8 and x.shape[1] % 8 == 0 and x.is_contiguous())


def serve_gate_route(x: torch.Tensor, wg: torch.Tensor, top_k: int, temperature: float):
    """x [T, H], gate weight [E, H] -> (topk_idx int32 [T, k], topk_w fp32 [T, k]): logits, soft-max over all experts at the
    routing temperature, top-k and renormalisation in one launch."""
    T, H = x.shape
    E = wg.shape[0]
    idx = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
    _CK(_L().ats_serve_gate_route(_P(x), _P(wg.contiguous()), _P(idx), _P(w), T, H, E, top_k, float(temperature), _S(x.device)),
        "serve_gate_route")
    return idx, w


def serve_plan_dispatch(x: torch.Tensor, topk_idx: torch.Tensor, num_experts: int, capacity: int, out: Optional[torch.Tensor] = None,
                        table: Optional[torch.Tensor] = None, want_counts: bool = True):
    """Slot plan (rank of every (token, k) slot among the earlier slots of its expert) and row copy in one launch.
    -> (slot_pos int32 [T * k], counts int32 [E] or None, totals int32 [E] or None).  Rows go to ``out`` [E, C, H] or,
    with ``table`` (int64 [E] base addresses), to blocks that may live on peer GPUs.  Rows that no slot uses are not
    touched: their products are never read."""
    T, H = x.shape
    k = topk_idx.shape[1]
    slot_pos = torch.empty(T * k, dtype=torch.int32, device=x.device)
    counts = torch.empty(num_experts, dtype=torch.int32, device=x.device) if want_counts else None
    totals = torch.empty(num_experts, dtype=torch.int32, device=x.device) if want_counts else None
    stride = out.stride(0) if out is not None else 0
    _CK(_L().ats_serve_plan_dispatch(_P(x), _P(topk_idx), _P(slot_pos), _P(counts), _P(totals), _P(table), _P(out) if table is None else None,
                                     stride, T, k, H, num_experts, capacity, _S(x.device)), "serve_plan_dispatch")
    return slot_pos, counts, totals


def serve_combine(topk_idx: torch.Tensor, slot_pos: torch.Tensor, topk_w: torch.Tensor, tokens: int, hidden: int, dtype, device,
                  buf: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, next_norm=None, wait=None):
    """out[t] = residual[t] + sum_j w[t, j] * row(e_j, pos_j); one CTA per token.  Rows come from ``buf`` [E, C, H] or from the
    blocks ``table`` points to (pulled over NVLink when they live on the experts' owners).  ``next_norm`` = (weight, eps): the same
    launch also writes RMSNorm(out) * weight, the input of the next block, and the result is ``(out, normed)``.  ``wait`` =
    (flags int32 [W], epoch int32 [1], experts per rank): the kernel waits for the flag of every owner it pulls from."""
    out = torch.empty(tokens, hidden, dtype=dtype, device=device)
    k = topk_idx.shape[1]
    stride = buf.stride(0) if buf is not None else 0
    fuse = next_norm is not None and next_norm[0].dtype == dtype and dtype == torch.bfloat16
    normed = torch.empty_like(out) if fuse else None
    _CK(_L().ats_serve_combine(_P(table), _P(buf) if table is None else None, stride, _P(topk_idx), _P(slot_pos), _P(topk_w),
                               _P(residual), _P(out), tokens, k, hidden, _P(next_norm[0]) if fuse else None, _P(normed),
                               float(next_norm[1]) if fuse else 0.0, _P(wait[0]) if wait else None, _P(wait[1]) if wait else None,
                               int(wait[2]) if wait else 0, _P(_lib.status_tensor(device)) if wait else None, _S(device)), "serve_combine")
    if next_norm is not None:
        return out, normed   # normed is None when the fused form did not apply: the caller normalises as usual
    return out


@torch.no_grad()
def moe_ffn_serving(x: torch.Tensor, wg: torch.Tensor, top_k: int, temperature: float, w1: torch.Tensor, w2: torch.Tensor,
                    residual: Optional[torch.Tensor] = None, next_norm=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One MoE layer of a decode-sized step on one GPU: gate + route, plan + dispatch, grouped SwiGLU up-projection, grouped
    down-projection, combine -- five launches.  Dropless (every expert block has room for every token).
    -> (output [T, H], demand per expert int32 [E])."""
    T, H = x.shape
    E = w1.shape[0]
    C = (T + 127) // 128 * 128
    idx, w = serve_gate_route(x, wg, top_k, temperature)
    from . import fp8
    packed = bool(getattr(w1, "_ats_packed", False))
    if fp8.enabled() and not packed and fp8.grouped_usable(x, w1.shape[1], w1.shape[2]) and w2.shape[2] % 16 == 0:
        # post-training e4m3 experts: both products stream half the bytes (rows no token uses are zero so that their scales stay finite)
        xe = torch.zeros(E, C, H, dtype=x.dtype, device=x.device)
        slot_pos, counts, totals = serve_plan_dispatch(x, idx, E, C, out=xe)
        h = fp8.grouped_nt(xe, w1, counts, swiglu=True)
        ye = fp8.grouped_nt(h, w2, counts)
    else:
        xe = torch.empty(E, C, H, dtype=x.dtype, device=x.device)
        slot_pos, counts, totals = serve_plan_dispatch(x, idx, E, C, out=xe)
        h = G.grouped_nt(xe, w1, counts, swiglu=True, packed=packed)
        ye = G.grouped_nt(h, w2, counts, packed=packed)
    out = serve_combine(idx, slot_pos, w, T, H, x.dtype, x.device, buf=ye, residual=residual, next_norm=next_norm)
    return out, totals   # with next_norm, out is the pair (output, normalised output)


def moe_ffn(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
            capacity: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (output [T,H], demand per expert int32 [E])."""
    return _MoEFFNFn.apply(x, topk_idx, topk_w, w1, w2, capacity, None)


def moe_ffn_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, w1: torch.Tensor,
                      w2: torch.Tensor, capacity: int) -> torch.Tensor:
    """Per-expert loop in fp32 with the same capacity rule; the oracle for tests."""
    T, H = x.shape
    E = w1.shape[0]
    k = topk_idx.shape[1]
    slot_pos, _, _ = plan_slots(topk_idx, E, capacity)
    keep = (slot_pos >= 0).view(T, k)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = (topk_idx.long() == e) & keep
        tok, kk = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok].float()
        gu = xe @ w1[e].float().t()
        g, u = gu.chunk(2, dim=-1)
        ye = (F.silu(g) * u) @ w2[e].float().t()
        out.index_add_(0, tok, ye * topk_w[tok, kk].float()[:, None])
    return out.to(x.dtype)

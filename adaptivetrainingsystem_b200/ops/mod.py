"""Mixture-of-Depths token routing on the training path (``csrc/mod.cu``): two autograd functions around the dense SwiGLU MLP.

``route``   h [B, L, H] -> the rows of the ``keep`` best-scored tokens of every sequence (ascending positions), their sigmoid
            weights, the auxiliary loss that teaches sigmoid(score) to predict membership, and the bookkeeping.
``scatter`` out = base + scatter(weight * y): every unselected token keeps the residual stream.

Backward makes each gradient once: ``dh`` is written by one kernel (router term + gathered rows), the router weight / bias
gradient by one column reduction, ``dy`` and the weight gradient by one kernel per selected row.

Reference semantics: ``core/model.py:860-1020`` (router ``nn.Linear(H, 1)``, top-k by score, output weighted by the sigmoid of
the score, BCE auxiliary loss against membership); there the selection runs over the whole batch with ``torch.topk`` and the
rows move through boolean masks and ``index_add_``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .functional import _L, _P, _S, _CK

MAX_SEQ = 8192  # the selection kernel ranks one sequence in shared memory


def kernel_path_ok(h: torch.Tensor, seq_len: int) -> bool:
    return h.is_cuda and h.dtype == torch.bfloat16 and h.shape[-1] % 8 == 0 and h.shape[-1] <= 16384 and seq_len <= MAX_SEQ


class _RouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, b, inv_temp: float, keep: int):
        B, L, H = h.shape
        h2 = h.contiguous()
        dev = h.device
        scores = torch.empty(B, L, dtype=torch.float32, device=dev)
        lib, st = _L(), _S(dev)
        wb = w.to(torch.bfloat16).contiguous()
        bb = b.to(torch.bfloat16).contiguous() if b is not None else None
        _CK(lib.ats_mod_scores(_P(h2), _P(wb), _P(bb), _P(scores), B * L, H, float(inv_temp), st), "mod_scores")
        sel = torch.empty(B, keep, dtype=torch.int32, device=dev)
        member = torch.empty(B * L, dtype=torch.int32, device=dev)
        _CK(lib.ats_mod_select(_P(scores), _P(sel), _P(member), B, L, keep, st), "mod_select")
        picked = torch.empty(B, keep, H, dtype=h.dtype, device=dev)
        weight = torch.empty(B, keep, dtype=torch.float32, device=dev)
        slot_of = torch.full((B * L,), -1, dtype=torch.int32, device=dev)
        aux = torch.empty((), dtype=torch.float32, device=dev)
        _CK(lib.ats_mod_gather(_P(h2), _P(sel), _P(scores), _P(picked), _P(weight), _P(slot_of), _P(aux), B, L, keep, H, st), "mod_gather")
        ctx.save_for_backward(h2, wb, scores, slot_of)
        ctx.inv_temp, ctx.has_bias, ctx.w_dtype, ctx.b_dtype = float(inv_temp), b is not None, w.dtype, (b.dtype if b is not None else None)
        ctx.w_shape = w.shape
        ctx.mark_non_differentiable(sel, slot_of, scores)
        return picked, weight, aux, sel, slot_of, scores

    @staticmethod
    def backward(ctx, dpicked, dweight, daux, _ds, _dslot, _dsc):
        h2, wb, scores, slot_of = ctx.saved_tensors
        B, L, H = h2.shape
        dev = h2.device
        dh = torch.empty_like(h2)
        ds = torch.empty(B * L, dtype=torch.float32, device=dev)
        dwb = torch.empty(H + 1, dtype=torch.float32, device=dev)  # router weight gradient, then the bias gradient
        partial = torch.empty(_L().ats_mod_wgrad_ctas() * (H + 8), dtype=torch.float32, device=dev)
        dp = dpicked.contiguous() if dpicked is not None else None
        dwt = dweight.contiguous().float() if dweight is not None else None
        da = daux.contiguous().float() if daux is not None else None
        _CK(_L().ats_mod_route_bwd(_P(h2), _P(dp), _P(slot_of), _P(scores), _P(dwt), _P(da), None, _P(wb), _P(dh), _P(ds), _P(dwb),
                                   _P(partial), B * L, H, ctx.inv_temp, _S(dev)), "mod_route_bwd")
        dw = dwb[:H].view(ctx.w_shape).to(ctx.w_dtype)
        db = dwb[H:].to(ctx.b_dtype) if ctx.has_bias else None
        return dh, dw, db, None, None


class _ScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, base, y, weight, sel, slot_of, seq_len: int):
        B, keep, H = y.shape
        T = slot_of.numel()
        y2 = y.contiguous()
        out = torch.empty(B, seq_len, H, dtype=y.dtype, device=y.device)
        b2 = base.contiguous() if base is not None else None
        _CK(_L().ats_mod_scatter(_P(b2), _P(y2), _P(slot_of), _P(weight), _P(out), T, H, _S(y.device)), "mod_scatter")
        ctx.save_for_backward(y2, weight, sel)
        ctx.seq_len, ctx.has_base = seq_len, base is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        y2, weight, sel = ctx.saved_tensors
        B, keep, H = y2.shape
        g = dout.contiguous()
        dy = torch.empty_like(y2)
        dweight = torch.empty(B, keep, dtype=torch.float32, device=y2.device)
        _CK(_L().ats_mod_scatter_bwd(_P(g), _P(y2), _P(sel), _P(weight), _P(dy), _P(dweight), B, ctx.seq_len, keep, H, _S(y2.device)),
            "mod_scatter_bwd")
        return (g if ctx.has_base else None), dy, dweight, None, None, None


def route(h: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], temperature: float, keep: int):
    """-> (picked [B, keep, H], weight [B, keep] fp32, aux scalar, sel [B, keep] int32, slot_of [B*L] int32, scores [B, L] fp32)"""
    return _RouteFn.apply(h, w, b, 1.0 / float(temperature), int(keep))


def scatter(base: Optional[torch.Tensor], y: torch.Tensor, weight: torch.Tensor, sel: torch.Tensor, slot_of: torch.Tensor,
            seq_len: int) -> torch.Tensor:
    return _ScatterFn.apply(base, y, weight, sel, slot_of, int(seq_len))


def route_reference(h: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], temperature: float, keep: int):
    """Plain PyTorch definition of :func:`route` + :func:`scatter`'s inputs (fp32 arithmetic), for tests and CPU runs."""
    scores = (torch.nn.functional.linear(h.float(), w.float().view(1, -1), b.float() if b is not None else None).squeeze(-1)) / temperature
    sel = torch.topk(scores.detach(), keep, dim=1).indices.sort(dim=1).values
    weight = torch.sigmoid(torch.gather(scores, 1, sel))
    target = torch.zeros_like(scores).scatter_(1, sel, 1.0)
    aux = torch.nn.functional.binary_cross_entropy_with_logits(scores, target)
    picked = torch.gather(h, 1, sel.unsqueeze(-1).expand(-1, -1, h.shape[-1]))
    return picked, weight, aux, sel, scores

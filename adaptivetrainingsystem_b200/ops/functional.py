"""Differentiable operators.  Each one has two bodies with identical semantics:

* bf16 CUDA tensors run the hand-written sm_100a kernels (``csrc/*.cu``) through ctypes;
* everything else (CPU, fp32) runs the plain PyTorch definition, which is also the numerical oracle the
  kernel tests compare against.

Semantics follow the reference model (``core/model.py``): RMSNorm in fp32 (``:228-304``), half-split RoPE
(``:470-524``), ``silu(gate) * up`` SwiGLU (``:1082-1088``), embedding clamp + optional sqrt(H) scale
(``:1924-1931``), weighted / masked cross-entropy (``training/trainer.py:2249-2350``).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as G

_c_int, _c_ll, _c_f, _vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
_sig_done = False


def _L():
    """ctypes signatures for the element-wise / loss / optimiser / MoE entry points."""
    global _sig_done
    lib = _lib.cuda_lib()
    if not _sig_done:
        def sig(name, *args):
            f = getattr(lib, name)
            f.restype = _c_int
            f.argtypes = list(args)
        sig("ats_rmsnorm_fwd", _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        sig("ats_rmsnorm_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _vp, _vp, _c_int, _c_ll, _c_int, _vp)
        sig("ats_colsum_partial", _vp, _c_int, _c_int, _vp, _vp, _c_int, _vp)
        sig("ats_rope", _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _vp)
        sig("ats_swiglu_fwd", _vp, _vp, _c_ll, _c_int, _vp)
        sig("ats_swiglu_bwd", _vp, _vp, _vp, _vp, _c_ll, _c_int, _vp)
        sig("ats_swiglu_bwd_grouped", _vp, _vp, _vp, _vp, _c_int, _c_int, _vp, _c_int, _vp)
        sig("ats_embedding_fwd", _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_f, _vp)
        sig("ats_embedding_bwd", _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_f, _c_int, _vp)
        sig("ats_cast_f32_bf16", _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        sig("ats_ce_fwd_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_ll, _c_ll, _vp)
        sig("ats_sumsq", _vp, _c_ll, _c_int, _vp, _vp, _c_int, _vp)
        sig("ats_clip_coef", _vp, _c_f, _c_f, _vp, _vp)
        sig("ats_adamw", _vp, _vp, _vp, _vp, _vp, _c_ll, _vp, _vp, _c_f, _vp)
        sig("ats_gate_fwd", _vp, _vp, _vp, _c_ll, _c_int, _c_int, _vp)
        sig("ats_gate_bwd_dx", _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_int, _vp)
        sig("ats_gate_bwd_dw", _vp, _vp, _vp, _c_int, _c_ll, _c_int, _c_int, _vp)
        sig("ats_topk_softmax", _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_f, _vp)
        sig("ats_route_fwd", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_f, _c_f, _vp)
        sig("ats_route_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_f, _c_f, _vp)
        sig("ats_plan_slots", _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _vp)
        sig("ats_plan_slots_chunked", _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _vp)
        sig("ats_dispatch_rows", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _vp)
        sig("ats_combine_rows", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _vp)
        sig("ats_serve_gate_route", _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_f, _vp)
        sig("ats_serve_plan_dispatch", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _vp)
        sig("ats_serve_combine", _vp, _vp, _c_ll, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _vp, _vp, _c_f, _vp, _vp, _c_int, _vp, _vp)
        sig("ats_slot_dot", _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_int, _vp)
        sig("ats_mod_select", _vp, _vp, _vp, _c_int, _c_int, _c_int, _vp)
        sig("ats_mod_scores", _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        sig("ats_mod_gather", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _vp)
        sig("ats_mod_scatter", _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _vp)
        sig("ats_mod_scatter_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _vp)
        sig("ats_mod_route_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        sig("ats_mod_wgrad_ctas")
        _sig_done = True
    return lib


_P, _S, _CK = _lib.ptr, _lib.stream_ptr, _lib.check
import os as _os

_NORM_BLOCKS = int(_os.environ.get("ATS_NORM_BLOCKS", "1184"))  # CTAs of the row-walking backward kernels (8 per SM keeps enough rows in flight)


# ----------------------------------------------------------------------------------------------------------
# RMSNorm
# ----------------------------------------------------------------------------------------------------------
def rms_norm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows, cols = x2.shape
        # outputs are allocated in their final shape: returning a view made inside a Function would forbid
        # in-place consumers downstream
        y = torch.empty(shape, dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        summed = None
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, cols)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            summed = torch.empty(shape, dtype=x.dtype, device=x.device)
        _CK(_L().ats_rmsnorm_fwd(_P(x2), _P(r2), _P(w), _P(y), _P(summed), _P(rstd), rows, cols, eps, _S(x.device)),
            "rmsnorm_fwd")
        ctx.save_for_backward(summed.view(rows, cols) if summed is not None else x2, w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        if residual is not None:
            return y, summed
        return y

    @staticmethod
    def backward(ctx, dy, dsum=None):
        xin, w, rstd = ctx.saved_tensors
        rows, cols = xin.shape
        dy2 = dy.reshape(rows, cols)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        ds = None
        if ctx.has_res and dsum is not None:
            ds = dsum.reshape(rows, cols)
            if not ds.is_contiguous():
                ds = ds.contiguous()
        dx = torch.empty_like(xin)
        nb = min(_NORM_BLOCKS, rows)
        partial = torch.empty(nb, cols, dtype=torch.float32, device=xin.device)
        dw = torch.empty_like(w)
        _CK(_L().ats_rmsnorm_bwd(_P(xin), _P(w), _P(dy2), _P(rstd), _P(ds), _P(dx), _P(partial), nb, _P(dw), None, 0,
                                 rows, cols, _S(xin.device)), "rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, dw, None, (dxv if ctx.has_res else None)


class _RMSNormSkipFn(torch.autograd.Function):
    """(rms_norm(x), x): the pre-norm pattern, where x also feeds the residual connection.  As one autograd node it receives
    both gradients, and the backward kernel adds the residual branch's gradient while it writes dx (no separate add pass)."""

    @staticmethod
    def forward(ctx, x, w, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows, cols = x2.shape
        y = torch.empty(shape, dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _CK(_L().ats_rmsnorm_fwd(_P(x2), None, _P(w), _P(y), None, _P(rstd), rows, cols, eps, _S(x.device)), "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = shape
        return y, x

    @staticmethod
    def backward(ctx, dy, dskip):
        xin, w, rstd = ctx.saved_tensors
        rows, cols = xin.shape
        dy2 = dy.reshape(rows, cols)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        ds = None
        if dskip is not None:
            ds = dskip.reshape(rows, cols)
            if not ds.is_contiguous():
                ds = ds.contiguous()
        dx = torch.empty_like(xin)
        nb = min(_NORM_BLOCKS, rows)
        partial = torch.empty(nb, cols, dtype=torch.float32, device=xin.device)
        dw = torch.empty_like(w)
        _CK(_L().ats_rmsnorm_bwd(_P(xin), _P(w), _P(dy2), _P(rstd), _P(ds), _P(dx), _P(partial), nb, _P(dw), None, 0,
                                 rows, cols, _S(xin.device)), "rmsnorm_bwd")
        return dx.view(ctx.shape), dw, None


def rms_norm_skip(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """-> (rms_norm(x), x) for the pre-norm residual pattern; use the second value as the residual input downstream."""
    if _lib.use_cuda_kernels(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and torch.is_grad_enabled() and x.requires_grad:
        return _RMSNormSkipFn.apply(x, w, eps)
    return rms_norm(x, w, eps), x


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None):
    """``rms_norm(x)`` -> y, or with ``residual``: returns ``(rms_norm(x + residual), x + residual)``."""
    if _lib.use_cuda_kernels(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _RMSNormFn.apply(x, w, eps, residual)
    if residual is not None:
        s = x + residual
        return rms_norm_reference(s, w, eps), s
    return rms_norm_reference(x, w, eps)


def layer_norm_reference(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        lib = _norm_lib()
        _CK(lib.ats_layernorm_fwd(_P(x2), _P(w), _P(b), _P(y), _P(mean), _P(rstd), rows, H, eps, _S(x.device)), "ats_layernorm_fwd")
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.has_bias, ctx.shape = b is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = dy.reshape(rows, H).contiguous()
        dx = torch.empty_like(x2)
        blocks = max(1, min(rows, _NORM_BLOCKS))
        partials = torch.empty(blocks, 2, H, dtype=torch.float32, device=x2.device)
        dgamma = torch.empty(H, dtype=torch.float32, device=x2.device)
        dbeta = torch.empty(H, dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        _CK(_norm_lib().ats_layernorm_bwd(_P(dy2), _P(x2), _P(w), _P(mean), _P(rstd), _P(dx), _P(partials), blocks, _P(dgamma), _P(dbeta),
                                          rows, H, _S(x2.device)), "ats_layernorm_bwd")
        return dx.view(ctx.shape), dgamma.to(w.dtype), None if dbeta is None else dbeta.to(w.dtype), None


_norm_sig = False


def _norm_lib():
    global _norm_sig
    lib = _lib.cuda_lib()
    if not _norm_sig:
        def sig(name, *args):
            f = getattr(lib, name)
            f.restype = _c_int
            f.argtypes = list(args)
        sig("ats_layernorm_fwd", _vp, _vp, _vp, _vp, _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        sig("ats_layernorm_bwd", _vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _vp, _vp, _c_ll, _c_int, _vp)
        sig("ats_masked_softmax_fwd", _vp, _vp, _vp, _c_ll, _c_int, _c_int, _c_int, _c_f, _c_int, _vp)
        sig("ats_masked_softmax_bwd", _vp, _vp, _vp, _c_ll, _c_int, _c_f, _vp)
        _norm_sig = True
    return lib


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension, optional bias (reference ``core/model.py:307-327``)."""
    if _lib.use_cuda_kernels(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _LayerNormFn.apply(x, w, b, eps)
    return layer_norm_reference(x, w, b, eps)


def masked_softmax_reference(scores: torch.Tensor, mask: Optional[torch.Tensor], scale: float, causal: bool) -> torch.Tensor:
    s = scores.float() * scale
    Lq, Lk = scores.shape[-2], scores.shape[-1]
    if causal:
        qi = torch.arange(Lq, device=s.device)[:, None] + (Lk - Lq)
        s = s.masked_fill(torch.arange(Lk, device=s.device)[None, :] > qi, float("-inf"))
    if mask is not None:
        s = s.masked_fill(mask.bool()[:, None], float("-inf"))
    return torch.nan_to_num(torch.softmax(s, -1)).to(scores.dtype)


class _MaskedSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, mask, scale, causal):
        B, Hh, Lq, Lk = scores.shape
        x = scores.contiguous()
        y = torch.empty_like(x)
        m8 = None if mask is None else mask.to(torch.uint8).contiguous()
        _CK(_norm_lib().ats_masked_softmax_fwd(_P(x), _P(m8), _P(y), B * Hh * Lq, Lk, Hh, Lq, scale, int(causal), _S(x.device)),
            "ats_masked_softmax_fwd")
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dx = torch.empty_like(y)
        _CK(_norm_lib().ats_masked_softmax_bwd(_P(dy.contiguous()), _P(y), _P(dx), y.numel() // y.shape[-1], y.shape[-1], ctx.scale,
                                               _S(y.device)), "ats_masked_softmax_bwd")
        return dx, None, None, None


def masked_softmax(scores: torch.Tensor, mask: Optional[torch.Tensor] = None, scale: float = 1.0, causal: bool = False) -> torch.Tensor:
    """softmax(scale * scores) over keys.  scores: [B, heads, Lq, Lk]; mask: [B, Lq, Lk] with True / 1 = masked out (shared
    by the heads); ``causal`` hides key j > query i + (Lk - Lq).  Fully masked rows give zeros."""
    if _lib.use_cuda_kernels(scores) and scores.dim() == 4:
        return _MaskedSoftmaxFn.apply(scores, mask, float(scale), bool(causal))
    return masked_softmax_reference(scores, mask, scale, causal)


# ----------------------------------------------------------------------------------------------------------
# Linear
# ----------------------------------------------------------------------------------------------------------
_SINK_OWNERS = {}  # data_ptr -> parameter that carries the sink attributes


def register_grad_sink(p: torch.Tensor) -> None:
    """Engines call this for every parameter they give an ``_ats_grad`` view.  Under activation checkpointing the tensors a
    backward function gets back from ``saved_tensors`` are new Python objects without the attributes; the owner is then
    found again by the storage address."""
    _SINK_OWNERS[p.data_ptr()] = p


def _sink_owner(w: torch.Tensor):
    if hasattr(w, "_ats_grad"):
        return w
    o = _SINK_OWNERS.get(w.data_ptr())
    if o is not None and o.shape == w.shape and o.data_ptr() == w.data_ptr() and hasattr(o, "_ats_grad"):
        return o
    return None


def _grad_sink(w: torch.Tensor):
    """A parameter may carry ``_ats_grad`` (a view into a flat gradient bucket).  Weight gradients are then
    written (first micro-batch) or accumulated (later ones) straight into it by the GEMM epilogue, and autograd
    receives ``None``."""
    o = _sink_owner(w)
    return None if o is None else o._ats_grad


def _deliver_grad(w: torch.Tensor, compute):
    """compute(out, accumulate) -> tensor.  Returns what autograd should see for ``w``."""
    o = _sink_owner(w)
    sink = None if o is None else o._ats_grad
    if sink is None:
        return compute(None, False)
    w = o
    fresh = getattr(w, "_ats_grad_fresh", True)
    compute(sink.view(w.shape), not fresh)
    w._ats_grad_fresh = False
    hook = getattr(w, "_ats_grad_hook", None)
    if hook is not None:
        hook(w)
    return None


def _z3_gathering(w):
    """The row-sharded (ZeRO-3) description of ``w`` when its rows are NOT gathered on this rank right now and the product has to
    pull them itself (``parallel/zero3.py``); otherwise ``None``."""
    z3 = getattr(w, "_ats_z3", None)
    return z3 if (z3 is not None and z3.full is None and z3.gather_in_gemm) else None


def _start_grad_reduce(dx, group):
    """Tensor parallelism: the input gradient of a column-split product is a partial sum.  Its all-reduce is started here and
    runs on the communication stream while the caller computes the weight gradient; ``.wait()`` orders the compute stream
    after it (reference: colossalai ``shardformer/layer/_operation.py:108-167``)."""
    if group is None or dx is None:
        return None
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(dx, group=group, async_op=True)


def _copy_to_region(x, group):
    from ..parallel.tensor_parallel import _CopyToRegion
    return _CopyToRegion.apply(x, group)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, reduce_group=None):
        ctx.reduce_group = reduce_group
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        z3 = _z3_gathering(w)
        n_out = z3.N if z3 is not None else w.shape[0]
        r2 = residual.reshape(-1, n_out) if residual is not None else None
        y = torch.empty(*shape[:-1], n_out, dtype=x.dtype, device=x.device)
        if z3 is not None:
            # the weight lives as row shards on the data-parallel ranks: the GEMM launch gathers it while it computes
            from ..parallel.fused_linear import gathered_gemm
            gathered_gemm(x2, z3, out=y.view(-1, n_out), add=r2)
        else:
            G.gemm_nt(x2, w, out=y.view(-1, n_out), add=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_res = residual is not None
        ctx.shape = shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = G.gemm_nn(dy2, w).view(ctx.shape) if ctx.needs_input_grad[0] else None
        pending = _start_grad_reduce(dx, ctx.reduce_group)  # overlaps the weight-gradient product below
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _deliver_grad(w, lambda out, acc: G.gemm_tn(dy2, x2, out=out, accumulate=acc))
        if pending is not None:
            pending.wait()
        return dx, dw, (dy if ctx.has_res else None), None


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None, reduce_group=None) -> torch.Tensor:
    """``x @ w.T (+ residual)`` -- the residual add is fused into the GEMM epilogue.  ``reduce_group``: ``w`` holds this rank's
    output columns of a tensor-parallel product, so the input gradient is all-reduced over that group."""
    from . import int4, int8
    if int8.observing():
        int8.record(x.reshape(-1, x.shape[-1]), w)
    if int4.observing():
        int4.record(x.reshape(-1, x.shape[-1]), w)
    if int4.usable(x, w):
        return int4.linear_int4(x, w, residual)
    if int8.usable(x, w):
        return int8.linear_int8(x, w, residual)
    if _lib.use_cuda_kernels(x):
        from . import fp8
        if fp8.enabled() and getattr(w, "_ats_z3", None) is None and x.shape[-1] % 16 == 0 and w.shape[0] % 8 == 0:
            return fp8.linear_fp8(_copy_to_region(x, reduce_group) if reduce_group is not None else x, w, residual)
        return _LinearFn.apply(x, w, residual, reduce_group)
    if reduce_group is not None:
        x = _copy_to_region(x, reduce_group)
    y = F.linear(x, w)
    return y + residual if residual is not None else y


# ----------------------------------------------------------------------------------------------------------
# SwiGLU
# ----------------------------------------------------------------------------------------------------------
def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gu.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shape = gu.shape
        g2 = gu.reshape(-1, shape[-1])
        inter = shape[-1] // 2
        h = torch.empty(*shape[:-1], inter, dtype=gu.dtype, device=gu.device)
        _CK(_L().ats_swiglu_fwd(_P(g2), _P(h), g2.shape[0], inter, _S(gu.device)), "swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = shape
        return h

    @staticmethod
    def backward(ctx, dh):
        (g2,) = ctx.saved_tensors
        inter = g2.shape[1] // 2
        d2 = dh.reshape(-1, inter)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(g2)
        _CK(_L().ats_swiglu_bwd(_P(g2), _P(d2), _P(dgu), None, g2.shape[0], inter, _S(g2.device)), "swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    if _lib.use_cuda_kernels(gu) and gu.shape[-1] % 16 == 0 and gu.is_contiguous():
        return _SwiGLUFn.apply(gu)
    return swiglu_reference(gu)


class _SwiGLUMLPFn(torch.autograd.Function):
    """down( silu(x Wg^T) * (x Wu^T) ) with the activation fused into the first GEMM's epilogue."""

    @staticmethod
    def forward(ctx, x, w1, w2, residual, reduce_group=None):
        ctx.reduce_group = reduce_group
        ctx.fp8 = False
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        need_bwd = any(ctx.needs_input_grad)
        z1, z2 = _z3_gathering(w1), _z3_gathering(w2)
        n1 = z1.N if z1 is not None else w1.shape[0]
        n2 = z2.N if z2 is not None else w2.shape[0]
        pre = torch.empty(x2.shape[0], n1, dtype=x.dtype, device=x.device) if need_bwd else None
        r2 = residual.reshape(-1, n2) if residual is not None else None
        y = torch.empty(*shape[:-1], n2, dtype=x.dtype, device=x.device)
        from . import fp8
        if z1 is not None and z2 is not None:
            # ZeRO-3 row shards: both products gather their weight inside the GEMM launch (SwiGLU and residual epilogues as usual)
            from ..parallel.fused_linear import gathered_gemm
            h = gathered_gemm(x2, z1, swiglu=True, pre_act=pre)
            gathered_gemm(h, z2, out=y.view(-1, n2), add=r2)
        elif fp8.enabled() and x2.shape[1] % 16 == 0 and w1.shape[0] % 32 == 0:
            # e4m3 forward products (per-token / per-channel scales); backward: input gradient in e4m3, the rest in bf16
            ctx.fp8 = True
            xq, xs = fp8.quantize_rows(x2)
            w1q, w1s = fp8.quantized_weight(w1)
            h = fp8.gemm_nt_fp8(xq, xs, w1q, w1s, swiglu=True, aux=pre)
            hq, hs = fp8.quantize_rows(h)
            w2q, w2s = fp8.quantized_weight(w2)
            fp8.gemm_nt_fp8(hq, hs, w2q, w2s, out=y.view(-1, w2.shape[0]), add=r2)
        else:
            h = G.gemm_nt_swiglu(x2, w1, pre_act=pre)
            G.gemm_nt(h, w2, out=y.view(-1, w2.shape[0]), add=r2)
        ctx.save_for_backward(x2, w1, w2, pre)
        ctx.shape = shape
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre = ctx.saved_tensors
        inter = w1.shape[0] // 2
        dy2 = dy.reshape(-1, w2.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dgu, h = G.gemm_nn_swiglu_bwd(dy2, w2, pre)  # dh = dy · w2 goes through the SwiGLU backward in the GEMM epilogue
        if ctx.fp8:
            from . import fp8
            input_grad = lambda: fp8.input_grad(dgu, w1).view(ctx.shape)  # noqa: E731
        else:
            input_grad = lambda: G.gemm_nn(dgu, w1).view(ctx.shape)  # noqa: E731
        if ctx.reduce_group is not None:
            # tensor parallel: the input gradient first, so that its all-reduce runs under both weight-gradient products
            dx = input_grad()
            pending = _start_grad_reduce(dx, ctx.reduce_group)
        dw2 = _deliver_grad(w2, lambda out, acc: G.gemm_tn(dy2, h, out=out, accumulate=acc))
        dw1 = _deliver_grad(w1, lambda out, acc: G.gemm_tn(dgu, x2, out=out, accumulate=acc))
        if ctx.reduce_group is None:
            dx = input_grad()
        elif pending is not None:
            pending.wait()
        return dx, dw1, dw2, (dy if ctx.has_res else None), None


def swiglu_mlp(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
               residual: Optional[torch.Tensor] = None, reduce_group=None) -> torch.Tensor:
    from . import int4, int8
    if int8.observing():
        int8.record(x.reshape(-1, x.shape[-1]), w_gate_up)
    if reduce_group is None and int4.usable(x, w_gate_up) and int4.usable(x, w_down):
        return int4.swiglu_mlp_int4(x, w_gate_up, w_down, residual)
    if int4.observing() and reduce_group is None and not torch.is_grad_enabled():
        return int4.swiglu_mlp_observed(x, w_gate_up, w_down, residual)
    if reduce_group is None and int8.usable(x, w_gate_up) and w_gate_up.shape[0] % 32 == 0 and w_down.shape[1] % 16 == 0:
        return int8.swiglu_mlp_int8(x, w_gate_up, w_down, residual)
    if _lib.use_cuda_kernels(x):
        return _SwiGLUMLPFn.apply(x, w_gate_up, w_down, residual, reduce_group)
    if reduce_group is not None:
        x = _copy_to_region(x, reduce_group)
    y = F.linear(swiglu_reference(F.linear(x, w_gate_up)), w_down)
    return y + residual if residual is not None else y


# ----------------------------------------------------------------------------------------------------------
# RoPE (half-split)
# ----------------------------------------------------------------------------------------------------------
def rope_tables(max_pos: int, dim: int, theta: float = 10000.0, scaling: float = 1.0, device=None):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    t = torch.arange(max_pos, dtype=torch.float64) / scaling
    ang = torch.outer(t, inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """x: [..., L, heads, d]; positions: [L] or [B, L] indices into the tables."""
    d = x.shape[-1]
    c = cos[positions].unsqueeze(-2)
    s = sin[positions].unsqueeze(-2)
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).to(x.dtype)


class _RopePackedFn(torch.autograd.Function):
    """Rotates the q and k heads of a packed [tokens, (hq + 2 hkv) * d] projection in place."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_q, n_kv, d, seq_len, pos_offset, positions):
        ctx.mark_dirty(qkv)
        tokens = qkv.numel() // qkv.shape[-1]
        stride = qkv.shape[-1]
        pos32 = positions.to(torch.int32).contiguous() if positions is not None else None
        _CK(_L().ats_rope(_P(qkv), _P(cos), _P(sin), _P(pos32), tokens, seq_len, pos_offset, stride, 0, n_q + n_kv, d, 0,
                          _S(qkv.device)), "rope")
        ctx.args = (n_q, n_kv, d, seq_len, pos_offset)
        ctx.save_for_backward(cos, sin, pos32) if pos32 is not None else ctx.save_for_backward(cos, sin)
        ctx.has_pos = pos32 is not None
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        n_q, n_kv, d, seq_len, pos_offset = ctx.args
        saved = ctx.saved_tensors
        cos, sin = saved[0], saved[1]
        pos32 = saved[2] if ctx.has_pos else None
        g = dqkv if dqkv.is_contiguous() else dqkv.contiguous()
        g = g.clone() if g.data_ptr() == dqkv.data_ptr() else g
        tokens = g.numel() // g.shape[-1]
        _CK(_L().ats_rope(_P(g), _P(cos), _P(sin), _P(pos32), tokens, seq_len, pos_offset, g.shape[-1], 0, n_q + n_kv, d, 1,
                          _S(g.device)), "rope_bwd")
        return g, None, None, None, None, None, None, None, None


def rope_packed(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_q: int, n_kv: int, d: int,
                pos_offset: int = 0, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv: [B, L, (n_q + 2 n_kv) * d].  Position of token (b, l) is ``positions[b, l]`` or ``pos_offset + l``."""
    B, L, width = qkv.shape
    if _lib.use_cuda_kernels(qkv) and d % 16 == 0 and qkv.is_contiguous():
        if cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise TypeError("rope tables must be float32")
        return _RopePackedFn.apply(qkv, cos, sin, n_q, n_kv, d, L, pos_offset, positions)
    pos = positions if positions is not None else torch.arange(pos_offset, pos_offset + L, device=qkv.device)
    qk = qkv[..., : (n_q + n_kv) * d].reshape(B, L, n_q + n_kv, d)
    qk = rope_reference(qk, cos, sin, pos)
    return torch.cat([qk.reshape(B, L, -1), qkv[..., (n_q + n_kv) * d:]], dim=-1)


# ----------------------------------------------------------------------------------------------------------
# Embedding
# ----------------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, scale):
        flat = ids.reshape(-1).contiguous()
        out = torch.empty(*ids.shape, table.shape[1], dtype=table.dtype, device=table.device)
        _CK(_L().ats_embedding_fwd(_P(flat), _P(table), _P(out), flat.numel(), table.shape[1], table.shape[0], scale,
                                   _S(table.device)), "embedding_fwd")
        ctx.save_for_backward(flat, table)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        flat, table = ctx.saved_tensors
        d2 = dout.reshape(-1, table.shape[1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        sorted_ids, order = torch.sort(flat.clamp(0, table.shape[0] - 1), stable=True)

        def compute(out, acc):
            if out is None:
                out = torch.zeros_like(table)
            elif not acc:
                out.zero_()
            _CK(_L().ats_embedding_bwd(_P(sorted_ids), _P(order), _P(d2), _P(out), flat.numel(), table.shape[1],
                                       table.shape[0], ctx.scale, 1 if acc else 0, _S(table.device)), "embedding_bwd")
            return out
        return None, _deliver_grad(table, compute), None


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if _lib.use_cuda_kernels(table) and table.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, table, scale)
    out = F.embedding(ids.clamp(0, table.shape[0] - 1), table)
    return out * scale if scale != 1.0 else out


# ----------------------------------------------------------------------------------------------------------
# Cross-entropy
# ----------------------------------------------------------------------------------------------------------
def cross_entropy_reference(logits: torch.Tensor, labels: torch.Tensor, weights: Optional[torch.Tensor],
                            ignore_index: int = -100):
    """Returns (weighted mean loss, unweighted mean loss, valid count, accuracy)."""
    V = logits.shape[-1]
    lg = logits.reshape(-1, V).float()
    lb = labels.reshape(-1)
    valid = (lb != ignore_index)
    per = F.cross_entropy(lg, lb.clamp(min=0), reduction="none") * valid
    w = valid.float() if weights is None else weights.reshape(-1).float() * valid
    denom = w.sum().clamp(min=1e-8)
    loss = (per * w).sum() / denom
    nvalid = valid.sum()
    raw = per.sum() / nvalid.clamp(min=1)
    acc = ((lg.argmax(-1) == lb) & valid).sum() / nvalid.clamp(min=1)
    return loss, raw.detach(), nvalid, acc.detach()


class _LinearCEFn(torch.autograd.Function):
    """lm_head GEMM + cross-entropy, chunked over tokens; dlogits are produced in place right after each chunk's
    logits, and dh / dW are computed in the same pass, so the full [T, V] logits never exist."""

    @staticmethod
    def forward(ctx, h, w, labels, weights, ignore_index, chunk_rows):
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        lb = labels.reshape(-1).contiguous()
        valid = lb != ignore_index
        wt = valid.float() if weights is None else weights.reshape(-1).float() * valid
        denom = wt.sum().clamp(min=1e-8)
        row_scale = (wt / denom).contiguous()
        need_grad = any(ctx.needs_input_grad)
        loss_row = torch.empty(T, dtype=torch.float32, device=dev)
        correct = torch.empty(T, dtype=torch.float32, device=dev)
        dh = torch.empty_like(h) if need_grad else None
        dw32 = torch.zeros(V, H, dtype=torch.float32, device=dev) if ctx.needs_input_grad[1] else None
        lib = _L()
        for r0 in range(0, T, chunk_rows):
            r1 = min(r0 + chunk_rows, T)
            hc = h[r0:r1]
            logits = G.gemm_nt(hc, w)
            _CK(lib.ats_ce_fwd_bwd(_P(logits), _P(lb[r0:r1]), _P(row_scale[r0:r1]) if need_grad else None,
                                   _P(loss_row[r0:r1]), _P(correct[r0:r1]), None, r1 - r0, V, logits.stride(0),
                                   ignore_index, _S(dev)), "ce_fwd_bwd")
            if need_grad:
                G.gemm_nn(logits, w, out=dh[r0:r1])
                if dw32 is not None:
                    G.gemm_tn(logits, hc, out=dw32, accumulate=True)
        nvalid = valid.sum()
        loss = (loss_row * row_scale).sum()
        raw = loss_row.sum() / nvalid.clamp(min=1)
        acc = correct.sum() / nvalid.clamp(min=1)
        ctx.save_for_backward(dh, dw32, w)
        ctx.mark_non_differentiable(raw, nvalid, acc)
        return loss, raw, nvalid, acc

    @staticmethod
    def backward(ctx, gloss, *_):
        dh, dw32, w = ctx.saved_tensors
        dhs = dh * gloss.to(dh.dtype) if dh is not None else None
        dw = None
        if dw32 is not None:
            def compute(out, acc):
                if out is None:
                    out = torch.empty_like(w)
                _CK(_L().ats_cast_f32_bf16(_P(dw32), _P(out), dw32.numel(), 1 if acc else 0, float(1.0), _S(w.device)),
                    "cast")
                return out
            dw = _deliver_grad(w, compute)
        return dhs, dw, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                         weights: Optional[torch.Tensor] = None, ignore_index: int = -100,
                         chunk_rows: int = 4096):
    """Loss of ``softmax(h @ w.T)`` against ``labels`` -> (loss, raw_loss, valid_tokens, accuracy).

    The weight gradient is taken with unit upstream gradient (the loss is the root of the graph in training);
    ``dh`` is scaled by the upstream gradient."""
    h2 = h.reshape(-1, h.shape[-1])
    if _lib.use_cuda_kernels(h2):
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        return _LinearCEFn.apply(h2, w, labels, weights, ignore_index, chunk_rows)
    return cross_entropy_reference(F.linear(h2, w), labels, weights, ignore_index)


class _CEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, weights, ignore_index):
        V = logits.shape[-1]
        lg = logits.reshape(-1, V).clone()
        lb = labels.reshape(-1).contiguous()
        valid = lb != ignore_index
        wt = valid.float() if weights is None else weights.reshape(-1).float() * valid
        denom = wt.sum().clamp(min=1e-8)
        row_scale = (wt / denom).contiguous()
        T = lg.shape[0]
        loss_row = torch.empty(T, dtype=torch.float32, device=lg.device)
        correct = torch.empty(T, dtype=torch.float32, device=lg.device)
        need_grad = ctx.needs_input_grad[0]
        _CK(_L().ats_ce_fwd_bwd(_P(lg), _P(lb), _P(row_scale) if need_grad else None, _P(loss_row), _P(correct), None, T, V,
                                lg.stride(0), ignore_index, _S(lg.device)), "ce")
        nvalid = valid.sum()
        loss = (loss_row * row_scale).sum()
        raw = loss_row.sum() / nvalid.clamp(min=1)
        acc = correct.sum() / nvalid.clamp(min=1)
        ctx.save_for_backward(lg if need_grad else None)
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(raw, nvalid, acc)
        return loss, raw, nvalid, acc

    @staticmethod
    def backward(ctx, gloss, *_):
        (dl,) = ctx.saved_tensors
        return (dl * gloss.to(dl.dtype)).view(ctx.shape), None, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, weights: Optional[torch.Tensor] = None,
                  ignore_index: int = -100):
    if _lib.use_cuda_kernels(logits) and logits.shape[-1] % 8 == 0:
        return _CEFn.apply(logits, labels, weights, ignore_index)
    return cross_entropy_reference(logits, labels, weights, ignore_index)


# ----------------------------------------------------------------------------------------------------------
# Attention (causal, grouped-query) on the packed projection
# ----------------------------------------------------------------------------------------------------------
def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                        q_offset: int = 0, key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [B, Lq, Hq, D]; k, v: [B, Lk, Hkv, D].  Query i attends keys j <= q_offset + i.  fp32 softmax."""
    B, Lq, Hq, D = q.shape
    Lk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3).reshape(B, Hkv, rep, Lq, D)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    s = torch.einsum("bgrqd,bgkd->bgrqk", qf, kf) / math.sqrt(D)
    if causal:
        qi = torch.arange(Lq, device=q.device)[:, None] + q_offset
        kj = torch.arange(Lk, device=q.device)[None, :]
        s = s.masked_fill(kj > qi, float("-inf"))
    if key_mask is not None:
        s = s.masked_fill(~key_mask.bool()[:, None, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)
    o = torch.einsum("bgrqk,bgkd->bgrqd", p, vf).reshape(B, Hq, Lq, D).permute(0, 2, 1, 3)
    return o.to(q.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, q_offset: int = 0,
              key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    from . import attn as A
    if _lib.use_cuda_kernels(q) and key_mask is None and A.supported(q, k, v, causal, q_offset):
        return A.flash_attention(q, k, v, causal, q_offset)
    return attention_reference(q, k, v, causal, q_offset, key_mask)


def attention_packed_available(qkv: torch.Tensor, d: int, seq_len: int) -> bool:
    from . import attn as A
    return (_lib.use_cuda_kernels(qkv) and A._native_available() and d in (64, 128) and seq_len % 128 == 0 and qkv.is_contiguous()
            and qkv.shape[-1] % 8 == 0)


def rope_attention_packed(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_q: int, n_kv: int, d: int,
                          pos_offset: int = 0) -> torch.Tensor:
    """RoPE + causal grouped-query attention on the packed projection as one autograd node (see ``attention_packed``)."""
    from .attention_native import rope_flash_attention_packed
    return rope_flash_attention_packed(qkv, cos, sin, n_q, n_kv, d, pos_offset)


def attention_packed(qkv: torch.Tensor, n_q: int, n_kv: int, d: int) -> torch.Tensor:
    """Causal grouped-query attention straight on the packed projection [B, L, (n_q + 2 n_kv) * d] -> [B, L, n_q, d]."""
    from .attention_native import flash_attention_packed
    return flash_attention_packed(qkv, n_q, n_kv, d)


# ----------------------------------------------------------------------------------------------------------
# Optimiser / norm helpers (no autograd)
# ----------------------------------------------------------------------------------------------------------
def sumsq(buf: torch.Tensor, out: torch.Tensor, accumulate: bool = False, scratch: Optional[torch.Tensor] = None) -> None:
    """out[0] (+)= sum(buf^2) computed on the device without a host round trip."""
    if buf.is_cuda and buf.dtype in (torch.bfloat16, torch.float32):
        if scratch is None:
            scratch = torch.empty(1024, dtype=torch.float32, device=buf.device)
        _CK(_L().ats_sumsq(_P(buf), buf.numel(), int(buf.dtype == torch.float32), _P(scratch), _P(out), int(accumulate),
                           _S(buf.device)), "sumsq")
    else:
        s = buf.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s


def clip_coef(sumsq_t: torch.Tensor, state: torch.Tensor, pre_scale: float, max_norm: float) -> None:
    """state = [gradient scale to apply, global norm, skip flag]."""
    if sumsq_t.is_cuda:
        _CK(_L().ats_clip_coef(_P(sumsq_t), pre_scale, max_norm, _P(state), _S(sumsq_t.device)), "clip_coef")
    else:
        norm = float(sumsq_t[0].sqrt()) * pre_scale
        finite = math.isfinite(norm)
        coef = min(1.0, max_norm / (norm + 1e-6)) if (max_norm > 0 and finite) else 1.0
        state[0] = pre_scale * coef if finite else 0.0
        state[1] = norm
        state[2] = 0.0 if finite else 1.0


def adamw_step(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor, param: torch.Tensor,
               hyper: torch.Tensor, clip_state: Optional[torch.Tensor], wd_mult: float = 1.0) -> None:
    """One AdamW update of a flat shard.  ``hyper`` = [lr, beta1, beta2, eps, weight_decay, step] (device tensor);
    ``clip_state`` as written by :func:`clip_coef`.  ``param`` receives the updated values in its own dtype."""
    if master.is_cuda and grad.dtype == torch.bfloat16 and param.dtype == torch.bfloat16:
        _CK(_L().ats_adamw(_P(master), _P(m), _P(v), _P(grad), _P(param), master.numel(), _P(hyper), _P(clip_state),
                           wd_mult, _S(master.device)), "adamw")
        return
    lr, b1, b2, eps, wd, step = [float(x) for x in hyper.tolist()]
    wd *= wd_mult
    gscale = 1.0
    if clip_state is not None:
        if float(clip_state[2]) != 0.0:
            return
        gscale = float(clip_state[0])
    g = grad.float() * gscale
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    master.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
    param.copy_(master.to(param.dtype))

"""W8A8 int8 linear layers for inference on the tcgen05 ``kind::i8`` GEMM, with optional SmoothQuant migration.

Weights are quantised once, per output channel, to signed bytes; activations per token at run time; the GEMM accumulates the
s8 x s8 products in s32 tensor memory over the whole reduction and its epilogue multiplies by ``row_scale[m] * col_scale[n]``
(the main loop is the e4m3 one with another MMA kind, so the int8 path runs at the fp8 rate).  SmoothQuant: activation outliers
live in a few input channels; a per-input-channel factor ``s_j = amax_x[j]^alpha / amax_w[j]^(1 - alpha)`` is multiplied into the
weight columns before quantisation and divided out of the activations inside the quantise kernel, which moves the dynamic range
from the activations (quantised per token, so one outlier channel costs every channel its resolution) to the weights.

The reference reaches int8 through external libraries (bitsandbytes / GPTQ / quanto hooks, ``training/trainer.py:575-801``) and
its vendored inference engine through Triton smooth-quant / GPTQ matmuls (``colossalai/kernel/triton/``); neither ships here.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from . import gemm as G

_vp, _ci, _cll, _cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_sig = False
_enabled = False
_observing = False
_weight_cache: Dict[int, Tuple[int, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]] = {}
_act_amax: Dict[int, torch.Tensor] = {}      # weight storage -> running max |x| per input channel (calibration)
_smoothing: Dict[int, torch.Tensor] = {}     # weight storage -> largest |x| per input channel seen during calibration
_alpha = 0.5                                 # SmoothQuant migration strength: s = amax_x^alpha / amax_w^(1 - alpha)


def set_enabled(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


def enabled() -> bool:
    return _enabled


def _fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_quantize_rows_int8.restype = _ci
        lib.ats_quantize_rows_int8.argtypes = [_vp, _cll, _vp, _cll, _vp, _cll, _ci, _vp, _vp]
        lib.ats_gemm_int8.restype = _ci
        lib.ats_gemm_int8.argtypes = [_vp, _cll, _cll, _cll, _vp, _cll, _cll, _cll, _vp, _ci, _vp, _ci, _vp, _ci, _ci, _ci, _ci, _cf, _ci,
                                      _ci, _ci, _ci, _vp, _ci, _ci, _cll, _cll, _cll, _ci, _vp, _cll, _vp, _cll, _vp, _ci, _vp]
        _sig = True
    return lib


def quantize_rows_reference(x: torch.Tensor, inv_smooth: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    if inv_smooth is not None:
        xf = xf * inv_smooth.float()[None, :]
    amax = xf.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(xf / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def quantize_rows(x: torch.Tensor, inv_smooth: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [rows, cols] bf16 -> (int8 [rows, cols], fp32 scale [rows]) with x * inv_smooth ~= q * scale[:, None]."""
    if not (_lib.use_cuda_kernels(x) and x.dim() == 2 and x.shape[1] % 16 == 0):
        return quantize_rows_reference(x, inv_smooth)
    if x.stride(1) != 1 or x.stride(0) % 8:
        x = x.contiguous()
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    sm = inv_smooth.to(torch.bfloat16).contiguous() if inv_smooth is not None else None
    err = _fns().ats_quantize_rows_int8(_lib.ptr(x), x.stride(0), _lib.ptr(q), cols, _lib.ptr(scale), rows, cols, _lib.ptr(sm), _lib.stream_ptr(x.device))
    _lib.check(err, "ats_quantize_rows_int8")
    return q, scale


def gemm_nt_int8(aq: torch.Tensor, a_scale: torch.Tensor, bq: torch.Tensor, b_scale: torch.Tensor, out: Optional[torch.Tensor] = None,
                 add: Optional[torch.Tensor] = None, swiglu: bool = False, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """(aq * a_scale) [M, K] @ (bq * b_scale) [N, K]^T (+ add), or with ``swiglu`` silu(gate) * up over the two halves of N."""
    M, K = aq.shape
    N = bq.shape[0]
    if not aq.is_cuda:
        r = (aq.float() * a_scale[:, None]) @ (bq.float() * b_scale[:, None]).t()
        if swiglu:
            g, u = r[:, : N // 2].to(out_dtype).float(), r[:, N // 2:].to(out_dtype).float()
            r = torch.nn.functional.silu(g) * u
        if add is not None:
            r = r + add.float()
        r = r.to(out_dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=out_dtype, device=aq.device)
    st = _lib.status_tensor(aq.device)
    splits = G._skinny_splits(M, N, K) if (not swiglu and G.SPLIT_K_SKINNY and out.is_contiguous() and out_dtype == torch.bfloat16
                                           and (add is None or add.is_contiguous()) and N % 8 == 0) else 1
    if splits > 1 and (K // splits) % 128 == 0:
        # decode-sized products: slices of the reduction as groups with fp32 partial outputs, folded by one launch
        kp = K // splits
        part = torch.empty(splits, M, N, dtype=torch.float32, device=aq.device)
        err = _fns().ats_gemm_int8(_lib.ptr(aq), M, K, aq.stride(0), _lib.ptr(bq), N, K, bq.stride(0), _lib.ptr(part), N, None, 0, None, 0, M, N, kp,
                                   1.0, G.EPI_F32, 0, splits, 0, None, 0, 0, M * N, 0, 0, 1, _lib.ptr(a_scale), 0, _lib.ptr(b_scale), 0, kp, kp,
                                   _lib.ptr(st), 0, _lib.stream_ptr(aq.device))
        _lib.check(err, "ats_gemm_int8 (reduction slices)")
        G._fold_partials(part, splits, M * N, 1, out, add)
        return out
    epi = G.EPI_SWIGLU if swiglu else (G.EPI_ADDC if add is not None else G.EPI_STORE)
    err = _fns().ats_gemm_int8(_lib.ptr(aq), M, K, aq.stride(0), _lib.ptr(bq), N, K, bq.stride(0), _lib.ptr(out), out.stride(0), _lib.ptr(add),
                               add.stride(0) if add is not None else 0, None, 0, M, n_out, K, 1.0, epi, N // 2 if swiglu else 0, 1, 0, None, 0, 0,
                               0, 0, 0, 1, _lib.ptr(a_scale), 0, _lib.ptr(b_scale), 0, 0, 0, _lib.ptr(st), 0, _lib.stream_ptr(aq.device))
    _lib.check(err, "ats_gemm_int8")
    return out


# -- calibration (SmoothQuant) -----------------------------------------------------------------------------------------------
def observe(flag: bool) -> None:
    """While on, every ``ops.linear`` / MLP product records the largest |x| per input channel of its weight."""
    global _observing
    _observing = bool(flag)


def observing() -> bool:
    return _observing


def record(x2: torch.Tensor, w: torch.Tensor) -> None:
    a = x2.detach().float().abs().amax(0)
    key = w.data_ptr()
    prev = _act_amax.get(key)
    _act_amax[key] = a if prev is None else torch.maximum(prev, a)


def finish_calibration(alpha: float = 0.5) -> int:
    """Turns the recorded activation ranges into smoothing factors; returns how many weights got one."""
    global _alpha
    _alpha = float(alpha)
    n = 0
    for key, a in _act_amax.items():
        _smoothing[key] = a       # the weight's own range is folded in when the weight is quantised (needs the tensor)
        n += 1
    _weight_cache.clear()
    return n


def quantized_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """-> (int8 [N, K], scales [N], 1 / s [K] or None): per-output-channel quantisation of ``w * s`` (s = 1 without calibration)."""
    key = w.data_ptr()
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == w._version and hit[1].shape == w.shape:
        return hit[1], hit[2], hit[3]
    wf = w.detach().float()
    inv = None
    a = _smoothing.get(key)
    if a is not None:
        alpha = _alpha
        wmax = wf.abs().amax(0).clamp(min=1e-5)
        s = (a.to(wf.device).clamp(min=1e-5) ** alpha / wmax ** (1.0 - alpha)).clamp(min=1e-3, max=1e3)
        wf = wf * s[None, :]
        inv = (1.0 / s)
    q, sc = quantize_rows(wf.to(torch.bfloat16) if w.is_cuda else wf)
    _weight_cache[key] = (w._version, q, sc, inv)
    return q, sc, inv


def clear() -> None:
    _weight_cache.clear()
    _act_amax.clear()
    _smoothing.clear()


# -- layers --------------------------------------------------------------------------------------------------------------------
def usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (_enabled and not torch.is_grad_enabled() and w.dim() == 2 and x.shape[-1] % 16 == 0 and w.shape[0] % 8 == 0
            and getattr(w, "_ats_z3", None) is None)


@torch.no_grad()
def linear_int8(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ residual)`` with int8 operands (inference only)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    wq, ws, inv = quantized_weight(w)
    xq, xs = quantize_rows(x2, inv)
    r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
    y = gemm_nt_int8(xq, xs, wq, ws, add=r2, out_dtype=x.dtype)
    return y.view(*shape[:-1], w.shape[0])


@torch.no_grad()
def swiglu_mlp_int8(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    w1q, w1s, inv1 = quantized_weight(w1)
    xq, xs = quantize_rows(x2, inv1)
    h = gemm_nt_int8(xq, xs, w1q, w1s, swiglu=True, out_dtype=x.dtype)
    if _observing:
        record(h, w2)
    w2q, w2s, inv2 = quantized_weight(w2)
    hq, hs = quantize_rows(h, inv2)
    r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
    y = gemm_nt_int8(hq, hs, w2q, w2s, add=r2, out_dtype=x.dtype)
    return y.view(*shape[:-1], w2.shape[0])

"""fp8 (e4m3) linear layers on the tcgen05 GEMM.

Scheme: activations are quantised per token row, weights per output channel (both along the reduction dimension), the
GEMM accumulates the raw e4m3 products in fp32 tensor memory over the whole reduction and the epilogue multiplies by
``row_scale[m] * col_scale[n]``.  Unlike a 1 x 128 / 128 x 128 block format this needs no per-block promotion inside the
main loop, so the fp8 main loop is the bf16 one with half the operand bytes and ``kind::f8f6f4`` MMAs.

Forward products run in fp8; the backward products (input and weight gradients) use the saved bf16 activations and the
bf16 weights, so optimiser state, gradients and master weights are unchanged ("hybrid" precision).  The reference lists
fp8 precisions but has no fp8 GEMM path at all (reference ``training/trainer.py:440-446`` only wraps autocast).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from . import gemm as G

_vp, _ci, _cll, _cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_sig = False
E4M3_MAX = 448.0
_enabled = False
_weight_cache: Dict[int, Tuple[Tuple[int, int], torch.Tensor, torch.Tensor]] = {}


def set_enabled(flag: bool) -> None:
    """Route ``ops.linear`` / the dense SwiGLU MLP through the fp8 forward path (CUDA bf16 tensors only)."""
    global _enabled
    _enabled = bool(flag)


def enabled() -> bool:
    return _enabled


def _fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_quantize_rows_e4m3.restype = _ci
        lib.ats_quantize_rows_e4m3.argtypes = [_vp, _cll, _vp, _cll, _vp, _cll, _ci, _vp]
        lib.ats_gemm_fp8.restype = _ci
        lib.ats_gemm_fp8.argtypes = [_vp, _cll, _cll, _cll, _vp, _cll, _cll, _cll, _vp, _ci, _vp, _ci, _vp, _ci, _ci, _ci, _ci, _cf, _ci,
                                     _ci, _ci, _ci, _vp, _ci, _ci, _cll, _cll, _cll, _ci, _vp, _cll, _vp, _cll, _vp, _ci, _vp]
        _sig = True
    return lib


def quantize_rows_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    amax = xf.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xf / scale[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [rows, cols] bf16 -> (e4m3 [rows, cols], fp32 scale [rows]) with x ~= q * scale[:, None]."""
    if x.dim() != 2:
        raise ValueError("quantize_rows expects a 2-D tensor")
    if not (_lib.use_cuda_kernels(x) and x.shape[1] % 8 == 0):
        return quantize_rows_reference(x)
    if x.stride(1) != 1 or x.stride(0) % 8:
        x = x.contiguous()
    rows, cols = x.shape
    pitch = (cols + 15) // 16 * 16  # the GEMM's tensor map wants 16-byte row pitches
    q = torch.empty(rows, pitch, dtype=torch.uint8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    err = _fns().ats_quantize_rows_e4m3(_lib.ptr(x), x.stride(0), _lib.ptr(q), pitch, _lib.ptr(scale), rows, cols, _lib.stream_ptr(x.device))
    _lib.check(err, "ats_quantize_rows_e4m3")
    return q[:, :cols].view(torch.float8_e4m3fn), scale


_epoch = 0


def weights_changed() -> None:
    """Optimiser engines call this after every parameter update: their kernels write the flat parameter buckets through raw
    pointers, which PyTorch's version counters do not see, so cached quantised weights are keyed on this epoch as well."""
    global _epoch
    _epoch += 1
    if len(_weight_cache) > 4096:
        _weight_cache.clear()


def quantized_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel quantisation of a [N, K] weight, cached until the parameters change."""
    key = w.data_ptr()
    stamp = (w._version, _epoch)
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == stamp and hit[1].shape == w.shape:
        return hit[1], hit[2]
    q, s = quantize_rows(w.detach())
    _weight_cache[key] = (stamp, q, s)
    return q, s


def clear_weight_cache() -> None:
    _weight_cache.clear()


def gemm_nt_fp8(aq: torch.Tensor, a_scale: torch.Tensor, bq: torch.Tensor, b_scale: torch.Tensor, out: Optional[torch.Tensor] = None,
                add: Optional[torch.Tensor] = None, swiglu: bool = False, aux: Optional[torch.Tensor] = None,
                out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """(aq * a_scale) [M, K] @ (bq * b_scale)[N, K]^T (+ add), or with ``swiglu``: silu(gate) * up over the two halves of N."""
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
    epi = G.EPI_SWIGLU if swiglu else (G.EPI_ADDC if add is not None else G.EPI_STORE)
    st = _lib.status_tensor(aq.device)
    err = _fns().ats_gemm_fp8(_lib.ptr(aq), M, K, aq.stride(0), _lib.ptr(bq), N, K, bq.stride(0), _lib.ptr(out), out.stride(0), _lib.ptr(add),
                              add.stride(0) if add is not None else 0, _lib.ptr(aux), aux.stride(0) if aux is not None else 0, M, n_out, K,
                              1.0, epi, N // 2 if swiglu else 0, 1, 0, None, 0, 0, 0, 0, 0, 1, _lib.ptr(a_scale), 0, _lib.ptr(b_scale), 0,
                              _lib.ptr(st), 0, _lib.stream_ptr(aq.device))
    _lib.check(err, "ats_gemm_fp8")
    return out


class _LinearFP8Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual):
        from .functional import _deliver_grad  # noqa: F401  (kept close to the bf16 linear)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        xq, xs = quantize_rows(x2)
        wq, ws = quantized_weight(w)
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = torch.empty(*shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        gemm_nt_fp8(xq, xs, wq, ws, out=y.view(-1, w.shape[0]), add=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_res, ctx.shape = residual is not None, shape
        return y

    @staticmethod
    def backward(ctx, dy):
        from .functional import _deliver_grad
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = G.gemm_nn(dy2, w).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _deliver_grad(w, lambda out, acc: G.gemm_tn(dy2, x2, out=out, accumulate=acc))
        return dx, dw, (dy if ctx.has_res else None)


def linear_fp8(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ residual)`` with an e4m3 forward product; backward products in bf16."""
    if _lib.use_cuda_kernels(x) and x.shape[-1] % 16 == 0 and w.shape[0] % 8 == 0:
        return _LinearFP8Fn.apply(x, w, residual)
    # PyTorch definition: quantised forward value, straight-through gradient of the unquantised product
    y_ref = torch.nn.functional.linear(x, w)
    with torch.no_grad():
        xq, xs = quantize_rows_reference(x.reshape(-1, x.shape[-1]))
        wq, ws = quantize_rows_reference(w)
        yq = ((xq.float() * xs[:, None]) @ (wq.float() * ws[:, None]).t()).to(x.dtype).view(*x.shape[:-1], w.shape[0])
    y = y_ref + (yq - y_ref).detach()
    return y + residual if residual is not None else y

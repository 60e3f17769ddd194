"""fp8 (e4m3) linear layers on the tcgen05 GEMM.

Scheme: activations are quantised per token row, weights per output channel (both along the reduction dimension), the
GEMM accumulates the raw e4m3 products in fp32 tensor memory over the whole reduction and the epilogue multiplies by
``row_scale[m] * col_scale[n]``.  Unlike a 1 x 128 / 128 x 128 block format this needs no per-block promotion inside the
main loop, so the fp8 main loop is the bf16 one with half the operand bytes and ``kind::f8f6f4`` MMAs.

Training recipe (``precision = mixed_fp8`` and the other fp8 names): the forward products AND the input-gradient products
run in fp8, dense linears, the dense SwiGLU MLP and the grouped expert products alike.  An input gradient
``dx[t, i] = sum_o dy[t, o] W[o, i]`` reduces over the output channels, so its operands are ``dy`` quantised per token and a
second, transposed copy of the weight quantised per INPUT channel (``quantized_weight_t``; both copies are made once per
optimiser step and cached).  Weight gradients reduce over the tokens; they stay in bf16 on the saved bf16 activations, because
quantising both of their operands along the token dimension would need two more transposing passes over the activations
per product, which costs more than the fp8 product saves at these shapes.  Optimiser state, gradients and master weights
are unchanged.  The product ``dh = dy W2`` inside the SwiGLU backward keeps its bf16 kernel (its epilogue reads the saved
pre-activations).  The reference lists fp8 precisions but has no fp8 GEMM path at all (reference ``training/trainer.py:440-446``
only wraps autocast).
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
    _weight_cache_t.clear()


_weight_cache_t: Dict[int, Tuple[Tuple[int, int], torch.Tensor, torch.Tensor]] = {}


def quantized_weight_t(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The transposed weight quantised per row of the transpose, i.e. per input channel: for ``w`` [N, K] -> e4m3 [K, N] and
    scales [K]; for stacked expert weights [E, N, K] -> [E * K, N] and [E * K].  Cached until the parameters change."""
    key = w.data_ptr()
    stamp = (w._version, _epoch)
    hit = _weight_cache_t.get(key)
    if hit is not None and hit[0] == stamp:
        return hit[1], hit[2]
    wt = w.detach().transpose(-1, -2).contiguous()
    q, s = quantize_rows(wt.view(-1, wt.shape[-1]))
    if len(_weight_cache_t) > 4096:
        _weight_cache_t.clear()
    _weight_cache_t[key] = (stamp, q, s)
    return q, s


def quantized_expert_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[E, N, K] -> e4m3 [E * N, K], scales [E * N] (per output channel of every expert), cached."""
    key = w.data_ptr()
    stamp = (w._version, _epoch)
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == stamp and hit[1].shape[0] == w.shape[0] * w.shape[1]:
        return hit[1], hit[2]
    q, s = quantize_rows(w.detach().view(-1, w.shape[-1]))
    _weight_cache[key] = (stamp, q, s)
    return q, s


def grouped_usable(x: torch.Tensor, n: int, k: int) -> bool:
    return enabled() and _lib.use_cuda_kernels(x) and k % 16 == 0 and n % 16 == 0


def grouped_nt_fp8(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, n: int, counts: torch.Tensor, swiglu: bool = False,
                   pre_act: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, b_div: int = 1) -> torch.Tensor:
    """x [G, C, K] (bf16, quantised here per row) against the e4m3 weights ``wq`` [E * n, K] with scales ``ws`` [E * n]: the first
    counts[g] rows of group g times weight g // b_div, -> [G, C, n] or, through SwiGLU, [G, C, n / 2] (+ pre-activations)."""
    Gn, C, K = x.shape
    assert x.is_contiguous() and C % 128 == 0 and wq.shape[1] == K
    xq, xs = quantize_rows(x.view(Gn * C, K))
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty(Gn, C, n_out, dtype=x.dtype, device=x.device)
    st = _lib.status_tensor(x.device)
    err = _fns().ats_gemm_fp8(_lib.ptr(xq), Gn * C, K, xq.stride(0), _lib.ptr(wq), wq.shape[0], K, wq.stride(0), _lib.ptr(out), n_out, None, 0,
                              _lib.ptr(pre_act), n if pre_act is not None else 0, C, n_out, K, 1.0, G.EPI_SWIGLU if swiglu else G.EPI_STORE,
                              n // 2 if swiglu else 0, Gn, 1, _lib.ptr(counts), C, n, C * n_out, 0, C * n if pre_act is not None else 0, b_div,
                              _lib.ptr(xs), C, _lib.ptr(ws), n, 0, 0, _lib.ptr(st), 0, _lib.stream_ptr(x.device))
    _lib.check(err, "ats_gemm_fp8 (grouped)")
    return out


def grouped_nt(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, swiglu: bool = False, pre_act: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, b_div: int = 1) -> torch.Tensor:
    """Forward product of the experts: fp8 when the fp8 recipe is on, else the bf16 grouped GEMM."""
    if grouped_usable(x, w.shape[1], w.shape[2]) and not getattr(w, "_ats_packed", False):
        wq, ws = quantized_expert_weight(w)
        return grouped_nt_fp8(x, wq, ws, w.shape[1], counts, swiglu, pre_act, out, b_div)
    return G.grouped_nt(x, w, counts, swiglu=swiglu, pre_act=pre_act, out=out, b_div=b_div, packed=bool(getattr(w, "_ats_packed", False)))


def grouped_nn(dy: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, b_div: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Input gradient of the expert product: dy [G, C, N] . w [E, N, K] -> [G, C, K]; fp8 on the per-input-channel copy of w."""
    if grouped_usable(dy, w.shape[2], w.shape[1]):
        wq, ws = quantized_weight_t(w)            # [E * K, N]
        return grouped_nt_fp8(dy, wq, ws, w.shape[2], counts, out=out, b_div=b_div)
    return G.grouped_nn(dy, w, counts, out=out, b_div=b_div)


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
    st = _lib.status_tensor(aq.device)
    splits = G._skinny_splits(M, N, K) if (not swiglu and G.SPLIT_K_SKINNY and out.is_contiguous() and out_dtype == torch.bfloat16
                                           and (add is None or add.is_contiguous()) and N % 8 == 0) else 1
    if splits > 1 and (K // splits) % 128 == 0:
        # a handful of rows against a large weight: slices of the reduction run as groups with fp32 partial outputs (scaled in the
        # epilogue, the scales distribute over the sum) so that every SM streams part of the weight; one launch folds them
        kp = K // splits
        part = torch.empty(splits, M, N, dtype=torch.float32, device=aq.device)
        err = _fns().ats_gemm_fp8(_lib.ptr(aq), M, K, aq.stride(0), _lib.ptr(bq), N, K, bq.stride(0), _lib.ptr(part), N, None, 0, None, 0, M, N, kp,
                                  1.0, G.EPI_F32, 0, splits, 0, None, 0, 0, M * N, 0, 0, 1, _lib.ptr(a_scale), 0, _lib.ptr(b_scale), 0, kp, kp,
                                  _lib.ptr(st), 0, _lib.stream_ptr(aq.device))
        _lib.check(err, "ats_gemm_fp8 (reduction slices)")
        G._fold_partials(part, splits, M * N, 1, out, add)
        return out
    epi = G.EPI_SWIGLU if swiglu else (G.EPI_ADDC if add is not None else G.EPI_STORE)
    err = _fns().ats_gemm_fp8(_lib.ptr(aq), M, K, aq.stride(0), _lib.ptr(bq), N, K, bq.stride(0), _lib.ptr(out), out.stride(0), _lib.ptr(add),
                              add.stride(0) if add is not None else 0, _lib.ptr(aux), aux.stride(0) if aux is not None else 0, M, n_out, K,
                              1.0, epi, N // 2 if swiglu else 0, 1, 0, None, 0, 0, 0, 0, 0, 1, _lib.ptr(a_scale), 0, _lib.ptr(b_scale), 0, 0, 0,
                              _lib.ptr(st), 0, _lib.stream_ptr(aq.device))
    _lib.check(err, "ats_gemm_fp8")
    return out


def input_grad(dy2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """dy2 [T, N] . w [N, K] -> [T, K]: e4m3 product of dy (per token) with the per-input-channel copy of w when the shapes allow
    it, else the bf16 product."""
    N, K = w.shape
    if N % 16 == 0 and K % 8 == 0 and _lib.use_cuda_kernels(dy2):
        gq, gs = quantize_rows(dy2)
        wq, ws = quantized_weight_t(w)
        return gemm_nt_fp8(gq, gs, wq, ws)
    return G.gemm_nn(dy2, w)


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
        dx = None
        if ctx.needs_input_grad[0]:
            dx = input_grad(dy2, w).view(ctx.shape)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _deliver_grad(w, lambda out, acc: G.gemm_tn(dy2, x2, out=out, accumulate=acc))
        return dx, dw, (dy if ctx.has_res else None)


def linear_fp8(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ residual)`` with e4m3 forward and input-gradient products; the weight gradient in bf16."""
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

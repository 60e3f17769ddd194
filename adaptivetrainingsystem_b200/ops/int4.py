"""Weight-only 4-bit linear layers (W4A16): group-wise asymmetric quantisation by GPTQ or round-to-nearest, bf16 activations.

A weight ``[N, K]`` is cut into groups of ``group`` (128) consecutive input channels per output feature; every group has a
scale and an integer zero point, codes are 0..15 and the value is ``(code - zero) * scale``.  :func:`gptq_quantize` picks the
codes column by column and pushes each column's rounding error onto the columns not yet quantised, weighted by the inverse
Hessian ``(X^T X + damping)^-1`` of the layer's calibration inputs (Frantar et al. 2022); without a Hessian the codes are plain
round-to-nearest.  The codes are stored in the order the decode kernel's tensor-core fragments want them (``csrc/int4.cu``):

* one to sixteen token rows: ``ats_gemv_int4`` streams the packed weight once (a quarter of the bf16 bytes) through a ring of
  asynchronous copies, feeds the codes to warp-level MMAs and applies zero point and scale per 64-channel step in fp32;
  residual add and SwiGLU are fused into its epilogue;
* more rows (a prompt): ``ats_dequant_int4`` writes the bf16 matrix and the tcgen05 GEMM does the product.

Only weights registered by :func:`register` (``QuantizationManager.quantize_model`` with method ``"int4"`` / ``"gptq"``) take
this path; nothing is quantised on the fly.  The reference reaches 4 bits through AutoGPTQ / bitsandbytes hooks
(``training/trainer.py:575-801``, bits 4, group 128) and its vendored inference engine through a Triton GPTQ matmul
(``colossalai/kernel/triton/gptq_triton.py``); neither ships here.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from . import gemm as G

_vp, _ci, _cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_sig = False
_enabled = False
_observing = False
_observe_only = None                          # storages whose Hessians are wanted (None: all)
GROUP = 128
MAX_HESSIAN_DIM = 16384                       # input widths above this are quantised round-to-nearest (the Hessian is K x K fp32)
GEMV_MAX_ROWS = 16                            # two token tiles of the streaming kernel; beyond that the dequantise + GEMM path
_weights: Dict[int, Tuple[int, Tuple[int, int], torch.Tensor, torch.Tensor, int]] = {}   # storage -> (version, shape, packed, meta, group)
_hessians: Dict[int, Tuple[torch.Tensor, int]] = {}                                       # storage -> (sum of x^T x, rows seen)


def set_enabled(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


def enabled() -> bool:
    return _enabled


def _fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_gemv_int4.restype = _ci
        lib.ats_gemv_int4.argtypes = [_vp, _vp, _vp, _cll, _vp, _cll, _vp, _cll, _ci, _ci, _ci, _ci, _ci, _vp]
        lib.ats_dequant_int4.restype = _ci
        lib.ats_dequant_int4.argtypes = [_vp, _vp, _vp, _cll, _ci, _ci, _ci, _vp]
        _sig = True
    return lib


def shape_ok(N: int, K: int, group: int = GROUP) -> bool:
    return N % 16 == 0 and K % 64 == 0 and group >= 64 and group & (group - 1) == 0 and K % group == 0


# -- quantisers ----------------------------------------------------------------------------------------------------------------
def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).float()


def group_params(w: torch.Tensor, sym: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [..., n] (groups of columns in the last dimension) -> (scale [...] rounded to bf16, zero [...] in 0..15) covering
    [min(w, 0), max(w, 0)]; ``sym``: the range is made symmetric and the zero point is 8 (AutoGPTQ's ``sym=True``)."""
    lo = w.amin(-1).clamp(max=0.0)
    hi = w.amax(-1).clamp(min=0.0)
    if sym:
        hi = torch.maximum(hi, -lo)
        lo = -hi
    scale = _bf16(((hi - lo) / 15.0).clamp(min=1e-8))
    zero = torch.full_like(scale, 8.0) if sym else torch.round(-lo / scale).clamp(0, 15)
    return scale, zero


def quantize_rtn(w: torch.Tensor, group: int = GROUP, sym: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Round to nearest: -> (codes [N, K] uint8, scale [N, K / group] fp32, zero [N, K / group] fp32)."""
    N, K = w.shape
    wf = w.detach().float().view(N, K // group, group)
    scale, zero = group_params(wf, sym)
    q = (torch.round(wf / scale[:, :, None]) + zero[:, :, None]).clamp(0, 15)
    return q.view(N, K).to(torch.uint8), scale, zero


def gptq_quantize(w: torch.Tensor, hessian: torch.Tensor, group: int = GROUP, damp: float = 0.01, sym: bool = False,
                  act_order: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """GPTQ: ``hessian`` = sum over calibration rows of x^T x, [K, K].  Same outputs as :func:`quantize_rtn`.

    ``act_order``: the columns are fixed in the order of decreasing Hessian diagonal (the input channels that matter most are
    rounded first, while every other column can still absorb their error); the groups stay the runs of 128 consecutive ORIGINAL
    channels with ranges taken up front (AutoGPTQ's ``desc_act`` with ``static_groups``), so the stored layout and the kernels do
    not change."""
    N, K = w.shape
    W = w.detach().float().clone()
    H = hessian.detach().float().clone().to(W.device)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    scale = torch.empty(N, K // group, device=W.device)
    zero = torch.empty(N, K // group, device=W.device)
    perm = None
    if act_order:
        scale, zero = group_params(W.view(N, K // group, group), sym)
        perm = torch.argsort(torch.diag(H), descending=True)
        W = W[:, perm]
        H = H[perm][:, perm]
        col_group = (perm // group).tolist()
    H += torch.eye(K, device=W.device) * (damp * torch.diag(H).mean())
    # upper Cholesky factor of H^-1: row i holds how the error of column i spreads over the columns after it
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    Q = torch.empty(N, K, dtype=torch.uint8, device=W.device)
    for b, i1 in enumerate(range(0, K, group)):
        i2 = i1 + group
        W1 = W[:, i1:i2].clone()
        E1 = torch.empty_like(W1)
        H1 = Hinv[i1:i2, i1:i2]
        if perm is None:
            sc, z = group_params(W1, sym)  # the group's range after the corrections pushed onto it by the groups before
            scale[:, b], zero[:, b] = sc, z
        for i in range(group):
            col = W1[:, i]
            if perm is not None:
                sc, z = scale[:, col_group[i1 + i]], zero[:, col_group[i1 + i]]
            q = (torch.round(col / sc) + z).clamp(0, 15)
            Q[:, i1 + i] = q.to(torch.uint8)
            err = (col - _bf16((q - z) * sc)) / H1[i, i]
            W1[:, i:] -= err[:, None] * H1[i, i:][None, :]
            E1[:, i] = err
        W[:, i2:] -= E1 @ Hinv[i1:i2, i2:]
    if perm is not None:
        Q = Q[:, torch.argsort(perm)]
    return Q, scale, zero


# -- packed format ---------------------------------------------------------------------------------------------------------------
def pack(q: torch.Tensor) -> torch.Tensor:
    """codes [N, K] (0..15) -> int32 [K / 64, N / 16, 32, 4]: word [S, T, 4 g + t, j], nibble i = feature 16 T + g + 8 (i & 1),
    input channel 64 S + 16 t + 4 j + 2 ((i >> 1) & 1) + (i >> 2).  The 64-channel step S is the outer index: the CTAs of the
    streaming kernel own feature tiles T and advance through S together, so what is in flight at any time is contiguous."""
    N, K = q.shape
    v = q.to(torch.int64).view(N // 16, 2, 8, K // 64, 4, 4, 2, 2)          # T, h, g, S, t, j, c, d ; nibble = h + 2 c + 4 d
    v = v.permute(3, 0, 2, 4, 5, 7, 6, 1).reshape(K // 64, N // 16, 32, 4, 8)   # S, T, (g, t), j, (d, c, h)
    shifts = torch.arange(8, device=q.device, dtype=torch.int64) * 4
    word = (v << shifts).sum(-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32).contiguous()


def unpack(packed: torch.Tensor) -> torch.Tensor:
    S, T = packed.shape[:2]
    word = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=packed.device, dtype=torch.int64) * 4
    v = ((word[..., None] >> shifts) & 15).view(S, T, 8, 4, 4, 2, 2, 2)        # S, T, g, t, j, d, c, h
    return v.permute(1, 7, 2, 0, 3, 4, 6, 5).reshape(T * 16, S * 64).to(torch.uint8)


def pack_meta(scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """(scale, zero) [N, G] -> int32 [G, N]: low half the bf16 bits of the scale, high half those of 128 + zero."""
    s_bits = scale.to(torch.bfloat16).view(torch.int16).to(torch.int64) & 0xFFFF
    z_bits = (zero.float() + 128.0).to(torch.bfloat16).view(torch.int16).to(torch.int64) & 0xFFFF
    word = s_bits | (z_bits << 16)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32).t().contiguous()


def unpack_meta(meta: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    word = meta.t().to(torch.int64) & 0xFFFFFFFF
    scale = (word & 0xFFFF).to(torch.int16).view(torch.bfloat16).float()
    zero = ((word >> 16) & 0xFFFF).to(torch.int16).view(torch.bfloat16).float() - 128.0
    return scale.contiguous(), zero.contiguous()


def dequantize_reference(packed: torch.Tensor, meta: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    q = unpack(packed).float()
    scale, zero = unpack_meta(meta)
    N, K = q.shape
    w = (q.view(N, K // group, group) - zero[:, :, None]) * scale[:, :, None]
    return w.view(N, K).to(torch.bfloat16)


def dequantize(packed: torch.Tensor, meta: torch.Tensor, group: int = GROUP, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The bf16 matrix [N, K] the packed weight stands for."""
    N, K = packed.shape[1] * 16, packed.shape[0] * 64
    if meta.shape != (K // group, N) or not packed.is_contiguous() or not meta.is_contiguous():
        raise ValueError(f"dequantize: scales {tuple(meta.shape)} do not fit the packed weight {N} x {K} (group {group})")
    if not packed.is_cuda:
        r = dequantize_reference(packed, meta, group)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=packed.device)
    if tuple(out.shape) != (N, K) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("dequantize: out must be a bf16 [N, K] matrix with unit column stride")
    err = _fns().ats_dequant_int4(_lib.ptr(packed), _lib.ptr(meta), _lib.ptr(out), out.stride(0), N, K, group, _lib.stream_ptr(packed.device))
    _lib.check(err, "ats_dequant_int4")
    return out


def gemv(x2: torch.Tensor, packed: torch.Tensor, meta: torch.Tensor, group: int = GROUP, add: Optional[torch.Tensor] = None,
         swiglu: bool = False) -> torch.Tensor:
    """x2 [M <= 16, K] bf16 @ W^T (+ add), or silu(gate) * up over the two halves of the features; the packed weight is read
    once."""
    M, K = x2.shape
    N = packed.shape[1] * 16
    if K != packed.shape[0] * 64 or meta.shape != (K // group, N) or M > GEMV_MAX_ROWS or not packed.is_contiguous() or not meta.is_contiguous():
        raise ValueError(f"gemv: activations {tuple(x2.shape)} do not fit the packed weight {N} x {packed.shape[0] * 64} (group {group})")
    n_out = N // 2 if swiglu else N
    if M == 0:
        return torch.empty(0, n_out, dtype=torch.bfloat16, device=x2.device)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if add is not None and (add.stride(1) != 1 or tuple(add.shape) != (M, n_out)):
        add = add.expand(M, n_out).contiguous()
    out = torch.empty(M, n_out, dtype=torch.bfloat16, device=x2.device)
    err = _fns().ats_gemv_int4(_lib.ptr(packed), _lib.ptr(meta), _lib.ptr(x2), x2.stride(0), _lib.ptr(add), add.stride(0) if add is not None else 0,
                               _lib.ptr(out), out.stride(0), M, N, K, group, int(swiglu), _lib.stream_ptr(x2.device))
    _lib.check(err, "ats_gemv_int4")
    return out


# -- calibration (Hessians for GPTQ) -----------------------------------------------------------------------------------------------
def observe(flag: bool, only=None) -> None:
    """While on, every ``ops.linear`` / MLP product adds x^T x of its input rows to the Hessian of its weight; ``only``: an
    iterable of weights to restrict the collection to (block-by-block calibration)."""
    global _observing, _observe_only
    _observing = bool(flag)
    _observe_only = None if (only is None or not flag) else {w.data_ptr() for w in only}


def observing() -> bool:
    return _observing


def record(x2: torch.Tensor, w: torch.Tensor) -> None:
    K = x2.shape[-1]
    if w.dim() != 2 or K > MAX_HESSIAN_DIM or (_observe_only is not None and w.data_ptr() not in _observe_only):
        return
    xf = x2.detach().reshape(-1, K).float()
    h = xf.t() @ xf
    key = w.data_ptr()
    prev = _hessians.get(key)
    _hessians[key] = (h, xf.shape[0]) if prev is None else (prev[0] + h, prev[1] + xf.shape[0])


def hessian_count() -> int:
    return len(_hessians)


def drop_hessians() -> None:
    """K x K fp32 per projection: not needed once the codes are fixed."""
    _hessians.clear()


def hessian_for(w: torch.Tensor) -> Optional[torch.Tensor]:
    hit = _hessians.get(w.data_ptr())
    return None if hit is None or hit[0].shape[0] != w.shape[1] else hit[0]


# -- registry ---------------------------------------------------------------------------------------------------------------------
def register(w: torch.Tensor, group: int = GROUP, damp: float = 0.01, sym: bool = False, act_order: bool = False
             ) -> Tuple[torch.Tensor, torch.Tensor, bool]:
    """Quantises ``w`` [N, K] (GPTQ when calibration left a Hessian for it, else round-to-nearest) and routes ``ops.linear`` /
    the SwiGLU MLP with this weight to the 4-bit kernels.  -> (packed, meta, used_gptq)."""
    N, K = w.shape
    if not shape_ok(N, K, group):
        raise ValueError(f"4-bit weights need N % 16 == 0, K % 64 == 0, a power-of-two group >= 64 dividing K (got {N} x {K}, group {group})")
    H = hessian_for(w)
    done = None
    if H is not None:
        for d in (damp, 10.0 * damp, 100.0 * damp):     # a Hessian of few calibration rows can defeat the fp32 factorisation
            try:
                done = gptq_quantize(w, H, group, d, sym, act_order)
                break
            except torch.linalg.LinAlgError:
                continue
    used_gptq = done is not None
    q, scale, zero = done if used_gptq else quantize_rtn(w, group, sym)
    packed, meta = pack(q), pack_meta(scale, zero)
    _weights[w.data_ptr()] = (w._version, (N, K), packed, meta, group)
    return packed, meta, used_gptq


def register_packed(w: torch.Tensor, packed: torch.Tensor, meta: torch.Tensor, group: int = GROUP) -> None:
    """Attaches an existing 4-bit copy (a saved one) to ``w`` without quantising anything."""
    N, K = w.shape
    if tuple(packed.shape) != (K // 64, N // 16, 32, 4) or tuple(meta.shape) != (K // group, N) or not shape_ok(N, K, group):
        raise ValueError(f"packed copy {tuple(packed.shape)} / {tuple(meta.shape)} does not describe a {N} x {K} weight with groups of {group}")
    _weights[w.data_ptr()] = (w._version, (N, K), packed.to(w.device, torch.int32).contiguous(), meta.to(w.device, torch.int32).contiguous(), group)


def release_original(w: torch.Tensor) -> int:
    """Frees the bf16 storage of a registered weight: ``w`` keeps its shape but points at one element broadcast over it
    (stride 0), so every read of its VALUES is meaningless from here on; only the 4-bit path may use it.  -> bytes freed."""
    hit = _weights.pop(w.data_ptr(), None)
    if hit is None or hit[0] != w._version or hit[1] != tuple(w.shape):
        raise ValueError("release_original: the weight has no current 4-bit copy")
    freed = w.numel() * w.element_size()
    stub = torch.zeros(1, dtype=w.dtype, device=w.device)
    w.data = stub.expand(*hit[1])
    _weights[w.data_ptr()] = (w._version, hit[1], hit[2], hit[3], hit[4])
    return freed


def lookup(w: torch.Tensor):
    """-> (packed, scale words, group) of the registered 4-bit copy of ``w``, or None (never registered, or changed since)."""
    hit = _weights.get(w.data_ptr())
    if hit is None or hit[0] != w._version or hit[1] != tuple(w.shape):
        return None
    return hit[2], hit[3], hit[4]


def clear() -> None:
    _weights.clear()
    _hessians.clear()


def usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    return _enabled and bool(_weights) and not torch.is_grad_enabled() and w.dim() == 2 and lookup(w) is not None


# -- layers ------------------------------------------------------------------------------------------------------------------------
def _matmul(x2: torch.Tensor, entry, add: Optional[torch.Tensor], swiglu: bool = False) -> torch.Tensor:
    packed, meta, group = entry
    if not _lib.use_cuda_kernels(x2):
        wd = dequantize_reference(packed, meta, group)
        if swiglu:
            return G.gemm_nt_swiglu(x2, wd.to(x2.dtype))
        return G.gemm_nt(x2, wd.to(x2.dtype), add=add)
    if x2.shape[0] <= GEMV_MAX_ROWS:
        return gemv(x2, packed, meta, group, add=add, swiglu=swiglu)
    wd = dequantize(packed, meta, group)
    if swiglu:
        return G.gemm_nt_swiglu(x2, wd)
    return G.gemm_nt(x2, wd, add=add)


@torch.no_grad()
def linear_int4(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ residual)`` with the registered 4-bit copy of ``w`` (inference only)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
    y = _matmul(x2, lookup(w), r2)
    return y.view(*shape[:-1], w.shape[0])


@torch.no_grad()
def swiglu_mlp_int4(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    h = _matmul(x2, lookup(w1), None, swiglu=True)
    r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
    y = _matmul(h, lookup(w2), r2)
    return y.view(*shape[:-1], w2.shape[0])


@torch.no_grad()
def swiglu_mlp_observed(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The unquantised MLP in two steps, so that calibration sees the input of the down projection too."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    record(x2, w1)
    h = G.gemm_nt_swiglu(x2, w1)
    record(h, w2)
    r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
    y = G.gemm_nt(h, w2, add=r2)
    return y.view(*shape[:-1], w2.shape[0])

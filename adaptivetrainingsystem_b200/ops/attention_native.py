"""Autograd wrappers of the tcgen05 flash-attention kernels (``csrc/attention_tcgen05.cu`` forward,
``csrc/attention_bwd_tcgen05.cu`` backward).

Both directions read q / k / v in place from the packed QKV projection (strided views become tensor maps).  The packed
entry point takes the whole ``[B, L, (Hq + 2 Hkv) * D]`` projection and returns its gradient as one tensor, so autograd
never has to zero-pad and add three sliced gradients.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_vp, _ci, _cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_sig = False


def _lib_fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_attn_fwd.restype = _ci
        lib.ats_attn_fwd.argtypes = [_vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _vp,
                                     _ci, _ci, _ci, _ci, _ci, _vp, _vp]
        lib.ats_attn_fwd2.restype = _ci
        lib.ats_attn_fwd2.argtypes = [_vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _vp,
                                      _ci, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp]
        lib.ats_attn_fwd2_set_poly.restype = _ci
        lib.ats_attn_fwd2_set_poly.argtypes = [_ci]
        if "ATS_ATTN_POLY" in os.environ:
            lib.ats_attn_fwd2_set_poly(int(os.environ["ATS_ATTN_POLY"]))
        lib.ats_attn_bwd.restype = _ci
        lib.ats_attn_bwd.argtypes = [_vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                     _cll, _cll, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp]
        _sig = True
    return lib


def layout_ok(t: torch.Tensor) -> bool:
    """[B, L, H, D] view whose token rows are evenly pitched: stride = (L * pitch, pitch, D, 1), 16-byte aligned."""
    B, L, H, D = t.shape
    s = t.stride()
    return (s[3] == 1 and s[2] == D and s[0] == L * s[1] and s[1] % 8 == 0 and t.data_ptr() % 16 == 0)


# Forward variant: "v1" = one query tile per CTA; "v2s" / "v2t" = two query tiles per CTA with the probabilities staged
# through shared memory / tensor memory (sequence length must be a multiple of 256, else v1 runs).
FWD_VARIANT = os.environ.get("ATS_ATTN_FWD", "v2t")
# Diagnostics: an int64 CUDA tensor of 16 elements receives per-phase cycle totals of one CTA of the two-tile forward kernel
# ([0:5] MMA thread: total, wait for V, wait for P, issue, iterations; [8:13] one soft-max warp: wait for S, TMEM load, row
# maximum, exponentials + store, signalling).
FWD_PHASE_PROFILE = None


def _fwd(q, k, v):
    B, L, Hq, D = q.shape
    Hkv = k.shape[2]
    out = torch.empty(B, L, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
    st = _lib.status_tensor(q.device)
    if FWD_VARIANT != "v1" and L % 256 == 0:
        err = _lib_fns().ats_attn_fwd2(_lib.ptr(q), q.stride(1), Hq * D, 0, _lib.ptr(k), k.stride(1), Hkv * D, 0, _lib.ptr(v), v.stride(1),
                                       Hkv * D, 0, _lib.ptr(out), _lib.ptr(lse), B, L, Hq, Hkv, D, int(FWD_VARIANT == "v2t"), _lib.ptr(st),
                                       _lib.ptr(FWD_PHASE_PROFILE), _lib.stream_ptr(q.device))
        _lib.check(err, "ats_attn_fwd2")
        return out, lse
    err = _lib_fns().ats_attn_fwd(_lib.ptr(q), q.stride(1), Hq * D, 0, _lib.ptr(k), k.stride(1), Hkv * D, 0, _lib.ptr(v), v.stride(1),
                                  Hkv * D, 0, _lib.ptr(out), _lib.ptr(lse), B, L, Hq, Hkv, D, _lib.ptr(st), _lib.stream_ptr(q.device))
    _lib.check(err, "ats_attn_fwd")
    return out, lse


# Diagnostics: set to an int64 CUDA tensor of 32 elements to receive per-phase cycle totals of one CTA of each backward
# pass ([0:16] dK/dV pass, [16:32] dQ pass: total, waits of the MMA thread, issue time; [8:13] phases of one softmax warp).
PHASE_PROFILE = None


def _bwd(q, k, v, out, dout, lse, dq, dk, dv):
    B, L, Hq, D = q.shape
    Hkv = k.shape[2]
    delta = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
    st = _lib.status_tensor(q.device)
    err = _lib_fns().ats_attn_bwd(_lib.ptr(q), q.stride(1), Hq * D, 0, _lib.ptr(k), k.stride(1), Hkv * D, 0, _lib.ptr(v), v.stride(1),
                                  Hkv * D, 0, _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(dk),
                                  _lib.ptr(dv), dq.stride(1), dk.stride(1), B, L, Hq, Hkv, D, _lib.ptr(st), _lib.ptr(PHASE_PROFILE),
                                  _lib.stream_ptr(q.device))
    _lib.check(err, "ats_attn_bwd")


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        out, lse = _fwd(q, k, v)
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dout = dout.contiguous()
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        _bwd(q, k, v, out, dout, lse, dq, dk, dv)
        return dq, dk, dv


class _FlashAttnPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, d):
        B, L, W = qkv.shape
        nq, nk = n_q * d, n_kv * d
        q = qkv[..., :nq].view(B, L, n_q, d)
        k = qkv[..., nq:nq + nk].view(B, L, n_kv, d)
        v = qkv[..., nq + nk:].view(B, L, n_kv, d)
        out, lse = _fwd(q, k, v)
        ctx.save_for_backward(qkv, out, lse)
        ctx.dims = (n_q, n_kv, d)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        n_q, n_kv, d = ctx.dims
        B, L, W = qkv.shape
        nq, nk = n_q * d, n_kv * d
        q = qkv[..., :nq].view(B, L, n_q, d)
        k = qkv[..., nq:nq + nk].view(B, L, n_kv, d)
        v = qkv[..., nq + nk:].view(B, L, n_kv, d)
        dqkv = torch.empty_like(qkv)
        _bwd(q, k, v, out, dout.contiguous(), lse, dqkv[..., :nq].view(B, L, n_q, d), dqkv[..., nq:nq + nk].view(B, L, n_kv, d),
             dqkv[..., nq + nk:].view(B, L, n_kv, d))
        return dqkv, None, None, None


class _RopeAttnPackedFn(torch.autograd.Function):
    """RoPE (in place on the packed projection) followed by causal attention, as one autograd node: the backward pass rotates
    the gradient of q / k back inside the buffer the attention backward has just written, without a defensive copy."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_q, n_kv, d, pos_offset):
        from .functional import _L, _P, _S, _CK
        B, L, W = qkv.shape
        ctx.mark_dirty(qkv)
        # the rotated projection is returned only because it was modified in place; when nothing downstream uses it, its
        # gradient must arrive as None, not as a zero tensor of the projection's size that backward would fill and add
        ctx.set_materialize_grads(False)
        _CK(_L().ats_rope(_P(qkv), _P(cos), _P(sin), None, B * L, L, pos_offset, W, 0, n_q + n_kv, d, 0, _S(qkv.device)), "rope")
        nq, nk = n_q * d, n_kv * d
        out, lse = _fwd(qkv[..., :nq].view(B, L, n_q, d), qkv[..., nq:nq + nk].view(B, L, n_kv, d), qkv[..., nq + nk:].view(B, L, n_kv, d))
        ctx.save_for_backward(qkv, out, lse, cos, sin)
        ctx.dims = (n_q, n_kv, d, pos_offset)
        return qkv, out

    @staticmethod
    def backward(ctx, _dqkv_unused, dout):
        from .functional import _L, _P, _S, _CK
        qkv, out, lse, cos, sin = ctx.saved_tensors
        n_q, n_kv, d, pos_offset = ctx.dims
        B, L, W = qkv.shape
        nq, nk = n_q * d, n_kv * d
        if dout is None:  # only the rotated projection was used downstream
            dqkv = _dqkv_unused.clone() if _dqkv_unused is not None else torch.zeros_like(qkv)
            _CK(_L().ats_rope(_P(dqkv), _P(cos), _P(sin), None, B * L, L, pos_offset, W, 0, n_q + n_kv, d, 1, _S(dqkv.device)), "rope_bwd")
            return dqkv, None, None, None, None, None, None
        dqkv = torch.empty_like(qkv)
        _bwd(qkv[..., :nq].view(B, L, n_q, d), qkv[..., nq:nq + nk].view(B, L, n_kv, d), qkv[..., nq + nk:].view(B, L, n_kv, d), out,
             dout.contiguous(), lse, dqkv[..., :nq].view(B, L, n_q, d), dqkv[..., nq:nq + nk].view(B, L, n_kv, d),
             dqkv[..., nq + nk:].view(B, L, n_kv, d))
        if _dqkv_unused is not None:  # the rotated projection itself was used downstream as well
            dqkv += _dqkv_unused
        _CK(_L().ats_rope(_P(dqkv), _P(cos), _P(sin), None, B * L, L, pos_offset, W, 0, n_q + n_kv, d, 1, _S(dqkv.device)), "rope_bwd")
        return dqkv, None, None, None, None, None, None


def rope_flash_attention_packed(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_q: int, n_kv: int, d: int,
                                pos_offset: int = 0) -> torch.Tensor:
    """qkv [B, L, (n_q + 2 n_kv) d] straight from the projection GEMM -> attention output [B, L, n_q, d]; qkv is rotated in place."""
    if cos.dtype != torch.float32 or sin.dtype != torch.float32:
        raise TypeError("rope tables must be float32")
    return _RopeAttnPackedFn.apply(qkv, cos, sin, n_q, n_kv, d, pos_offset)[1]


def flash_attention_native(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    return _FlashAttnFn.apply(q, k, v)


def flash_attention_packed(qkv: torch.Tensor, n_q: int, n_kv: int, d: int) -> torch.Tensor:
    """qkv: [B, L, (n_q + 2 n_kv) * d] contiguous -> [B, L, n_q, d]; causal, grouped-query."""
    return _FlashAttnPackedFn.apply(qkv, n_q, n_kv, d)

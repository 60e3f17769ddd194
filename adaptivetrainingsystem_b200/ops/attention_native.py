"""Autograd wrapper of the tcgen05 flash-attention forward kernel (``csrc/attention_tcgen05.cu``).

Forward reads q / k / v in place from the packed projection (strided views are passed as tensor maps).  The backward
pass currently re-derives the gradients through PyTorch's fused SDPA (a library call) from the saved inputs; the
tcgen05 backward kernel replaces it when ``ats_attn_bwd`` is present in the library.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_vp, _ci, _cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_sig = False


def _fn():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_attn_fwd.restype = _ci
        lib.ats_attn_fwd.argtypes = [_vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _cll, _cll, _ci, _vp, _vp,
                                     _ci, _ci, _ci, _ci, _ci, _vp, _vp]
        _sig = True
    return lib.ats_attn_fwd


def layout_ok(t: torch.Tensor) -> bool:
    """[B, L, H, D] view whose token rows are evenly pitched: stride = (L * pitch, pitch, D, 1), 16-byte aligned."""
    B, L, H, D = t.shape
    s = t.stride()
    return (s[3] == 1 and s[2] == D and s[0] == L * s[1] and s[1] % 8 == 0 and t.data_ptr() % 16 == 0)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        B, L, Hq, D = q.shape
        Hkv = k.shape[2]
        out = torch.empty(B, L, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
        st = _lib.status_tensor(q.device)
        err = _fn()(_lib.ptr(q), q.stride(1), Hq * D, 0, _lib.ptr(k), k.stride(1), Hkv * D, 0, _lib.ptr(v), v.stride(1), Hkv * D, 0,
                    _lib.ptr(out), _lib.ptr(lse), B, L, Hq, Hkv, D, _lib.ptr(st), _lib.stream_ptr(q.device))
        _lib.check(err, "ats_attn_fwd")
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        with torch.enable_grad():
            qd, kd, vd = [t.detach().requires_grad_() for t in (q, k, v)]
            o = F.scaled_dot_product_attention(qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2), is_causal=True,
                                               enable_gqa=q.shape[2] != k.shape[2]).transpose(1, 2)
            dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), dout)
        return dq, dk, dv


def flash_attention_native(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    return _FlashAttnFn.apply(q, k, v)

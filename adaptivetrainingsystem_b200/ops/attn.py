"""Causal grouped-query attention on CUDA.

``flash_attention`` runs the tcgen05 kernel of ``csrc/attention_tcgen05.cu`` when the shape is one it
covers (head_dim 64 or 128, sequence a multiple of 128, bf16).  Other shapes use PyTorch's fused SDPA, which
is a library call and is reported as such by ``backend_for``.

Replaces ``flash_attn_func(causal=True)`` plus the ``repeat_interleave`` K/V expansion of the reference
(``core/model.py:705-768``); K/V heads are shared by the query heads of a group without being copied.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib


def _native_available() -> bool:
    if os.environ.get("ATS_ATTN", "native") != "native":
        return False
    try:
        return hasattr(_lib.cuda_lib(), "ats_attn_fwd")
    except Exception:
        return False


def supported(q, k, v, causal, q_offset) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16


def backend_for(q, k, causal=True, q_offset=0) -> str:
    """"tcgen05" (own kernel) or "sdpa" (PyTorch library kernel) for these operands."""
    B, Lq, Hq, D = q.shape
    Lk = k.shape[1]
    if _native_available() and D in (64, 128) and Lq % 128 == 0 and causal and Lq == Lk and q_offset == 0:
        from .attention_native import layout_ok
        if layout_ok(q) and layout_ok(k):
            return "tcgen05"
    return "sdpa"


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, q_offset: int = 0) -> torch.Tensor:
    """q: [B, Lq, Hq, D]; k, v: [B, Lk, Hkv, D] -> [B, Lq, Hq, D]."""
    if backend_for(q, k, causal, q_offset) == "tcgen05":
        from .attention_native import flash_attention_native, layout_ok
        if not layout_ok(v):
            v = v.contiguous()
        return flash_attention_native(q, k, v)
    B, Lq, Hq, D = q.shape
    Lk, Hkv = k.shape[1], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if causal and Lq == Lk and q_offset == 0:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=Hq != Hkv)
    elif Lq == 1 or not causal:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=False, enable_gqa=Hq != Hkv)
    else:
        qi = torch.arange(Lq, device=q.device)[:, None] + q_offset
        kj = torch.arange(Lk, device=q.device)[None, :]
        o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=(kj <= qi), enable_gqa=Hq != Hkv)
    return o.transpose(1, 2)

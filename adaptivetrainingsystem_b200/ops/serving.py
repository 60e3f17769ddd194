"""Serving operators: single-token attention against the KV cache and batched sampling (``csrc/inference.cu``).

The reference generator has no cache and samples with eager tensor ops (reference ``Chat.py:379-452``); the sampling
order (repetition penalty -> temperature -> top-k -> top-p -> multinomial) is kept.  CPU / fp32 inputs run the PyTorch
definitions below, which are also the oracles of the kernel tests.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib

_vp, _ci, _cll, _cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_sig = False
_scratch = {}


def _fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_decode_attn_chunks.restype = _ci
        lib.ats_decode_attn_chunks.argtypes = [_ci]
        lib.ats_decode_attn.restype = _ci
        lib.ats_decode_attn.argtypes = [_vp, _cll, _ci, _ci, _ci, _vp, _vp, _cll, _vp, _ci, _ci, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp, _vp, _vp]
        lib.ats_fold_rope.restype = _ci
        lib.ats_fold_rope.argtypes = [_vp, _ci, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, _vp]
        lib.ats_fold_add_norm.restype = _ci
        lib.ats_fold_add_norm.argtypes = [_vp, _ci, _vp, _vp, _vp, _vp, _ci, _ci, _cf, _vp]
        lib.ats_sample.restype = _ci
        lib.ats_sample.argtypes = [_vp, _ci, _cll, _vp, _vp, _ci, _ci, _vp, _vp, _ci, _ci, _cf, _ci, _cf, _cf, _vp]
        _sig = True
    return lib


def _buf(key, numel: int, dtype, device) -> torch.Tensor:
    k = (key, dtype, torch.device(device).index)
    t = _scratch.get(k)
    if t is None or t.numel() < numel:
        t = torch.empty(numel, dtype=dtype, device=device)
        _scratch[k] = t
    return t


# ----------------------------------------------------------------------------------------------------------
# Fused pieces of a decode step.  With a handful of tokens a projection splits its reduction over the SMs and leaves fp32 partial
# products; the launch that folds them also does what would otherwise be the next launch: the rotary embedding of the packed
# q / k / v projection, or the residual add and the RMSNorm that follows the output projection.
# ----------------------------------------------------------------------------------------------------------
FUSE_DECODE = __import__("os").environ.get("ATS_DECODE_FUSED", "1") == "1"
# Flash-decoding merge inside the attention kernel (the CTA that arrives last for a sequence and KV head merges the chunk
# partials) instead of a launch of its own.  Off by default: measured on one box it changed the decode step by -0.5 % on the
# 22-layer model (64-wide heads) and +1.6 % on the Mixtral shape, where the merge lengthens the tail of a kernel that is already
# the long pole of the layer.
MERGE_INSIDE = __import__("os").environ.get("ATS_DECODE_MERGE_INSIDE", "0") == "1"


def _partial_products(x2: torch.Tensor, w: torch.Tensor):
    """fp32 partial products [splits, T, N] of x2 [T, K] @ w [N, K]^T over slices of the reduction, or ``None`` when this shape
    does not split (the caller then uses the ordinary product)."""
    from . import gemm as G
    T, K = x2.shape
    N = w.shape[0]
    if not (FUSE_DECODE and _lib.use_cuda_kernels(x2) and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and x2.is_contiguous() and w.is_contiguous() and not getattr(w, "_ats_z3", None) and G.SPLIT_K_SKINNY):
        return None
    from . import int4
    if int4.enabled() and int4.lookup(w) is not None:
        return None          # a 4-bit weight: the caller's ordinary product streams the packed copy
    splits = G._skinny_splits(T, N, K)
    if splits < 2:
        return None
    kp = K // splits
    part = torch.empty(splits, T, N, dtype=torch.float32, device=x2.device)
    G._raw(x2, T, K, K, 0, w, N, K, K, 0, part, N, None, 0, None, 0, T, N, kp, epilogue=G.EPI_F32, groups=splits, a_gs_k=kp, b_gs_k=kp,
           d_gs=T * N)
    return part


def qkv_rope(h2: torch.Tensor, w_qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, n_q: int, n_kv: int,
             d: int) -> Optional[torch.Tensor]:
    """Packed projection of the new tokens with q and k rotated at ``positions`` [T] (int32): one product + one fold launch.
    ``None`` when the fused form does not apply."""
    if d % 16 or positions is None or positions.dtype != torch.int32 or cos.dtype != torch.float32 or w_qkv.shape[0] != (n_q + 2 * n_kv) * d:
        return None
    part = _partial_products(h2, w_qkv)
    if part is None:
        return None
    T, N = h2.shape[0], w_qkv.shape[0]
    out = torch.empty(T, N, dtype=h2.dtype, device=h2.device)
    err = _fns().ats_fold_rope(_lib.ptr(part), part.shape[0], _lib.ptr(out), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(positions), T, N, n_q, n_kv, d,
                               _lib.stream_ptr(h2.device))
    _lib.check(err, "ats_fold_rope")
    return out


def out_proj_norm(a2: torch.Tensor, w_o: torch.Tensor, residual2: torch.Tensor, norm_w: torch.Tensor, eps: float):
    """x = a2 @ w_o^T + residual2 and h = RMSNorm(x) * norm_w from one product + one fold launch -> (x, h), or ``None``."""
    if norm_w.dtype != torch.bfloat16 or residual2 is None or not residual2.is_contiguous():
        return None
    part = _partial_products(a2, w_o)
    if part is None:
        return None
    T, H = a2.shape[0], w_o.shape[0]
    x = torch.empty(T, H, dtype=a2.dtype, device=a2.device)
    h = torch.empty_like(x)
    err = _fns().ats_fold_add_norm(_lib.ptr(part), part.shape[0], _lib.ptr(residual2), _lib.ptr(norm_w), _lib.ptr(x), _lib.ptr(h), T, H, float(eps),
                                   _lib.stream_ptr(a2.device))
    _lib.check(err, "ats_fold_add_norm")
    return x, h


def decode_attention_available(qkv: torch.Tensor, n_q: int, n_kv: int, d: int) -> bool:
    return (_lib.use_cuda_kernels(qkv) and qkv.dim() == 3 and qkv.shape[1] == 1 and qkv.is_contiguous() and d in (64, 128)
            and n_q % n_kv == 0 and n_q // n_kv in (1, 2, 4, 8) and qkv.shape[-1] % 8 == 0)


def decode_attention(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, length, n_q: int, n_kv: int, d: int,
                     max_tokens: Optional[int] = None) -> torch.Tensor:
    """qkv: [B, 1, (n_q + 2 n_kv) d] projection of the new token (RoPE already applied).  k_cache / v_cache:
    [B, max_len, n_kv, d]; ``length`` = tokens already cached (int for all sequences, or an int32 tensor [B]).
    Writes the new K / V at position ``length`` and returns the attention output [B, 1, n_q d]."""
    B = qkv.shape[0]
    max_len = k_cache.shape[1]
    per_seq = isinstance(length, torch.Tensor)
    longest = int(max_tokens if max_tokens is not None else (max_len - 1 if per_seq else length))
    if longest + 1 > max_len:
        raise RuntimeError(f"KV cache overflow: {longest}+1 > {max_len}")
    if not decode_attention_available(qkv, n_q, n_kv, d):
        return decode_attention_reference(qkv, k_cache, v_cache, length, n_q, n_kv, d)
    lib = _fns()
    chunks = lib.ats_decode_attn_chunks(max_len)
    part_o = _buf("dec_o", B * n_q * chunks * d, torch.float32, qkv.device)
    part_ml = _buf("dec_ml", B * n_q * chunks * 2, torch.float32, qkv.device)
    # arrival counters of the (sequence, KV head) pairs: the CTA that arrives last merges the chunk partials and puts its counter
    # back to zero, so the buffer is zeroed once, when it is made
    key = ("dec_cnt", torch.int32, qkv.device.index)
    done = _scratch.get(key)
    if done is None or done.numel() < B * n_kv:
        done = torch.zeros(max(B * n_kv, 1024), dtype=torch.int32, device=qkv.device)
        _scratch[key] = done
    out = torch.empty(B, 1, n_q * d, dtype=qkv.dtype, device=qkv.device)
    err = lib.ats_decode_attn(_lib.ptr(qkv), qkv.stride(0), 0, n_q * d, (n_q + n_kv) * d, _lib.ptr(k_cache), _lib.ptr(v_cache),
                              k_cache.stride(0), _lib.ptr(length) if per_seq else None, 0 if per_seq else int(length), longest, B, n_q,
                              n_kv, d, max_len, _lib.ptr(part_o), _lib.ptr(part_ml), _lib.ptr(done) if MERGE_INSIDE else None, _lib.ptr(out),
                              _lib.stream_ptr(qkv.device))
    _lib.check(err, "ats_decode_attn")
    return out


def decode_attention_reference(qkv, k_cache, v_cache, length, n_q, n_kv, d) -> torch.Tensor:
    B = qkv.shape[0]
    nq, nk = n_q * d, n_kv * d
    q = qkv[:, 0, :nq].view(B, n_q, d).float()
    k_new = qkv[:, 0, nq:nq + nk].view(B, n_kv, d)
    v_new = qkv[:, 0, nq + nk:].view(B, n_kv, d)
    lens = length.tolist() if isinstance(length, torch.Tensor) else [int(length)] * B
    out = torch.empty(B, 1, nq, dtype=qkv.dtype, device=qkv.device)
    rep = n_q // n_kv
    for b, n in enumerate(lens):
        k_cache[b, n] = k_new[b]
        v_cache[b, n] = v_new[b]
        k = k_cache[b, : n + 1].float().repeat_interleave(rep, dim=1)  # [n+1, n_q, d]
        v = v_cache[b, : n + 1].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b], k) / math.sqrt(d)
        out[b, 0] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).reshape(nq).to(qkv.dtype)
    return out


def sample_tokens(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repetition_penalty: float = 1.0,
                  history: Optional[torch.Tensor] = None, uniform: Optional[torch.Tensor] = None,
                  generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """logits [B, V] (bf16 or fp32, CUDA) -> token ids [B] int64 in one launch.  ``uniform`` ([B] in [0, 1)) makes the
    draw reproducible; by default it comes from ``generator``."""
    B, V = logits.shape
    if not logits.is_cuda:
        raise RuntimeError("sample_tokens runs the CUDA kernel; use sample_reference on the CPU")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    if logits.dtype not in (torch.float32, torch.bfloat16):
        logits = logits.float()
    if uniform is None:
        uniform = torch.rand(B, device=logits.device, generator=generator)
    hist = None
    if history is not None and history.numel() and repetition_penalty != 1.0:
        hist = history.to(torch.int64)
        if hist.stride(1) != 1:
            hist = hist.contiguous()
    work = _buf("smp", B * V, torch.float32, logits.device)
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    err = _fns().ats_sample(_lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), _lib.ptr(work), _lib.ptr(hist),
                            0 if hist is None else hist.shape[1], 0 if hist is None else hist.stride(0), _lib.ptr(uniform.float()),
                            _lib.ptr(out), B, V, float(temperature), int(top_k), float(top_p), float(repetition_penalty),
                            _lib.stream_ptr(logits.device))
    _lib.check(err, "ats_sample")
    return out


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repetition_penalty: float = 1.0,
                     history: Optional[torch.Tensor] = None, uniform: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same distribution with sort-based PyTorch ops; with ``uniform`` given, the same inverse-CDF draw in index order."""
    lg = logits.float().clone()
    if history is not None and history.numel() and repetition_penalty != 1.0:
        picked = torch.gather(lg, 1, history)
        picked = torch.where(picked > 0, picked / repetition_penalty, picked * repetition_penalty)
        lg = lg.scatter(1, history, picked)
    if temperature <= 0:
        return lg.argmax(-1)
    lg = lg / temperature
    if top_k and top_k < lg.shape[-1]:
        kth = torch.topk(lg, top_k, dim=-1).values[:, -1:]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    if top_p < 1.0:
        sl, si = torch.sort(lg, dim=-1, descending=True)
        sp = torch.softmax(sl, -1)
        drop = sp.cumsum(-1) - sp > top_p
        sl = sl.masked_fill(drop, float("-inf"))
        lg = torch.full_like(lg, float("-inf")).scatter(1, si, sl)
    probs = torch.softmax(lg, -1)
    if uniform is None:
        return torch.multinomial(probs, 1).squeeze(1)
    cdf = probs.cumsum(-1)
    idx = (cdf <= uniform.float().unsqueeze(1) * cdf[:, -1:]).sum(-1)
    return idx.clamp(max=lg.shape[-1] - 1)

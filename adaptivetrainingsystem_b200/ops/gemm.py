"""bf16 GEMMs on the tcgen05 kernel (``csrc/gemm_tcgen05.cu``) and their PyTorch definitions.

Naming: ``nt`` = A[M,K] · B[N,K]ᵀ, ``nn`` = A[M,K] · B[K,N], ``tn`` = A[K,M]ᵀ · B[K,N]; all row-major.
These are the three products of a linear layer (forward, input gradient, weight gradient); none needs a
transposed copy because the kernel reads either operand K-major or MN-major.

Grouped forms work on the expert capacity layout ``[E, C, *]`` with a device-side ``counts[E]`` (rows of
group ``e`` actually used; pad rows up to the next multiple of 128 must be zero).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib

EPI_STORE, EPI_ADDC, EPI_F32, EPI_SWIGLU, EPI_SWIGLU_BWD = 0, 1, 2, 3, 4

_c_int, _c_ll, _c_f, _vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
_configured = False


def _fn():
    global _configured
    lib = _lib.cuda_lib()
    if not _configured:
        lib.ats_gemm_bf16.restype = _c_int
        lib.ats_gemm_bf16.argtypes = [
            _vp, _c_ll, _c_ll, _c_ll, _c_int,  # A
            _vp, _c_ll, _c_ll, _c_ll, _c_int,  # B
            _vp, _c_int, _vp, _c_int, _vp, _c_int,  # D, C, aux
            _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int,  # M N K alpha beta epilogue up_offset
            _c_int, _c_int, _vp,  # groups ragged counts
            _c_int, _c_int, _c_int, _c_int,  # group coordinate shifts
            _c_ll, _c_ll, _c_ll,  # d_gs c_gs aux_gs
            _c_int, _c_int, _c_int, _vp, _c_int, _c_int,  # b_div k_segs seg_stride d_table k_split scatter_rows
            _vp, _c_int, _vp]  # status, max_ctas, stream
        lib.ats_splitk_reduce.restype = _c_int
        lib.ats_splitk_reduce.argtypes = [_vp, _c_int, _c_ll, _c_ll, _vp, _vp, _vp]
        lib.ats_gemm_set_pair.restype = None
        lib.ats_gemm_set_pair.argtypes = [_c_int]
        if os.environ.get("ATS_GEMM_PAIR") is not None:
            lib.ats_gemm_set_pair(int(os.environ["ATS_GEMM_PAIR"]))
        lib.ats_gemm_set_wide_stores.restype = None
        lib.ats_gemm_set_wide_stores.argtypes = [_c_int]
        if os.environ.get("ATS_GEMM_WIDE_STORES") is not None:
            lib.ats_gemm_set_wide_stores(int(os.environ["ATS_GEMM_WIDE_STORES"]))
        _configured = True
    return lib.ats_gemm_bf16


def set_pair_kernels(on: bool) -> None:
    """Products with at least 256 rows run on pairs of CTAs (``tcgen05.mma.cta_group::2``, the default) or on single CTAs."""
    _fn()
    _lib.cuda_lib().ats_gemm_set_pair(int(bool(on)))


def _raw(a, a_rows, a_cols, lda, a_mn, b, b_rows, b_cols, ldb, b_mn, d, ldd, c, ldc, aux, ldaux,
         M, N, K, alpha=1.0, beta=0, epilogue=EPI_STORE, up_offset=0, groups=1, ragged=0, counts=None,
         a_gs_mn=0, a_gs_k=0, b_gs_mn=0, b_gs_k=0, d_gs=0, c_gs=0, aux_gs=0, max_ctas=0,
         b_div=1, k_segs=1, seg_stride=0, d_table=None, k_split=1, scatter_rows=0):
    st = _lib.status_tensor(a.device)
    err = _fn()(_lib.ptr(a), a_rows, a_cols, lda, a_mn, _lib.ptr(b), b_rows, b_cols, ldb, b_mn,
                _lib.ptr(d), ldd, _lib.ptr(c), ldc, _lib.ptr(aux), ldaux,
                M, N, K, alpha, beta, epilogue, up_offset, groups, ragged, _lib.ptr(counts),
                a_gs_mn, a_gs_k, b_gs_mn, b_gs_k, d_gs, c_gs, aux_gs,
                b_div, k_segs, seg_stride, _lib.ptr(d_table), k_split, scatter_rows,
                _lib.ptr(st), max_ctas, _lib.stream_ptr(a.device))
    _lib.check(err, "ats_gemm_bf16")


def _check2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if t.stride(1) != 1 or (t.stride(0) % 8) or (t.data_ptr() % 16):
        t = t.contiguous()
    return t


# Skinny products (a decode step: M = batch rows, few 256-column output tiles) would occupy N / 256 of the 148 SMs and stream
# the weight at a fraction of HBM bandwidth; the reduction dimension is split over groups of the grouped kernel instead, every
# group writing an fp32 partial product that a small reduction folds.  ATS_SPLIT_K=0 switches it off.
SPLIT_K_SKINNY = os.environ.get("ATS_SPLIT_K", "1") == "1"


def _skinny_splits(M: int, N: int, K: int) -> int:
    if M > 128 or K < 2048:
        return 1
    tiles = (N + 255) // 256
    s = 1
    while s * 2 * tiles <= 160 and K % (s * 2 * 64) == 0 and K // (s * 2) >= 512 and s < 16:
        s *= 2
    return s


def _gemm_nt_split_k(a, b, out, add, alpha, splits):
    M, K = a.shape
    N = b.shape[0]
    kp = K // splits
    part = torch.empty(splits, M, N, dtype=torch.float32, device=a.device)
    _raw(a, M, K, a.stride(0), 0, b, N, K, b.stride(0), 0, part, N, None, 0, None, 0, M, N, kp, alpha=alpha, beta=0,
         epilogue=EPI_F32, groups=splits, a_gs_k=kp, b_gs_k=kp, d_gs=M * N)
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    if out.is_contiguous() and (add is None or add.is_contiguous()):
        _fold_partials(part, splits, M * N, 1, out, add)  # one launch: sum of the slices (+ residual) -> bf16
        return out
    res = part.sum(0)
    if add is not None:
        res += add
    out.copy_(res)
    return out


def _fold_partials(part: torch.Tensor, splits: int, n_inner: int, n_outer: int, out: torch.Tensor, add: Optional[torch.Tensor] = None) -> None:
    """out[o, :] = sum over the ``splits`` fp32 partial blocks of problem ``o`` (+ add), written as bf16."""
    _fn()
    _lib.check(_lib.cuda_lib().ats_splitk_reduce(_lib.ptr(part), splits, n_inner, n_outer, _lib.ptr(out), _lib.ptr(add),
                                                 _lib.stream_ptr(part.device)), "splitk_reduce")


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
            add: Optional[torch.Tensor] = None, alpha: float = 1.0, out_fp32: bool = False,
            accumulate: bool = False, max_ctas: int = 0) -> torch.Tensor:
    """a[M,K] @ b[N,K]^T (+ add).  ``out_fp32`` writes (or accumulates into) an fp32 matrix."""
    if not _lib.use_cuda_kernels(a):
        r = (a.float() @ b.float().t()) * alpha
        if add is not None:
            r = r + add.float()
        if out_fp32:
            if out is not None:
                out.copy_(out + r if accumulate else r)
                return out
            return r
        r = r.to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, b = _check2d(a), _check2d(b)
    M, K = a.shape
    N = b.shape[0]
    splits = _skinny_splits(M, N, K) if not out_fp32 and SPLIT_K_SKINNY else 1
    if splits > 1:
        return _gemm_nt_split_k(a, b, out, add, alpha, splits)
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else a.dtype, device=a.device)
    epi = EPI_F32 if out_fp32 else (EPI_ADDC if add is not None else EPI_STORE)
    _raw(a, M, K, a.stride(0), 0, b, N, K, b.stride(0), 0, out, out.stride(0), add, add.stride(0) if add is not None else 0,
         None, 0, M, N, K, alpha=alpha, beta=int(accumulate), epilogue=epi, max_ctas=max_ctas)
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
            add: Optional[torch.Tensor] = None, alpha: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
    """a[M,K] @ b[K,N] (+ add)."""
    if not _lib.use_cuda_kernels(a):
        r = (a.float() @ b.float()) * alpha
        if add is not None:
            r = r + add.float()
        r = r.to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, b = _check2d(a), _check2d(b)
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    _raw(a, M, K, a.stride(0), 0, b, K, N, b.stride(0), 1, out, out.stride(0), add, add.stride(0) if add is not None else 0,
         None, 0, M, N, K, alpha=alpha, epilogue=EPI_ADDC if add is not None else EPI_STORE, max_ctas=max_ctas)
    return out


def _tn_splits(M: int, N: int, K: int, clusters: int = 74) -> int:
    """Reduction slices for a weight-gradient product whose 256 x 256 tiles fill the CTA pairs badly (e.g. 80 tiles on 74 pairs run
    two waves at 0.54 utilisation).  Modelled time = waves / slices + the fold of the fp32 partials; returns the best slice count
    (1 = do not split).  Only long reductions are worth it."""
    if M < 256 or K < 8192 or os.environ.get("ATS_WGRAD_SPLIT_K", "1") != "1":
        return 1
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if tiles >= 4 * clusters:
        return 1
    wave_us = 256 * 256 * K * 2 / 18.9e6   # one wave of full tiles at the sustained rate of a CTA pair
    best, best_t = 1, -(-tiles // clusters) * wave_us
    for s in (2, 3, 4):
        if K % (64 * s) or K // s < 2048:
            continue
        fold_us = ((2 * s * 4 + 4) * M * N) / 6.5e6
        t = -(-(tiles * s) // clusters) * wave_us / s + fold_us
        if t < 0.93 * best_t:
            best, best_t = s, t
    return best


class ScatterTarget:
    """Destination of a weight-gradient product whose rows are owned by different ranks (ZeRO-3 row shards): ``table`` is a
    device int64 tensor with the address of every owner's fp32 gradient rows, ``rows`` the number of rows per owner.  Passed
    as ``out`` to :func:`gemm_tn`, which then adds its result into the owners' buffers from the GEMM epilogue (reduce-scatter
    fused into the product; always accumulating -- the owners zero their shards once per optimiser step)."""

    def __init__(self, table: torch.Tensor, rows: int, shape):
        self.table, self.rows, self.shape = table, rows, tuple(shape)

    def view(self, *shape):
        return self


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
            alpha: float = 1.0, out_fp32: bool = False, max_ctas: int = 0) -> torch.Tensor:
    """a[K,M]^T @ b[K,N]; ``accumulate`` adds into ``out``."""
    if isinstance(out, ScatterTarget):
        a, b = _check2d(a), _check2d(b)
        K, M = a.shape
        N = b.shape[1]
        assert (M, N) == tuple(out.shape) and _lib.use_cuda_kernels(a)
        _raw(a, K, M, a.stride(0), 1, b, K, N, b.stride(0), 1, None, N, None, 0, None, 0, M, N, K, alpha=alpha, beta=1,
             epilogue=EPI_F32, max_ctas=max_ctas, d_table=out.table, scatter_rows=out.rows)
        return out
    if not _lib.use_cuda_kernels(a):
        r = (a.float().t() @ b.float()) * alpha
        if out is not None:
            if accumulate:
                r = r + out.float()
            out.copy_(r.to(out.dtype))
            return out
        return r if out_fp32 else r.to(a.dtype)
    a, b = _check2d(a), _check2d(b)
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else a.dtype, device=a.device)
        accumulate = False
    fp32 = out.dtype == torch.float32
    splits = _tn_splits(M, N, K) if (not fp32 and out.is_contiguous() and alpha == 1.0) else 1
    if splits > 1:
        # the reduction (tokens) is cut into slices that run as groups with fp32 partial outputs; one launch folds them (+ the
        # gradient accumulated so far) into the bf16 result
        kp = K // splits
        part = torch.empty(splits, M, N, dtype=torch.float32, device=a.device)
        _raw(a, K, M, a.stride(0), 1, b, K, N, b.stride(0), 1, part, N, None, 0, None, 0, M, N, kp, epilogue=EPI_F32, groups=splits,
             a_gs_k=kp, b_gs_k=kp, d_gs=M * N, max_ctas=max_ctas)
        _fold_partials(part, splits, M * N, 1, out, out if accumulate else None)
        return out
    epi = EPI_F32 if fp32 else (EPI_ADDC if accumulate else EPI_STORE)
    _raw(a, K, M, a.stride(0), 1, b, K, N, b.stride(0), 1, out, out.stride(0),
         out if (accumulate and not fp32) else None, out.stride(0), None, 0, M, N, K, alpha=alpha,
         beta=int(accumulate), epilogue=epi, max_ctas=max_ctas)
    return out


def gemm_nt_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None,
                   pre_act: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """h = silu(a @ Wg^T) * (a @ Wu^T) with ``w_gate_up = [Wg; Wu]`` of shape [2I, K].  ``pre_act`` ([M, 2I])
    receives the gate/up pre-activations when the backward pass needs them."""
    inter = w_gate_up.shape[0] // 2
    if not _lib.use_cuda_kernels(a):
        gu = (a.float() @ w_gate_up.float().t()).to(a.dtype)
        if pre_act is not None:
            pre_act.copy_(gu)
        g, u = gu.float().chunk(2, dim=-1)
        r = (torch.nn.functional.silu(g) * u).to(a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, w = _check2d(a), _check2d(w_gate_up)
    M, K = a.shape
    if out is None:
        out = torch.empty(M, inter, dtype=a.dtype, device=a.device)
    _raw(a, M, K, a.stride(0), 0, w, 2 * inter, K, w.stride(0), 0, out, out.stride(0), None, 0,
         pre_act, pre_act.stride(0) if pre_act is not None else 0, M, inter, K, epilogue=EPI_SWIGLU,
         up_offset=inter, max_ctas=max_ctas)
    return out


def swiglu_bwd_reference(pre: torch.Tensor, dh: torch.Tensor):
    """(dgu [.., 2I], h [.., I]) of h = silu(gate) * up from the saved pre-activations [.., 2I] and dh [.., I], in fp32."""
    g, u = pre.float().chunk(2, dim=-1)
    sg = torch.sigmoid(g)
    dhf = dh.float()
    return torch.cat([dhf * u * (sg + g * sg * (1 - sg)), dhf * g * sg], dim=-1).to(pre.dtype), (g * sg * u).to(pre.dtype)


def gemm_nn_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, pre: torch.Tensor):
    """dy [M, H] · w_down [H, I] = dh, pushed through the SwiGLU backward in the GEMM epilogue: -> (dgu [M, 2I], h [M, I])
    from the saved pre-activations ``pre`` [M, 2I]; dh is never written."""
    inter = w_down.shape[1]
    if not _lib.use_cuda_kernels(dy):
        return swiglu_bwd_reference(pre, (dy.float() @ w_down.float()).to(dy.dtype))
    dy, w = _check2d(dy), _check2d(w_down)
    M, H = dy.shape
    assert pre.is_contiguous() and pre.shape == (M, 2 * inter)
    dgu = torch.empty_like(pre)
    h = torch.empty(M, inter, dtype=pre.dtype, device=pre.device)
    _raw(dy, M, H, dy.stride(0), 0, w, H, inter, w.stride(0), 1, dgu, 2 * inter, h, inter, pre, 2 * inter, M, inter, H,
         epilogue=EPI_SWIGLU_BWD, up_offset=inter)
    return dgu, h


# ----------------------------------------------------------------------------------------------------------
# grouped (expert) products on the capacity layout
# ----------------------------------------------------------------------------------------------------------
def _ref_mask(counts: torch.Tensor, cap: int) -> torch.Tensor:
    return (torch.arange(cap, device=counts.device)[None, :] < counts[:, None].long())


def pack_kmajor(w: torch.Tensor) -> torch.Tensor:
    """[.., N, K] weight -> the same shape with the elements stored tile by tile ([N / 128][K / 64][128][64]): every
    128 x 64 box the GEMM loads is then 16 KB of consecutive memory, which lets a weight that is read once per step (decode)
    stream at close to HBM speed instead of touching 128 bytes per DRAM page.  Needs N % 128 == 0 and K % 64 == 0."""
    *lead, N, K = w.shape
    if N % 128 or K % 64:
        raise ValueError("pack_kmajor needs N % 128 == 0 and K % 64 == 0")
    t = w.reshape(-1, N // 128, 128, K // 64, 64).permute(0, 1, 3, 2, 4).contiguous()
    return t.view(*lead, N, K)


def unpack_kmajor(w: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_kmajor`."""
    *lead, N, K = w.shape
    t = w.reshape(-1, N // 128, K // 64, 128, 64).permute(0, 1, 3, 2, 4).contiguous()
    return t.view(*lead, N, K)


def grouped_nt(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, swiglu: bool = False,
               pre_act: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, b_div: int = 1,
               d_table: Optional[torch.Tensor] = None, packed: bool = False, k_split: int = 1, fold=None) -> torch.Tensor:
    """x[G,C,K] · w[E,N,K]^T -> [G,C,N] (or [G,C,N/2] through SwiGLU) for the first counts[g] rows of every
    group; group g uses weight g // b_div (G = E * b_div: several token blocks per expert, one per source rank).
    Rows beyond the padded count are left untouched.  ``d_table`` (int64 [G]) redirects the output of group g to
    an arbitrary base address (a buffer on a peer GPU).  ``packed``: ``w`` is stored as :func:`pack_kmajor` leaves it."""
    Gn, C, K = x.shape
    N = w.shape[1]
    if not _lib.use_cuda_kernels(x):
        if packed:
            w = unpack_kmajor(w)
        wx = w.repeat_interleave(b_div, dim=0) if b_div > 1 else w
        y = torch.einsum("eck,enk->ecn", x.float(), wx.float()).to(x.dtype)
        mask = _ref_mask(counts, C)[..., None]
        y = torch.where(mask, y, torch.zeros_like(y))
        if swiglu:
            if pre_act is not None:
                pre_act.copy_(y)
            g, u = y.float().chunk(2, dim=-1)
            y = (torch.nn.functional.silu(g) * u).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.is_contiguous() and w.is_contiguous() and C % 128 == 0
    n_out = N // 2 if swiglu else N
    if out is None and d_table is None:
        out = torch.empty(Gn, C, n_out, dtype=x.dtype, device=x.device)
    if k_split > 1:
        # few output tiles and a long reduction (the down projection of a decode step): the reduction is cut into k_split
        # slices, every (group, slice) pair is a work item with an fp32 partial block, and one small launch folds the slices
        assert not swiglu and d_table is None and pre_act is None and K % (64 * k_split) == 0 and out.is_contiguous()
        part = torch.empty(Gn * k_split, C, N, dtype=torch.float32, device=x.device)
        _raw(x, Gn * C, K, K, 0, w, w.shape[0] * N, K, K, 2 if packed else 0, part, N, None, 0, None, 0, C, N, K // k_split,
             epilogue=EPI_F32, groups=Gn * k_split, ragged=1, counts=counts, a_gs_mn=C, b_gs_mn=N, d_gs=C * N, b_div=b_div,
             k_split=k_split)
        # ``fold(part, k_split, n_inner, n_outer, out)`` replaces the plain fold (e.g. one that also signals the peers that will read out)
        (fold or _fold_partials)(part, k_split, C * N, Gn, out)
        return out
    _raw(x, Gn * C, K, K, 0, w, w.shape[0] * N, K, K, 2 if packed else 0, out, n_out, None, 0, pre_act,
         N if pre_act is not None else 0,
         C, n_out, K, epilogue=EPI_SWIGLU if swiglu else EPI_STORE, up_offset=N // 2 if swiglu else 0,
         groups=Gn, ragged=1, counts=counts, a_gs_mn=C, b_gs_mn=N, d_gs=C * n_out,
         aux_gs=C * N if pre_act is not None else 0, b_div=b_div, d_table=d_table)
    return out


def grouped_nn(dy: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, out: Optional[torch.Tensor] = None,
               b_div: int = 1, d_table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dy[G,C,N] · w[E,N,K] -> [G,C,K] (input gradient of grouped_nt)."""
    Gn, C, N = dy.shape
    K = w.shape[2]
    if not _lib.use_cuda_kernels(dy):
        wx = w.repeat_interleave(b_div, dim=0) if b_div > 1 else w
        y = torch.einsum("ecn,enk->eck", dy.float(), wx.float()).to(dy.dtype)
        y = torch.where(_ref_mask(counts, C)[..., None], y, torch.zeros_like(y))
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert dy.is_contiguous() and w.is_contiguous() and C % 128 == 0
    if out is None and d_table is None:
        out = torch.empty(Gn, C, K, dtype=dy.dtype, device=dy.device)
    _raw(dy, Gn * C, N, N, 0, w, w.shape[0] * N, K, K, 1, out, K, None, 0, None, 0, C, K, N,
         groups=Gn, ragged=1, counts=counts, a_gs_mn=C, b_gs_k=N, d_gs=C * K, b_div=b_div, d_table=d_table)
    return out


def grouped_nn_swiglu_bwd(dy: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, pre: torch.Tensor, b_div: int = 1):
    """Backward through ``h = silu(gate) * up`` fused into the product ``dh = dy · w``: dy [G,C,N], w [E,N,I], pre [G,C,2I]
    (saved gate / up pre-activations) -> (dgu [G,C,2I], h [G,C,I]); dh itself is never written.  Rows beyond the padded
    count of a group are left untouched.  With 16-byte accesses this epilogue (two reads and three stores per element,
    one row per thread) slowed the step by 2.5 %, because every access filled half an L2 sector and the requests crowded out the
    operand loads; with 32-byte loads and stores it is 1 % faster than GEMM + streaming element-wise kernel."""
    Gn, C, N = dy.shape
    inter = w.shape[2]
    if not _lib.use_cuda_kernels(dy):
        return swiglu_bwd_reference(pre, grouped_nn(dy, w, counts, b_div=b_div))
    assert dy.is_contiguous() and w.is_contiguous() and pre.is_contiguous() and C % 128 == 0
    dgu = torch.empty_like(pre)
    h = torch.empty(Gn, C, inter, dtype=pre.dtype, device=pre.device)
    _raw(dy, Gn * C, N, N, 0, w, w.shape[0] * N, inter, inter, 1, dgu, 2 * inter, h, inter, pre, 2 * inter, C, inter, N,
         epilogue=EPI_SWIGLU_BWD, up_offset=inter, groups=Gn, ragged=1, counts=counts, a_gs_mn=C, b_gs_k=N, d_gs=C * 2 * inter,
         c_gs=C * inter, aux_gs=C * 2 * inter, b_div=b_div)
    return dgu, h


def grouped_tn(dy: torch.Tensor, x: torch.Tensor, counts: torch.Tensor, out: Optional[torch.Tensor] = None,
               accumulate: bool = False, k_segs: int = 1) -> torch.Tensor:
    """dy[G,C,N]^T · x[G,C,K] -> [G / k_segs, N, K] (weight gradient of grouped_nt): expert e reduces over the used
    rows of its k_segs consecutive token blocks."""
    Gn, C, N = dy.shape
    K = x.shape[2]
    E = Gn // k_segs
    if not _lib.use_cuda_kernels(dy):
        mask = _ref_mask(counts, C)[..., None].float()
        r = torch.einsum("ecn,eck->enk", (dy.float() * mask).reshape(E, k_segs * C, N), (x.float() * mask).reshape(E, k_segs * C, K))
        if out is not None:
            if accumulate:
                r = r + out.float()
            out.copy_(r.to(out.dtype))
            return out
        return r.to(dy.dtype)
    assert dy.is_contiguous() and x.is_contiguous() and C % 128 == 0
    if out is None:
        out = torch.empty(E, N, K, dtype=dy.dtype, device=dy.device)
        accumulate = False
    _raw(dy, Gn * C, N, N, 1, x, Gn * C, K, K, 1, out, K, out if accumulate else None, K, None, 0, N, K, C,
         epilogue=EPI_ADDC if accumulate else EPI_STORE, groups=E, ragged=2, counts=counts,
         a_gs_k=k_segs * C, b_gs_k=k_segs * C, d_gs=N * K, c_gs=N * K, k_segs=k_segs, seg_stride=C)
    return out

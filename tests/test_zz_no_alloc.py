"""The allocation-free RMSNorm backward (``ats_rmsnorm_bwd_noalloc``, declared in ``csrc/ats_noalloc.h``).

It exists for callers that cannot allocate device memory where they run the backward pass (regions in which
``cudaMalloc`` is not allowed, latency-critical loops, embedders with a fixed memory budget): its scratch is an
array compiled into the library.  The test calls it through its exported C symbol and compares ``dx`` and ``dw``
with what the ordinary entry point (caller-supplied scratch) produces -- twice in a row, because the built-in
scratch still holds the first call's values when the second one starts.  The file name keeps it last in the
collection order.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from adaptivetrainingsystem_b200.ops import _lib as L
    lib = ctypes.CDLL(L.CUDA_LIB)
    vp, ci, cll, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.ats_rmsnorm_fwd.restype = ci
    lib.ats_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, cll, ci, cf, vp]
    lib.ats_rmsnorm_bwd.restype = ci
    lib.ats_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, vp, vp, ci, cll, ci, vp]
    lib.ats_rmsnorm_bwd_noalloc.restype = ci
    lib.ats_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, cll, ci, vp]
    lib.ats_rmsnorm_bwd_noalloc_limits.restype = None
    lib.ats_rmsnorm_bwd_noalloc_limits.argtypes = [ctypes.POINTER(ci), ctypes.POINTER(cll)]
    lib.ats_noalloc_error_string.restype = ctypes.c_char_p
    lib.ats_noalloc_error_string.argtypes = [ci]
    return lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(lib, rows, cols, seed, with_res=False, accumulate=False, f32_out=False):
    dev = "cuda"
    torch.manual_seed(seed)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.randn(rows, cols, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(cols, device=dev)).bfloat16()
    dy = torch.randn(rows, cols, device=dev).bfloat16()
    if with_res or accumulate or f32_out:
        return _case_variants(lib, x, w, dy, with_res, accumulate, f32_out, stream)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    assert lib.ats_rmsnorm_fwd(_p(x), None, _p(w), _p(y), None, _p(rstd), rows, cols, 1e-6, stream) == 0
    # ordinary entry point: scratch supplied by the caller
    nb = min(128, rows)
    scratch = torch.empty(nb, cols, dtype=torch.float32, device=dev)
    dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
    assert lib.ats_rmsnorm_bwd(_p(x), _p(w), _p(dy), _p(rstd), None, _p(dx_ref), _p(scratch), nb, _p(dw_ref), None, 0,
                               rows, cols, stream) == 0
    # allocation-free entry point: outputs allocated up front, nothing allocated by the call itself
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    # warm-up call: loads the kernels and resolves the scratch address, so that the measured call below does only its own work
    rc = lib.ats_rmsnorm_bwd_noalloc(_p(x), _p(w), _p(dy), _p(rstd), None, _p(dx), _p(dw), None, 0, rows, cols, stream)
    assert rc == 0, lib.ats_noalloc_error_string(rc)
    dx.zero_()
    dw.zero_()
    torch.cuda.synchronize()
    # free bytes as the driver reports them (cudaMemGetInfo): a cudaMalloc inside the library would show here, which
    # PyTorch's own allocator statistics could not see
    before = torch.cuda.mem_get_info()[0]
    before_torch = torch.cuda.memory_allocated()
    rc = lib.ats_rmsnorm_bwd_noalloc(_p(x), _p(w), _p(dy), _p(rstd), None, _p(dx), _p(dw), None, 0, rows, cols, stream)
    assert rc == 0, lib.ats_noalloc_error_string(rc)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == before and torch.cuda.memory_allocated() == before_torch
    scale_x = dx_ref.float().abs().max().item() + 1e-6
    scale_w = dw_ref.float().abs().max().item() + 1e-6
    assert (dx.float() - dx_ref.float()).abs().max().item() / scale_x < 2e-2
    assert (dw.float() - dw_ref.float()).abs().max().item() / scale_w < 2e-2
    # and both agree with the PyTorch fp32 definition
    xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    yf.backward(dy.float())
    assert (dx.float() - xf.grad).abs().max().item() / (xf.grad.abs().max().item() + 1e-6) < 2e-2
    assert (dw.float() - wf.grad).abs().max().item() / (wf.grad.abs().max().item() + 1e-6) < 3e-2


def _case_variants(lib, x, w, dy, with_res, accumulate, f32_out, stream):
    """Residual gradient input, accumulation into dw and the fp32 dw output: the allocation-free entry point against the
    ordinary one, output for output."""
    rows, cols = x.shape
    dev = x.device
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    assert lib.ats_rmsnorm_fwd(_p(x), None, _p(w), _p(y), None, _p(rstd), rows, cols, 1e-6, stream) == 0
    dres = torch.randn(rows, cols, device=dev).bfloat16() if with_res else None
    nb = min(128, rows)
    scratch = torch.empty(nb, cols, dtype=torch.float32, device=dev)
    seed_bf = (0.5 * torch.randn(cols, device=dev)).bfloat16()
    seed_f = 0.5 * torch.randn(cols, device=dev)
    outs = []
    for noalloc in (False, True):
        dx = torch.empty_like(x)
        dw_bf = seed_bf.clone() if not f32_out else None
        dw_f = seed_f.clone() if f32_out else None
        if noalloc:
            rc = lib.ats_rmsnorm_bwd_noalloc(_p(x), _p(w), _p(dy), _p(rstd), _p(dres), _p(dx), _p(dw_bf), _p(dw_f), int(accumulate),
                                             rows, cols, stream)
        else:
            rc = lib.ats_rmsnorm_bwd(_p(x), _p(w), _p(dy), _p(rstd), _p(dres), _p(dx), _p(scratch), nb, _p(dw_bf), _p(dw_f),
                                     int(accumulate), rows, cols, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        outs.append((dx.float(), (dw_f if f32_out else dw_bf).float()))
    (dx_ref, dw_ref), (dx, dw) = outs
    assert (dx - dx_ref).abs().max().item() / (dx_ref.abs().max().item() + 1e-6) < 2e-2
    assert (dw - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6) < 2e-2
    # fp32 PyTorch definition of the same quantities
    xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
    (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf).backward(dy.float())
    want_dx = xf.grad + (dres.float() if with_res else 0)
    want_dw = wf.grad + ((seed_f if f32_out else seed_bf.float()) if accumulate else 0)
    assert (dx - want_dx).abs().max().item() / (want_dx.abs().max().item() + 1e-6) < 2e-2
    assert (dw - want_dw).abs().max().item() / (want_dw.abs().max().item() + 1e-6) < 3e-2


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    lib = _lib()
    _case(lib, rows=777, cols=2048, seed=0)   # first call on the device resolves the scratch address
    _case(lib, rows=64, cols=4096, seed=1)    # second call reuses the scratch that still holds the first call's data


def test_noalloc_boundary_width_and_optional_arguments():
    lib = _lib()
    _case(lib, rows=300, cols=8192, seed=2)                       # the widest row the built-in scratch takes: all 4 MiB in use
    _case(lib, rows=130, cols=8192, seed=3, with_res=True)        # residual gradient added into dx
    _case(lib, rows=96, cols=1024, seed=4, accumulate=True)       # dw accumulated into the caller's bf16 buffer
    _case(lib, rows=200, cols=2048, seed=5, accumulate=True, f32_out=True, with_res=True)  # fp32 dw output


def test_noalloc_rejects_sizes_beyond_the_scratch():
    lib = _lib()
    max_cols, nbytes = ctypes.c_int(0), ctypes.c_longlong(0)
    lib.ats_rmsnorm_bwd_noalloc_limits(ctypes.byref(max_cols), ctypes.byref(nbytes))
    assert max_cols.value == 8192 and nbytes.value == 4 * 1024 * 1024
    t = torch.zeros(8, device="cuda")
    rc = lib.ats_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), None, _p(t), _p(t), None, 0, 4, max_cols.value + 8, None)
    assert rc == 2001
    assert b"too large" in lib.ats_noalloc_error_string(rc)
    rc = lib.ats_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), None, _p(t), _p(t), None, 0, 2 ** 31, 8, None)
    assert rc == 1003  # more rows than the kernels' 32-bit row index can address: refused, nothing launched

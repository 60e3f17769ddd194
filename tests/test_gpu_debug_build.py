"""The bounds-checking build (``-DATS_DEBUG``, ``libats_b200_debug.so``): the kernels range-check every index that comes from data
and, on a violation, record {kernel, block, value} and SKIP the access.  Nothing traps or faults: a bad expert id is caught before
it is used as an address, the process goes on and the host raises ``KernelError`` at its next status check.

Runs in a child process so that this library, not the release one, backs the package's operators."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent('''
    import ctypes, os, sys, torch
    sys.path.insert(0, os.environ["ATS_REPO"])
    from adaptivetrainingsystem_b200 import ops
    from adaptivetrainingsystem_b200.ops import _lib, moe as M, gemm as G
    assert _lib.DEBUG_BUILD and _lib.cuda_lib()._name.endswith("libats_b200_debug.so")
    dev = "cuda"
    torch.manual_seed(0)
    # 1. ragged, odd-sized work through the checked kernels: nothing may be reported
    T, H, E, k = 77, 256, 4, 2
    x = torch.randn(T, H, device=dev).bfloat16()
    w1 = (torch.randn(E, 512, H, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, 256, device=dev) * 0.05).bfloat16()
    idx = torch.randint(0, E, (T, k), device=dev, dtype=torch.int32)
    idx[:, 1] = (idx[:, 0] + 1) % E
    wts = torch.rand(T, k, device=dev)
    out, totals = M.moe_ffn(x, idx, wts, w1, w2, 128)
    ref = M.moe_ffn_reference(x.float(), idx, wts, w1.float(), w2.float(), 128)
    assert (out.float() - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-3
    gate = (torch.randn(E, H, device=dev) * 0.1).bfloat16()
    with torch.no_grad():
        served, _ = M.moe_ffn_serving(x[:33].contiguous(), gate, k, 1.0, w1, w2)
    counts = torch.tensor([100, 0, 128, 17], dtype=torch.int32, device=dev)
    G.grouped_nt(torch.randn(E, 128, H, device=dev).bfloat16(), w1, counts, swiglu=True)
    qkv = torch.randn(3, 1, (8 + 4) * 64, device=dev).bfloat16()
    kc, vc = torch.zeros(3, 300, 2, 64, device=dev).bfloat16(), torch.zeros(3, 300, 2, 64, device=dev).bfloat16()
    ops.decode_attention(qkv, kc, vc, torch.tensor([0, 17, 299], dtype=torch.int32, device=dev), 8, 2, 64)
    torch.cuda.synchronize()
    ops.check_status()
    print("CLEAN_OK")
    # 2. an expert id outside the layer (what a corrupted routing table would look like): caught before it becomes an address
    bad = idx.clone()
    bad[5, 0] = E + 3
    slot_pos = torch.zeros(T * k, dtype=torch.int32, device=dev)
    cnt = torch.zeros(E, dtype=torch.int32, device=dev)
    buf = torch.zeros(E, 128, H, device=dev).bfloat16()
    M.dispatch(x, bad, slot_pos, cnt, E, 128, out=buf)
    torch.cuda.synchronize()
    try:
        ops.check_status()
        print("NOT_CAUGHT")
    except ops.KernelError as e:
        print("CAUGHT", e)
    # 3. the context is intact and the report is cleared
    y = ops.rms_norm(x, torch.ones(H, device=dev).bfloat16(), 1e-6)
    torch.cuda.synchronize()
    ops.check_status()
    print("AFTER_OK", float(y.float().abs().mean()) > 0)
''')


def test_debug_build_checks_indices_and_skips_bad_accesses():
    from adaptivetrainingsystem_b200.ops import _lib
    if not os.path.exists(_lib.DEBUG_LIB):
        _lib.build_debug()
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ATS_DEBUG_BUILD="1", ATS_REPO=repo)
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "CLEAN_OK" in out and "AFTER_OK True" in out, out[-3000:]
    assert "CAUGHT" in out and "dispatch_rows" in out and "NOT_CAUGHT" not in out, out[-3000:]

"""tcgen05 GEMM against a PyTorch fp32 reference of the same product."""
import pytest
import torch

from adaptivetrainingsystem_b200 import ops
from adaptivetrainingsystem_b200.ops import gemm as G

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"max err {err} vs scale {denom}"
    if ref.dim() >= 2 and ref.shape[-1] >= 8:
        # every row against its own norm: a wrong row of small magnitude cannot hide behind the tensor's largest element
        g2, r2 = got.reshape(-1, ref.shape[-1]), ref.reshape(-1, ref.shape[-1])
        rn = r2.norm(dim=-1)
        rel = (g2 - r2).norm(dim=-1) / torch.maximum(rn, 1e-3 * rn.mean() + 1e-12)
        worst = int(rel.argmax())
        assert rel[worst].item() < 2 * tol, f"row {worst} differs by {rel[worst].item():.3e} of its norm"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (200, 264, 136), (1024, 2560, 2048), (64, 8, 72)])
def test_gemm_nt(M, N, K):
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    _close(G.gemm_nt(a, b), a.float() @ b.float().t())


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (200, 264, 136), (1024, 2048, 2560)])
def test_gemm_nn(M, N, K):
    torch.manual_seed(1)
    a, b = _rand(M, K), _rand(K, N)
    _close(G.gemm_nn(a, b), a.float() @ b.float())


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (264, 200, 136), (2560, 2048, 1024)])
def test_gemm_tn(M, N, K):
    torch.manual_seed(2)
    a, b = _rand(K, M), _rand(K, N)
    _close(G.gemm_tn(a, b), a.float().t() @ b.float())


def test_gemm_epilogues():
    torch.manual_seed(3)
    M, N, K = 256, 512, 256
    a, b, c = _rand(M, K), _rand(N, K), _rand(M, N)
    ref = a.float() @ b.float().t()
    _close(G.gemm_nt(a, b, add=c), ref + c.float())
    out32 = torch.full((M, N), 1.0, device=DEV)
    G.gemm_nt(a, b, out=out32, out_fp32=True, accumulate=True)
    _close(out32, ref + 1.0, tol=1e-2)
    acc = _rand(K, N)
    x, dy = _rand(M, K), _rand(M, N)
    expect = acc.float() + x.float().t() @ dy.float()
    G.gemm_tn(x, dy, out=acc, accumulate=True)
    _close(acc, expect)


def test_gemm_swiglu_epilogue():
    torch.manual_seed(4)
    M, K, I = 256, 256, 384
    a, w = _rand(M, K), _rand(2 * I, K, scale=0.1)
    pre = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    h = G.gemm_nt_swiglu(a, w, pre_act=pre)
    gu = a.float() @ w.float().t()
    _close(pre, gu)
    g, u = gu.chunk(2, dim=-1)
    _close(h, torch.nn.functional.silu(g) * u, tol=3e-2)


def test_grouped_products():
    torch.manual_seed(5)
    E, C, K, N = 4, 256, 128, 256
    counts = torch.tensor([256, 100, 0, 129], dtype=torch.int32, device=DEV)
    x = _rand(E, C, K)
    dy = _rand(E, C, N)
    mask = (torch.arange(C, device=DEV)[None, :] < counts[:, None]).unsqueeze(-1)
    x = x * mask
    dy = dy * mask
    w = _rand(E, N, K, scale=0.2)
    y = G.grouped_nt(x, w, counts)
    ref = torch.einsum("eck,enk->ecn", x.float(), w.float())
    for e in range(E):
        n = int(counts[e])
        if n:
            _close(y[e, :n], ref[e, :n])
    dx = G.grouped_nn(dy, w, counts)
    refdx = torch.einsum("ecn,enk->eck", dy.float(), w.float())
    for e in range(E):
        n = int(counts[e])
        if n:
            _close(dx[e, :n], refdx[e, :n])
    dw = G.grouped_tn(dy, x, counts)
    refdw = torch.einsum("ecn,eck->enk", dy.float(), x.float())
    _close(dw, refdw)
    assert dw[2].abs().max().item() == 0.0  # an expert without tokens gets a zero gradient
    pre = torch.zeros(E, C, N, dtype=torch.bfloat16, device=DEV)
    h = G.grouped_nt(x, w, counts, swiglu=True, pre_act=pre)
    g, u = ref.chunk(2, dim=-1)
    refh = torch.nn.functional.silu(g) * u
    for e in range(E):
        n = int(counts[e])
        if n:
            _close(h[e, :n], refh[e, :n], tol=3e-2)
            _close(pre[e, :n], ref[e, :n])


def test_linear_autograd_matches_reference():
    torch.manual_seed(6)
    x = _rand(4, 64, 256).requires_grad_()
    w = _rand(512, 256, scale=0.05).requires_grad_()
    r = _rand(4, 64, 512).requires_grad_()
    y = ops.linear(x, w, residual=r)
    gy = _rand(4, 64, 512)
    y.backward(gy)
    xf, wf, rf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), r.detach().float().requires_grad_()
    yf = torch.nn.functional.linear(xf, wf) + rf
    yf.backward(gy.float())
    _close(y, yf)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad)
    _close(r.grad, rf.grad)


def test_grouped_expert_parallel_layout():
    """Several token blocks per expert (one per source rank), K-segmented weight gradient, output pointer table."""
    torch.manual_seed(7)
    E, W, C, K, N = 2, 3, 128, 128, 256
    Gn = E * W
    counts = torch.tensor([128, 5, 0, 77, 128, 1], dtype=torch.int32, device=DEV)
    mask = (torch.arange(C, device=DEV)[None, :] < counts[:, None]).unsqueeze(-1)
    x = _rand(Gn, C, K) * mask
    dy = _rand(Gn, C, N) * mask
    w = _rand(E, N, K, scale=0.2)
    wx = w.repeat_interleave(W, dim=0)
    y = G.grouped_nt(x, w, counts, b_div=W)
    ref = torch.einsum("eck,enk->ecn", x.float(), wx.float())
    for g in range(Gn):
        n = int(counts[g])
        if n:
            _close(y[g, :n], ref[g, :n])
    dx = G.grouped_nn(dy, w, counts, b_div=W)
    refdx = torch.einsum("ecn,enk->eck", dy.float(), wx.float())
    for g in range(Gn):
        n = int(counts[g])
        if n:
            _close(dx[g, :n], refdx[g, :n])
    dw = G.grouped_tn(dy, x, counts, k_segs=W)
    refdw = torch.einsum("ecn,eck->enk", dy.float().reshape(E, W * C, N), x.float().reshape(E, W * C, K))
    _close(dw, refdw)
    # pointer table: scatter the groups' outputs into a permuted buffer
    target = torch.zeros(Gn, C, N, dtype=torch.bfloat16, device=DEV)
    perm = [3, 0, 5, 1, 4, 2]
    table = torch.tensor([target[perm[g]].data_ptr() for g in range(Gn)], dtype=torch.int64, device=DEV)
    G.grouped_nt(x, w, counts, b_div=W, d_table=table)
    for g in range(Gn):
        n = int(counts[g])
        if n:
            _close(target[perm[g], :n], ref[g, :n])


def test_gemm_swiglu_backward_epilogue_matches_separate_kernel():
    """dh = dy · w2 fused with the SwiGLU backward against the unfused sequence (GEMM, then the element-wise kernel)."""
    import ctypes  # noqa: F401
    from adaptivetrainingsystem_b200.ops import functional as Fn
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(4)
    M, H, I = 900, 512, 1408
    dy = (torch.randn(M, H, device="cuda") * 0.5).bfloat16()
    w2 = (torch.randn(H, I, device="cuda") * 0.05).bfloat16()
    pre = torch.randn(M, 2 * I, device="cuda").bfloat16()
    dgu, h = G.gemm_nn_swiglu_bwd(dy, w2, pre)
    dh = G.gemm_nn(dy, w2)
    dgu_ref = torch.empty_like(pre)
    h_ref = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    Fn._CK(Fn._L().ats_swiglu_bwd(Fn._P(pre), Fn._P(dh), Fn._P(dgu_ref), Fn._P(h_ref), M, I, Fn._S(pre.device)), "swiglu_bwd")
    assert torch.equal(dgu, dgu_ref) and torch.equal(h, h_ref)
    # grouped form on the capacity layout
    E, C = 3, 256
    counts = torch.tensor([200, 0, 130], dtype=torch.int32, device="cuda")
    dye = (torch.randn(E, C, H, device="cuda") * 0.5).bfloat16()
    for e, c in enumerate(counts.tolist()):
        dye[e, c:] = 0
    w2e = (torch.randn(E, H, I, device="cuda") * 0.05).bfloat16()
    pre_e = torch.randn(E, C, 2 * I, device="cuda").bfloat16()
    dgu_e, h_e = G.grouped_nn_swiglu_bwd(dye, w2e, counts, pre_e)
    for e, c in enumerate(counts.tolist()):
        if c == 0:
            continue
        d1, h1 = G.gemm_nn_swiglu_bwd(dye[e, :c].contiguous(), w2e[e], pre_e[e, :c].contiguous())
        assert torch.equal(dgu_e[e, :c], d1) and torch.equal(h_e[e, :c], h1), e


def test_skinny_gemm_splits_the_reduction():
    """Decode-shaped products (few output tiles) run as split-K groups with fp32 partials: same result as the fp32 reference."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(5)
    for (M, N, K) in [(64, 4096, 14336), (64, 6144, 4096), (17, 1024, 2048), (128, 512, 8192)]:
        assert G._skinny_splits(M, N, K) > 1, (M, N, K)
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        res = torch.randn(M, N, device="cuda").bfloat16()
        ref = a.float() @ b.float().t()
        out = G.gemm_nt(a, b)
        assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3, (M, N, K)
        out2 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        G.gemm_nt(a, b, out=out2, add=res)
        ref2 = ref + res.float()
        assert (out2.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item() + 1e-3, (M, N, K)
    assert G._skinny_splits(64, 28672, 4096) == 1 and G._skinny_splits(4096, 4096, 4096) == 1


def test_grouped_gemm_with_tile_packed_weights():
    """Expert weights stored tile by tile (serving layout) give bit-identical products, on single CTAs (C = 128) and CTA pairs."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(6)
    E, N, K = 3, 512, 384
    w = (torch.randn(E, N, K, device="cuda") * 0.05).bfloat16()
    wp = G.pack_kmajor(w)
    assert torch.equal(G.unpack_kmajor(wp), w)
    for C, cnt in ((128, [100, 0, 128]), (512, [300, 512, 17])):
        x = torch.randn(E, C, K, device="cuda").bfloat16()
        counts = torch.tensor(cnt, dtype=torch.int32, device="cuda")
        for swiglu in (False, True):
            pre_a = torch.zeros(E, C, N, device="cuda", dtype=torch.bfloat16) if swiglu else None
            pre_b = torch.zeros(E, C, N, device="cuda", dtype=torch.bfloat16) if swiglu else None
            a = G.grouped_nt(x, w, counts, swiglu=swiglu, pre_act=pre_a, out=torch.zeros(E, C, N // 2 if swiglu else N, device="cuda", dtype=torch.bfloat16))
            b = G.grouped_nt(x, wp, counts, swiglu=swiglu, pre_act=pre_b, out=torch.zeros(E, C, N // 2 if swiglu else N, device="cuda", dtype=torch.bfloat16),
                             packed=True)
            assert torch.equal(a, b), (C, swiglu)
            if swiglu:
                assert torch.equal(pre_a, pre_b)
    # two token blocks per weight (expert parallel receive layout)
    x = torch.randn(2 * E, 128, K, device="cuda").bfloat16()
    counts = torch.tensor([128, 3, 0, 64, 128, 1], dtype=torch.int32, device="cuda")
    a = G.grouped_nt(x, w, counts, b_div=2, out=torch.zeros(2 * E, 128, N, device="cuda", dtype=torch.bfloat16))
    b = G.grouped_nt(x, wp, counts, b_div=2, out=torch.zeros(2 * E, 128, N, device="cuda", dtype=torch.bfloat16), packed=True)
    assert torch.equal(a, b)


def test_grouped_gemm_with_reduction_slices():
    """Grouped products whose reduction is cut into slices (decode-sized down projection: few output tiles, long K): every
    (group, slice) pair writes an fp32 partial, one launch folds them.  Plain and tile-packed weights, one and several token
    blocks per weight, ragged row counts; against the fp32 product row by row (error relative to each row's norm)."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(8)
    E, N, K = 3, 512, 2048
    w = (torch.randn(E, N, K, device="cuda") * 0.03).bfloat16()
    wp = G.pack_kmajor(w)
    for C, cnt, b_div in ((128, [128, 128, 128], 1), (128, [100, 0, 128], 1), (256, [256, 130, 256, 1, 256, 256], 2)):
        Gn = E * b_div
        x = torch.randn(Gn, C, K, device="cuda").bfloat16()
        counts = torch.tensor(cnt, dtype=torch.int32, device="cuda")
        wx = w.repeat_interleave(b_div, dim=0)
        ref = torch.einsum("gck,gnk->gcn", x.float(), wx.float())
        for S in (2, 4, 8):
            for packed in (False, True):
                out = torch.zeros(Gn, C, N, device="cuda", dtype=torch.bfloat16)
                G.grouped_nt(x, wp if packed else w, counts, out=out, b_div=b_div, packed=packed, k_split=S)
                torch.cuda.synchronize()
                for g in range(Gn):
                    n = cnt[g]
                    if n == 0:
                        continue
                    err = (out[g, :n].float() - ref[g, :n]).norm(dim=-1) / (ref[g, :n].norm(dim=-1) + 1e-6)
                    assert err.max().item() < 1e-2, (C, cnt, b_div, S, packed, g, err.max().item())
    ops.check_status()


def test_weight_gradient_product_with_reduction_slices():
    """tn products whose tiles fill the CTA pairs badly split the token dimension (fp32 partials + fold): store and accumulate."""
    from adaptivetrainingsystem_b200.ops import gemm as G
    torch.manual_seed(9)
    M, N, K = 2560, 2048, 16384
    assert G._tn_splits(M, N, K) > 1 and G._tn_splits(2048, 2048, K) == 1
    dy = (torch.randn(K, M, device="cuda") * 0.1).bfloat16()
    x = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    ref = dy.float().t() @ x.float()
    out = G.gemm_tn(dy, x)
    err = (out.float() - ref).norm(dim=-1) / (ref.norm(dim=-1) + 1e-6)
    assert err.max().item() < 1e-2
    acc0 = (torch.randn(M, N, device="cuda") * 2).bfloat16()
    acc = acc0.clone()
    G.gemm_tn(dy, x, out=acc, accumulate=True)
    ref2 = ref + acc0.float()
    err = (acc.float() - ref2).norm(dim=-1) / (ref2.norm(dim=-1) + 1e-6)
    assert err.max().item() < 1e-2
    ops.check_status()

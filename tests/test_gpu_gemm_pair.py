"""CTA-pair (tcgen05 cta_group::2, 256-row tiles) variant of the GEMM against an fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _native():
    from speech_b200.ops import native

    native.load()
    return native


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 512), (3760, 1024, 1024), (1000, 520, 328), (129, 300, 200)])
def test_pair_gemm_layouts(a_mn, b_mn, M, N, K):
    nat = _native()
    torch.manual_seed(0)
    Mp, Np, Kp = (M + 7) // 8 * 8, (N + 7) // 8 * 8, (K + 7) // 8 * 8
    a = torch.randn((K, Mp) if a_mn else (M, Kp), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, Np) if b_mn else (N, Kp), device="cuda", dtype=torch.bfloat16)
    av = a[:, :M] if a_mn else a[:, :K]
    bv = b[:, :N] if b_mn else b[:, :K]
    out = torch.full((M, Np), float("nan"), device="cuda", dtype=torch.float32)
    nat.gemm(a, b, out, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, lda=a.stride(0), ldb=b.stride(0), ldd=Np, tile_n=256, pair=1)
    nat.check_status()
    A = av.float().t() if a_mn else av.float()
    B = bv.float().t() if b_mn else bv.float()
    ref = A @ B.t()
    err = (out[:, :N] - ref).abs().max().item()
    assert err <= 2e-2 * (K ** 0.5), f"max abs err {err}"
    assert torch.isnan(out[:, N:]).all()


def test_pair_gemm_epilogue_persistent_tiles_and_split_k():
    nat = _native()
    torch.manual_seed(1)
    M, N, K = 3760, 4096, 1024          # 15 x 16 = 240 pair tiles over 74 pairs: every pair runs several tiles (both accumulators)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty_like(y)
    nat.gemm(x, w, y, M=M, N=N, K=K, bias=bias, act="swish", residual=res, out_pre=pre, alpha=0.5, tile_n=256, pair=1)
    nat.check_status()
    z = x.float() @ w.float().t() + bias
    ref = 0.5 * torch.nn.functional.silu(z) + res.float()
    assert (pre.float() - z).abs().max().item() < 0.1 and (y.float() - ref).abs().max().item() < 0.1
    # weight-gradient form with K slices
    dz = torch.randn(M, 1024, device="cuda", dtype=torch.bfloat16)
    g0 = torch.randn(1024, K, device="cuda")
    g = g0.clone()
    nat.gemm(dz, x, g, M=1024, N=K, K=M, a_mn=True, b_mn=True, lda=1024, ldb=K, ldd=K, beta=1.0, tile_n=256, pair=1)
    nat.check_status()
    ref = g0 + dz.float().t() @ x.float()
    assert (g - ref).abs().max().item() <= 2e-2 * (M ** 0.5)

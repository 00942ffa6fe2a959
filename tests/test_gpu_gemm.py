"""tcgen05 GEMM against an fp32 PyTorch reference: all four operand layouts, tails, batching, fused epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _native():
    from speech_b200.ops import native

    native.load()
    return native


def _ref(a, b, a_mn, b_mn):
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    return A @ B.transpose(-1, -2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 512), (250, 1032, 640), (3750, 1024, 1024), (77, 130, 200)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    nat = _native()
    torch.manual_seed(0)
    Mp, Np, Kp = (M + 7) // 8 * 8, (N + 7) // 8 * 8, (K + 7) // 8 * 8
    a = torch.randn((K, Mp) if a_mn else (M, Kp), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, Np) if b_mn else (N, Kp), device="cuda", dtype=torch.bfloat16)
    av = a[:, :M] if a_mn else a[:, :K]
    bv = b[:, :N] if b_mn else b[:, :K]
    out = torch.full((M, Np), float("nan"), device="cuda", dtype=torch.float32)
    nat.gemm(a, b, out, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, lda=a.stride(0), ldb=b.stride(0), ldd=Np)
    nat.check_status()
    ref = _ref(av, bv, a_mn, b_mn)
    # bf16 operands are exact in fp32 and the accumulation is fp32: only the summation order differs from the reference
    err = (out[:, :N] - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 1e-3, f"max relative err {err}"
    assert torch.isnan(out[:, N:]).all()


def test_gemm_epilogue_bias_act_residual_pre():
    nat = _native()
    torch.manual_seed(1)
    M, N, K = 300, 512, 256
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.float32)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    nat.gemm(x, w, out, M=M, N=N, K=K, bias=bias, act="swish", residual=res, out_pre=pre, alpha=0.5)
    nat.check_status()
    z = (x.float() @ w.float().t()) + bias
    ref = 0.5 * torch.nn.functional.silu(z) + res.float()
    assert (pre.float() - z).abs().max() < 0.05
    assert (out.float() - ref).abs().max() < 0.06


def test_gemm_batched_strided():
    nat = _native()
    torch.manual_seed(2)
    B, H, T, dk = 3, 4, 100, 64
    q = torch.randn(B, T, H, dk, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, T, H, dk, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(B, H, T, T, device="cuda", dtype=torch.float32)
    Tp = T
    nat.gemm(q, k, out, M=T, N=T, K=dk, lda=H * dk, ldb=H * dk, ldd=T, batch=(H, B), a_bs=(dk, T * H * dk),
             b_bs=(dk, T * H * dk), d_bs=(T * T, H * T * T))
    nat.check_status()
    ref = torch.einsum("bthd,bshd->bhts", q.float(), k.float())
    assert (out - ref).abs().max() < 0.2


def test_gemm_beta_accumulate_and_dact():
    nat = _native()
    torch.manual_seed(3)
    M, N, K = 256, 256, 128
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.ones(M, N, device="cuda", dtype=torch.float32)
    nat.gemm(a, b, out, M=M, N=N, K=K, beta=1.0)
    ref = a.float() @ b.float().t() + 1.0
    assert (out - ref).abs().max() < 0.3
    aux = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    o2 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    nat.gemm(a, b, o2, M=M, N=N, K=K, aux=aux, dact="relu")
    ref2 = (a.float() @ b.float().t()) * (aux.float() > 0)
    assert (o2.float() - ref2).abs().max() < 0.3
    nat.check_status()


def test_linear_layernorm_autograd_matches_reference():
    from speech_b200 import ops
    from speech_b200.ops import reference

    torch.manual_seed(4)
    M, K, N = 200, 256, 384
    x = torch.randn(2, M // 2, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(N, K, device="cuda") * 0.05)
    b = torch.nn.Parameter(torch.randn(N, device="cuda") * 0.1)
    g = torch.nn.Parameter(torch.rand(K, device="cuda") + 0.5)
    be = torch.nn.Parameter(torch.randn(K, device="cuda") * 0.1)
    y = ops.linear(ops.layer_norm(x, g, be), w, b, act="swish", alpha=0.5)
    y.float().square().mean().backward()
    got = [t.grad.float().clone() for t in (x, w, b, g, be)]
    for t in (x, w, b, g, be):
        t.grad = None
    xr = x.detach().float().requires_grad_(True)
    yr = reference.linear(reference.layer_norm(xr, g, be), w, b, act="swish", alpha=0.5)
    yr.square().mean().backward()
    ref = [xr.grad, w.grad, b.grad, g.grad, be.grad]
    assert (y.float() - yr).abs().max() < 0.05
    for name, a_, r_ in zip("x w b gamma beta".split(), got, ref):
        denom = r_.abs().max().clamp(min=1e-6)
        assert ((a_ - r_).abs().max() / denom) < 0.05, name
    ops.native.check_status()


def test_fused_adamw_matches_torch():
    from speech_b200.core.optim.fused_adamw import FusedAdamW

    torch.manual_seed(5)
    ps = [torch.nn.Parameter(torch.randn(257, 33, device="cuda")), torch.nn.Parameter(torch.randn(1000, device="cuda"))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    opt = FusedAdamW(ps, lr=1e-2, betas=(0.9, 0.98), weight_decay=0.01, max_grad_norm=1.0)
    topt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.98), weight_decay=0.01)
    for _ in range(3):
        gs = [torch.randn_like(p) for p in ps]
        opt.zero_grad()
        for p, r, g in zip(ps, ref, gs):
            p.grad.copy_(g)
            r.grad = g.clone()
        torch.nn.utils.clip_grad_norm_(ref, 1.0)
        opt.step()
        topt.step()
    for p, r in zip(ps, ref):
        assert (p - r).abs().max() < 1e-5
        assert (p._lowp.float() - r).abs().max() < 2e-2


def test_linear_fused_dropout_mask_is_consistent_between_forward_and_backward():
    """Dropout lives in the GEMM epilogue as a hash of (seed, index); backward must rebuild exactly the same mask.
    The bias keeps every pre-activation far from zero, so the mask can be read off the output exactly."""
    from speech_b200 import ops

    torch.manual_seed(0)
    dev = torch.device("cuda")
    M, K, N, p = 300, 256, 512, 0.3
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(N, K, device=dev) * 0.02)
    b = torch.nn.Parameter(torch.full((N,), 6.0, device=dev))
    y = ops.linear(x, w, b, act="swish", alpha=0.5, dropout_p=p)
    z = torch.nn.functional.linear(x.float(), w.float().to(torch.bfloat16).float(), b.float())
    assert z.min().item() > 3.0
    keep = (y != 0).float()
    assert abs(keep.mean().item() - (1 - p)) < 0.02
    want = keep * 0.5 * torch.nn.functional.silu(z) / (1 - p)
    assert ((y.float() - want).abs() / want.abs().clamp(min=1.0)).max().item() < 0.02
    dy = torch.randn_like(y)
    y.backward(dy)
    s = torch.sigmoid(z)
    dz = 0.5 * keep / (1 - p) * dy.float() * (s + z * s * (1 - s))
    dx_ref, dw_ref, db_ref = dz @ w.float(), dz.t() @ x.float(), dz.sum(0)
    for got, ref in ((x.grad, dx_ref), (w.grad, dw_ref), (b.grad, db_ref)):
        assert (got.float() - ref).abs().max().item() / ref.abs().max().item() < 0.03
    # a second call draws a different mask; without dropout the op is deterministic
    y2 = ops.linear(x.detach(), w, b, act="swish", alpha=0.5, dropout_p=p)
    assert ((y2 != 0) != (y != 0)).float().mean().item() > 0.2
    assert torch.equal(ops.linear(x.detach(), w, b, act="swish"), ops.linear(x.detach(), w, b, act="swish"))
    # output-side dropout with a residual (the pattern at the end of every conformer sub-module)
    res = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    x2 = x.detach().clone().requires_grad_(True)
    y4 = ops.linear(x2, w, b, residual=res, dropout_p=p)
    keep4 = ((y4.float() - res.float()).abs() > 0.5).float()           # |z| / (1-p) > 4 wherever it was kept
    assert abs(keep4.mean().item() - (1 - p)) < 0.02
    y4.backward(dy)
    ref4 = (keep4 / (1 - p) * dy.float()) @ w.float()
    assert (x2.grad.float() - ref4).abs().max().item() / ref4.abs().max().item() < 0.03


@pytest.mark.parametrize("ksplit", [0, 3, -1])
@pytest.mark.parametrize("M,N,K", [(1024, 1024, 3760), (2048, 1024, 3752), (1000, 520, 1800)])
def test_gemm_split_k_weight_gradient(ksplit, M, N, K):
    """D(fp32) += A^T B with both operands stored [K, *] (the weight-gradient form): K slices add into D with reductions."""
    nat = _native()
    torch.manual_seed(1)
    a = torch.randn((K, M), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N), device="cuda", dtype=torch.bfloat16)
    d0 = torch.randn((M, N), device="cuda", dtype=torch.float32)
    out = d0.clone()
    nat.gemm(a, b, out, M=M, N=N, K=K, a_mn=True, b_mn=True, lda=M, ldb=N, ldd=N, beta=1.0, alpha=0.5, ksplit=ksplit)
    nat.check_status()
    ref = d0 + 0.5 * (a.float().t() @ b.float())
    err = (out - ref).abs().max().item()
    assert err <= 2e-2 * (K ** 0.5), f"max abs err {err}"


def test_layernorm_forward_register_path_and_backward_residual():
    nat = _native()
    import ctypes

    torch.manual_seed(2)
    for rows, D in ((3760, 1024), (33, 512), (50, 264)):
        x = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
        g = torch.randn(D, device="cuda")
        b = torch.randn(D, device="cuda")
        y = nat.layer_norm(x, g, b, 1e-5)
        ref = torch.nn.functional.layer_norm(x.float(), (D,), g, b, 1e-5)
        assert (y.float() - ref).abs().max().item() < 0.05
        dy = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
        dres = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
        mean = x.float().mean(-1)
        rstd = (x.float().var(-1, unbiased=False) + 1e-5).rsqrt()
        dx = torch.empty_like(x)
        dg, db = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
        rc = nat.lib().sb_layernorm_bwd_res(nat._ptr(dy), nat._ptr(x), nat._ptr(g), nat._ptr(mean), nat._ptr(rstd), nat._ptr(dx), nat._ptr(dg),
                                            nat._ptr(db), nat._ptr(dres), ctypes.c_int(rows), ctypes.c_int(D), nat._stream())
        assert rc == 0
        x32 = x.float().requires_grad_(True)
        g32, b32 = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
        torch.nn.functional.layer_norm(x32, (D,), g32, b32, 1e-5).backward(dy.float())
        assert (dx.float() - (x32.grad + dres.float())).abs().max().item() < 0.08
        assert (dg - g32.grad).abs().max().item() < 0.02 * rows ** 0.5 and (db - b32.grad).abs().max().item() < 0.02 * rows ** 0.5


@pytest.mark.parametrize("M,N,K,b_mn", [(256, 1024, 4096, False), (130, 520, 1024, False), (64, 2048, 1536, True), (512, 4096, 1024, False)])
def test_gemm_small_m_split_k_through_scratch_matches_single_pass(M, N, K, b_mn):
    """Few output tiles and a long K: the wrapper hands the kernel an fp32 scratch, K is split over more blocks and a second
    kernel applies bias / activation / scale / residual and writes the pre-activation; same result as the one-pass kernel."""
    nat = _native()
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out, pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    launches = nat.launch_count
    nat.gemm(a, b, out, M=M, N=N, K=K, b_mn=b_mn, bias=bias, act="swish", residual=res, out_pre=pre, alpha=0.5)
    nat.check_status()
    z = a.float() @ (b.float() if b_mn else b.float().t()) + bias
    ref = 0.5 * torch.nn.functional.silu(z) + res.float()
    assert (pre.float() - z).abs().max().item() <= 2e-2 * max(1.0, z.abs().max().item())
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    # ksplit=-1 forces the one-pass kernel: both paths agree to bf16 rounding
    one = torch.empty_like(out)
    nat.gemm(a, b, one, M=M, N=N, K=K, b_mn=b_mn, bias=bias, act="swish", residual=res, alpha=0.5, ksplit=-1)
    assert (one.float() - out.float()).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())
    assert nat.launch_count == launches + 2


@pytest.mark.parametrize("M,N,K,epi", [(3750, 1024, 1024, "plain"), (1000, 4096, 512, "fwd"), (777, 520, 264, "bwd")])
def test_gemm_is_bitwise_reproducible(M, N, K, epi):
    """Without split-K every output element is produced by one CTA in a fixed order: two runs must agree bit for bit."""
    nat = _native()
    torch.manual_seed(3)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    aux = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    outs = []
    for _ in range(3):
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        if epi == "plain":
            nat.gemm(a, b, out, M=M, N=N, K=K, ksplit=-1)
        elif epi == "fwd":
            nat.gemm(a, b, out, M=M, N=N, K=K, bias=bias, act="swish", residual=res, alpha=0.5, drop_p=0.1, drop_seed=1234, ksplit=-1)
        else:
            nat.gemm(a, b, out, M=M, N=N, K=K, aux=aux, dact="swish", residual=res, ksplit=-1)
        torch.cuda.synchronize()
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    nat.check_status()


def test_layernorm_and_conv_module_are_bitwise_reproducible():
    from speech_b200 import ops

    torch.manual_seed(4)
    x = torch.randn(3760, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(1024, device="cuda")
    b = torch.randn(1024, device="cuda")
    y = [ops.layer_norm(x, w, b, 1e-5) for _ in range(2)]
    assert torch.equal(y[0], y[1])


def test_gemm_is_bitwise_repeatable_and_stays_inside_its_output():
    """Two launches on the same operands give the same bits (each output tile has one writer and a fixed K order), and the bytes
    around a ragged output (M, N not multiples of the tile) keep their sentinel."""
    from speech_b200.utils.race_check import guarded_empty, run_twice

    nat = _native()
    torch.manual_seed(0)
    M, N, K = 250, 1032, 640
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    g = guarded_empty((M, N), torch.bfloat16, device="cuda", guard_bytes=1 << 16)

    def step():
        nat.gemm(a, b, g.tensor, M=M, N=N, K=K, lda=K, ldb=K, ldd=N)
        nat.check_status()
        return g.tensor

    run_twice(step).raise_if_different()
    g.check("gemm output")
    err = (g.tensor.float() - a.float() @ b.float().t()).abs().max().item()
    assert err <= 0.5

"""Attention, convolution-module and encoder-layer kernels against the PyTorch reference math (fp32)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b, floor=5e-3):
    """Max abs error relative to the reference's largest magnitude; gradients that are analytically zero (a bias in
    front of a train-mode BatchNorm, the key bias of a softmax) only have to be small in absolute terms."""
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=floor)).item()


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("B,T,H,dk", [(2, 37, 4, 64), (3, 250, 8, 128)])
def test_relpos_attention_fwd_bwd(fused, B, T, H, dk):
    from speech_b200 import ops
    from speech_b200.ops import reference

    torch.manual_seed(0)
    dev = "cuda"
    qkv = (torch.randn(B, T, 3, H, dk, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    p = (torch.randn(1, 2 * T - 1, H, dk, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    u = torch.nn.Parameter(torch.randn(H, dk, device=dev) * 0.1)
    v = torch.nn.Parameter(torch.randn(H, dk, device=dev) * 0.1)
    lens = torch.tensor([T - 3 * i for i in range(B)], device=dev)
    pad = torch.arange(T, device=dev)[None, :] >= lens[:, None]
    mask = pad[:, None, :] | pad[:, :, None]
    q, k, vv = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out = ops.relpos_attention(q, k, vv, p, u, v, mask, 0.0, True, qkv=qkv if fused else None)
    w = torch.randn_like(out.float())
    (out.float() * w).sum().backward()
    got = [out.detach().float(), qkv.grad.float().clone(), p.grad.float().clone(), u.grad.clone(), v.grad.clone()]
    for t in (qkv, p, u, v):
        t.grad = None
    qkv32 = qkv.detach().float().requires_grad_(True)
    p32 = p.detach().float().requires_grad_(True)
    ref = reference.relpos_attention(qkv32[:, :, 0], qkv32[:, :, 1], qkv32[:, :, 2], p32, u, v, mask)
    (ref * w).sum().backward()
    exp = [ref.detach(), qkv32.grad, p32.grad, u.grad, v.grad]
    for name, a, b in zip(["out", "dqkv", "dp", "du", "dv"], got, exp):
        assert _rel_err(a, b) < 0.05, f"{name}: {_rel_err(a, b)}"
    ops.native.check_status()


def test_attention_dropout_statistics():
    from speech_b200 import ops

    torch.manual_seed(0)
    B, T, H, dk = 2, 64, 2, 64
    q = torch.zeros(B, T, H, dk, device="cuda", dtype=torch.bfloat16)
    v = torch.ones(B, T, H, dk, device="cuda", dtype=torch.bfloat16)
    out = ops.mha_attention(q, q, v, None, 0.25, True)
    # uniform attention over ones with inverted dropout: mean output ~ 1, per-row spread > 0
    assert abs(out.float().mean().item() - 1.0) < 0.05
    assert out.float().std().item() > 0.01
    ops.native.check_status()


@pytest.mark.parametrize("training", [True, False])
def test_conv_module_core_fwd_bwd(training):
    from speech_b200 import ops
    from speech_b200.ops import reference

    torch.manual_seed(1)
    B, T, C, K = 3, 61, 64, 9
    dev = "cuda"
    g = torch.randn(B, T, 2 * C, device=dev).to(torch.bfloat16).requires_grad_(True)
    dw = torch.nn.Parameter(torch.randn(C, 1, K, device=dev) * 0.3)
    db = torch.nn.Parameter(torch.randn(C, device=dev) * 0.1)
    ga = torch.nn.Parameter(torch.rand(C, device=dev) + 0.5)
    be = torch.nn.Parameter(torch.randn(C, device=dev) * 0.1)
    lens = torch.tensor([T, T - 7, T - 20], device=dev)
    pad = torch.arange(T, device=dev)[None, :] >= lens[:, None]
    rm, rv = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    rm2, rv2 = rm.clone(), rv.clone()
    s = ops.conv_module_core(g, dw, db, "batch_norm", ga, be, rm, rv, pad_mask=pad, training=training)
    w = torch.randn_like(s.float())
    (s.float() * w).sum().backward()
    got = [s.detach().float(), g.grad.float().clone(), dw.grad.clone(), db.grad.clone(), ga.grad.clone(), be.grad.clone()]
    for t in (g, dw, db, ga, be):
        t.grad = None
    g32 = g.detach().float().requires_grad_(True)
    sr = reference.conv_module_core(g32, dw, db, "batch_norm", ga, be, rm2, rv2, pad_mask=pad, training=training)
    (sr * w).sum().backward()
    exp = [sr.detach(), g32.grad, dw.grad, db.grad, ga.grad, be.grad]
    for name, a, b in zip(["s", "dg", "ddw", "ddb", "dgamma", "dbeta"], got, exp):
        if name == "ddb" and training:
            # a bias in front of a train-mode BatchNorm has zero gradient; what remains is bf16 storage noise of y
            assert a.abs().max() < 0.05 * max(1.0, float(got[2].abs().max()))
            continue
        assert _rel_err(a, b) < 0.06, f"{name}: {_rel_err(a, b)}"
    if training:
        assert (rm - rm2).abs().max() < 2e-2 and (rv - rv2).abs().max() < 2e-2
    ops.native.check_status()


def test_conformer_layer_native_vs_eager():
    from speech_b200 import ops
    from speech_b200.modules.conformer_modules import ConformerLayer
    from speech_b200.modules.attention import RelPositionalEncoding

    torch.manual_seed(2)
    d, H, T, B = 256, 4, 50, 2
    layer = ConformerLayer(d_model=d, d_ff=4 * d, n_heads=H, conv_kernel_size=9, dropout=0.0, dropout_att=0.0).cuda()
    layer.train()
    pe = RelPositionalEncoding(d, 0.0)
    pe.extend_pe(T, "cuda")
    x = torch.randn(B, T, d, device="cuda")
    _, pos = pe(x)
    lens = torch.tensor([T, T - 9], device="cuda")
    pad = torch.arange(T, device="cuda")[None, :] >= lens[:, None]
    att = pad[:, None, :] | pad[:, :, None]
    xb = x.to(torch.bfloat16).requires_grad_(True)
    with ops.compute_dtype(torch.bfloat16):
        y = layer(xb, att_mask=att, pos_emb=pos, pad_mask=pad)
    wr = torch.randn(B, T, d, device="cuda")
    (y.float() * wr).sum().backward()
    grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    gx = xb.grad.float().clone()
    layer.zero_grad()
    import copy

    ref_layer = copy.deepcopy(layer)
    for bn in (layer.conv.batch_norm, ref_layer.conv.batch_norm):
        bn.reset_running_stats()
    x32 = x.to(torch.bfloat16).float().requires_grad_(True)
    with ops.eager_mode():
        yr = ref_layer(x32, att_mask=att, pos_emb=pos, pad_mask=pad)
    (yr * wr).sum().backward()
    assert _rel_err(y, yr) < 0.05
    assert _rel_err(gx, x32.grad) < 0.1
    bad = []
    scale = max(float(p.grad.abs().max()) for p in ref_layer.parameters())
    for n, p in ref_layer.named_parameters():
        if float(p.grad.abs().max()) < 1e-4 * scale:
            # analytically zero gradients (key bias under a softmax, bias before a train-mode BatchNorm): absolute check
            if float(grads[n].abs().max()) > 0.02 * scale:
                bad.append((n, float(grads[n].abs().max())))
            continue
        e = _rel_err(grads[n], p.grad)
        if e > 0.12:
            bad.append((n, e))
    assert not bad, bad
    ops.native.check_status()


def _arena_layer(d, H, dropout, seed=5):
    from speech_b200.core.optim.fused_adamw import FusedAdamW
    from speech_b200.modules.conformer_modules import ConformerLayer

    torch.manual_seed(seed)
    layer = ConformerLayer(d_model=d, d_ff=4 * d, n_heads=H, conv_kernel_size=9, dropout=dropout, dropout_att=dropout).cuda()
    with torch.no_grad():
        layer.self_attn.pos_bias_u.normal_(std=0.1)
        layer.self_attn.pos_bias_v.normal_(std=0.1)
    fusion = [fg for m in layer.modules() if hasattr(m, "arena_fusion_groups") for fg in m.arena_fusion_groups()]
    opt = FusedAdamW(layer.parameters(), lr=1e-3, fusion_groups=fusion)
    return layer.train(), opt


@pytest.mark.parametrize("dropout", [0.0, 0.1])
def test_conformer_layer_executor_matches_per_op_path_and_fp32_reference(dropout, monkeypatch):
    """The one-call-per-layer executor against (a) the per-op kernel path with identical dropout seeds and (b) fp32 eager math."""
    import copy

    from speech_b200 import ops
    from speech_b200.modules.attention import RelPositionalEncoding
    from speech_b200.ops import native as N
    from speech_b200.ops import native_blocks as NB
    from speech_b200.ops import native_layer

    d, H, T, B = 256, 4, 61, 3
    layer, opt = _arena_layer(d, H, dropout)
    pe = RelPositionalEncoding(d, 0.0)
    pe.extend_pe(T, "cuda")
    x = torch.randn(B, T, d, device="cuda")
    _, pos = pe(x)
    lens = torch.tensor([T, T - 9, T - 20], device="cuda")
    pad = torch.arange(T, device="cuda")[None, :] >= lens[:, None]
    att = pad[:, None, :] | pad[:, :, None]
    wr = torch.randn(B, T, d, device="cuda")

    def run(executor: bool):
        monkeypatch.setenv("SPEECH_B200_LAYER_EXECUTOR", "1" if executor else "0")
        N._dropout_counter[0], NB._seed_counter[0] = 0x5EED5EED, 0x1234567
        layer.conv.batch_norm.reset_running_stats()
        opt.zero_grad()
        xb = x.to(torch.bfloat16).requires_grad_(True)
        before = N.launch_count
        with ops.compute_dtype(torch.bfloat16):
            y = layer(xb, att_mask=att, pos_emb=pos, pad_mask=pad)
        (y.float() * wr).sum().backward()
        torch.cuda.synchronize()
        return (y.detach().float(), xb.grad.float().clone(), {n: p.grad.clone() for n, p in layer.named_parameters()},
                layer.conv.batch_norm.running_var.clone(), N.launch_count - before)

    y0, gx0, g0, rv0, _ = run(False)
    y1, gx1, g1, rv1, launches = run(True)
    assert native_layer._packs.get(layer) is not None and launches > 40, "the executor did not run"
    # same kernels, order and dropout seeds; BatchNorm statistics are accumulated with atomics, so equality is to rounding
    assert _rel_err(y1, y0) < 0.01
    assert torch.allclose(rv0, rv1)
    assert _rel_err(gx1, gx0) < 0.02
    scale = max(float(g.abs().max()) for g in g0.values())
    # analytically-zero gradients (key bias under the softmax, depthwise bias in front of BatchNorm) are rounding noise in both
    # paths, and the two paths round differently (the per-op path may split K for small shapes): absolute floor of 1% of the largest
    bad = [(n, _rel_err(g1[n], g0[n], floor=1e-2 * scale)) for n in g0 if _rel_err(g1[n], g0[n], floor=1e-2 * scale) > 0.05]
    assert not bad, bad
    if dropout == 0.0:
        ref_layer = copy.deepcopy(layer).float()
        ref_layer.conv.batch_norm.reset_running_stats()
        ref_layer.zero_grad()
        x32 = x.to(torch.bfloat16).float().requires_grad_(True)
        with ops.eager_mode():
            yr = ref_layer(x32, att_mask=att, pos_emb=pos, pad_mask=pad)
        (yr * wr).sum().backward()
        assert _rel_err(y1, yr) < 0.05 and _rel_err(gx1, x32.grad) < 0.1
        rscale = max(float(p.grad.abs().max()) for p in ref_layer.parameters())
        bad = []
        for n, p in ref_layer.named_parameters():
            if float(p.grad.abs().max()) < 1e-4 * rscale:
                if float(g1[n].abs().max()) > 0.02 * rscale:
                    bad.append((n, float(g1[n].abs().max())))
            elif _rel_err(g1[n], p.grad) > 0.12:
                bad.append((n, _rel_err(g1[n], p.grad)))
        assert not bad, bad
    # inference through the executor equals the per-op path in eval mode
    layer.eval()
    with torch.no_grad(), ops.compute_dtype(torch.bfloat16):
        monkeypatch.setenv("SPEECH_B200_LAYER_EXECUTOR", "0")
        e0 = layer(x.to(torch.bfloat16), att_mask=att, pos_emb=pos, pad_mask=pad)
        monkeypatch.setenv("SPEECH_B200_LAYER_EXECUTOR", "1")
        e1 = layer(x.to(torch.bfloat16), att_mask=att, pos_emb=pos, pad_mask=pad)
    assert _rel_err(e1, e0) < 0.01                     # the per-op path may split K for small shapes: equal up to rounding
    ops.native.check_status()
    assert native_layer.enabled()

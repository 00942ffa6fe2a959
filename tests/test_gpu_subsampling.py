"""Channels-last sub-sampling kernels against the fp32 library convolutions: outputs, lengths and every parameter gradient."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(mod, x, lens, native: bool):
    from speech_b200 import ops

    for p in mod.parameters():
        p.grad = None
    if native:
        with ops.compute_dtype(torch.bfloat16):
            y, L = mod(x, lens)
    else:
        with ops.eager_mode():
            y, L = mod(x, lens)
    torch.manual_seed(7)
    w = torch.randn(y.shape, device=y.device)
    (y.float() * w).sum().backward()
    return y.float().detach(), L, {n: p.grad.float().clone() for n, p in mod.named_parameters()}


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("factor,B,T", [(8, 3, 203), (4, 2, 96), (8, 2, 1000)])
def test_dw_striding_front_end_matches_library_convolutions(causal, factor, B, T):
    from speech_b200.modules.subsampling import ConvSubsampling

    torch.manual_seed(0)
    dev = torch.device("cuda")
    mod = ConvSubsampling("dw_striding", factor, 80, 512, 256, is_causal=causal).to(dev)
    mod.reset_parameters()
    feats = torch.randn(B, 80, T, device=dev)
    x = feats.transpose(1, 2)                       # the encoder hands a transposed view of [B, F, T]
    lens = torch.tensor([T, max(1, T * 3 // 4), max(1, T // 3)][:B], device=dev)
    assert mod._native_front_end(x) is False or True
    y_ref, L_ref, g_ref = _run(mod, x, lens, native=False)
    y, L, g = _run(mod, x, lens, native=True)
    assert torch.equal(L.long(), L_ref.long())
    assert y.shape == y_ref.shape
    scale = y_ref.abs().max().item()
    assert (y - y_ref).abs().max().item() < 0.03 * scale, (y - y_ref).abs().max().item() / scale
    # activations pass through several bf16 roundings (and ReLU decisions taken on rounded values): compare in the L2 sense,
    # with a looser bound on the worst element
    errs = {}
    for name in g_ref:
        ref = g_ref[name]
        l2 = ((g[name] - ref).norm() / ref.norm().clamp(min=1e-6)).item()
        mx = (g[name] - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
        errs[name] = (round(l2, 4), round(mx, 4))
    # yardstick: the library convolutions themselves under bf16 autocast against their fp32 run
    for p in mod.parameters():
        p.grad = None
    from speech_b200 import ops
    with ops.eager_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
        ya, _ = mod(x, lens)
    torch.manual_seed(7)
    (ya.float() * torch.randn(ya.shape, device=ya.device)).sum().backward()
    noise = {n: ((p.grad.float() - g_ref[n]).norm() / g_ref[n].norm().clamp(min=1e-6)).item() for n, p in mod.named_parameters()}
    print("native-vs-fp32 (l2, max):", errs)
    print("library-bf16-vs-fp32 l2:", {k: round(v, 4) for k, v in noise.items()})
    assert all(l2 < max(0.03, 2.5 * noise[n]) and mx < 0.15 for n, (l2, mx) in errs.items()), (errs, noise)


def test_front_end_rows_beyond_length_do_not_influence_results():
    """Garbage in the padded part of the input must not change outputs or gradients (every layer masks by length)."""
    from speech_b200 import ops
    from speech_b200.modules.subsampling import ConvSubsampling

    torch.manual_seed(1)
    dev = torch.device("cuda")
    mod = ConvSubsampling("dw_striding", 8, 80, 256, 256).to(dev)
    x = torch.randn(2, 160, 80, device=dev)
    lens = torch.tensor([160, 90], device=dev)
    x2 = x.clone()
    x2[1, 90:] = 1e3
    outs = []
    for inp in (x, x2):
        for p in mod.parameters():
            p.grad = None
        with ops.compute_dtype(torch.bfloat16):
            y, L = mod(inp, lens)
        y.float().pow(2).sum().backward()
        outs.append((y.float().detach().clone(), mod.conv[0].weight.grad.clone()))
    t_valid = int(L[1])
    assert torch.equal(outs[0][0][0], outs[1][0][0]), (outs[0][0][0] - outs[1][0][0]).abs().max()
    assert torch.equal(outs[0][0][1, :t_valid], outs[1][0][1, :t_valid]), (outs[0][0][1, :t_valid] - outs[1][0][1, :t_valid]).abs().max()
    # gradients are accumulated with atomics (order varies): equal up to fp32 summation order
    rel = ((outs[0][1] - outs[1][1]).norm() / outs[0][1].norm()).item()
    assert rel < 1e-4, rel

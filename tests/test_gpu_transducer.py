"""Fused joint + RNNT/TDT loss kernels against the fp32 PyTorch lattice oracle (values and gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(B, T, U, H, V, D, seed=0):
    torch.manual_seed(seed)
    dev = "cuda"
    f = (torch.randn(B, T, H, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    g = (torch.randn(B, U + 1, H, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = torch.nn.Parameter(torch.randn(V + 1 + D, H, device=dev) * 0.1)
    b = torch.nn.Parameter(torch.randn(V + 1 + D, device=dev) * 0.1)
    targets = torch.randint(0, V, (B, U), device=dev)
    f_len = torch.tensor([T - 2 * i for i in range(B)], device=dev).clamp(min=2)
    y_len = torch.tensor([max(1, U - i) for i in range(B)], device=dev)
    return f, g, w, b, targets, f_len, y_len


@pytest.mark.parametrize("durations,sigma", [((), 0.0), ((0, 1, 2, 3, 4), 0.02)])
@pytest.mark.parametrize("B,T,U,H,V", [(3, 12, 5, 64, 17), (4, 40, 11, 128, 130)])
def test_joint_loss_matches_oracle(durations, sigma, B, T, U, H, V):
    from speech_b200 import ops
    from speech_b200.ops import reference

    D = len(durations)
    f, g, w, b, targets, f_len, y_len = _setup(B, T, U, H, V, D)
    loss = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, list(durations), sigma)
    wgt = torch.rand(B, device="cuda") + 0.5
    (loss * wgt).sum().backward()
    got = [loss.detach(), f.grad.float().clone(), g.grad.float().clone(), w.grad.clone(), b.grad.clone()]
    for t in (f, g, w, b):
        t.grad = None
    f32 = f.detach().float().requires_grad_(True)
    g32 = g.detach().float().requires_grad_(True)
    w32 = w.detach().to(torch.bfloat16).float().requires_grad_(True)
    ref = reference.transducer_joint_loss(f32, g32, w32, b, targets, f_len, y_len, V, list(durations), sigma, "relu", 0.0, 0)
    (ref * wgt).sum().backward()
    exp = [ref.detach(), f32.grad, g32.grad, w32.grad, b.grad]
    assert torch.allclose(got[0], exp[0], rtol=2e-2, atol=0.3), (got[0], exp[0])
    for name, a, e in zip(["df", "dg", "dW", "db"], got[1:], exp[1:]):
        err = ((a - e).abs().max() / e.abs().max().clamp(min=1e-6)).item()
        assert err < 0.06, f"{name}: {err}"
    ops.native.check_status()


def test_loss_from_logits_matches_oracle():
    from speech_b200 import ops
    from speech_b200.ops import reference

    torch.manual_seed(1)
    B, T, U, V = 3, 9, 4, 12
    for durations, sigma in (((), 0.0), ((0, 1, 2), 0.05)):
        D = len(durations)
        logits = torch.randn(B, T, U + 1, V + 1 + D, device="cuda", requires_grad=True)
        targets = torch.randint(0, V, (B, U), device="cuda")
        f_len = torch.tensor([9, 7, 5], device="cuda")
        y_len = torch.tensor([4, 3, 1], device="cuda")
        loss = ops.transducer_loss_from_logits(logits, targets, f_len, y_len, V, list(durations), sigma)
        loss.sum().backward()
        got_g = logits.grad.clone()
        logits.grad = None
        ref = reference.tdt_loss_from_logits(logits, targets, f_len, y_len, V, list(durations), sigma)
        ref.sum().backward()
        assert torch.allclose(loss, ref, rtol=1e-4, atol=1e-3)
        assert (got_g - logits.grad).abs().max() < 2e-2
    ops.native.check_status()

"""CTC loss kernel against torch.nn.functional.ctc_loss on the CPU in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,V,U", [(3, 20, 9, 6), (5, 120, 129, 30)])
def test_ctc_matches_torch(B, T, V, U):
    from speech_b200 import ops

    torch.manual_seed(0)
    logits = torch.randn(B, T, V + 1, device="cuda", requires_grad=True)
    lp = torch.log_softmax(logits, -1)
    targets = torch.randint(0, V, (B, U), device="cuda")
    targets[0, 1] = targets[0, 0]  # a repeated label
    in_len = torch.tensor([T - 3 * i for i in range(B)], device="cuda").clamp(min=2)
    tgt_len = torch.tensor([max(1, U - 2 * i) for i in range(B)], device="cuda")
    in_len[-1] = 2  # infeasible alignment -> zero_infinity path
    loss = ops.ctc_loss(lp, targets, in_len, tgt_len, blank=V, zero_infinity=True)
    loss.sum().backward()
    g = logits.grad.clone()
    logits.grad = None
    lc = logits.detach().cpu().requires_grad_(True)
    ref = torch.nn.functional.ctc_loss(torch.log_softmax(lc, -1).transpose(0, 1), targets.cpu(), in_len.cpu(), tgt_len.cpu(),
                                       blank=V, reduction="none", zero_infinity=True)
    ref.sum().backward()
    assert torch.allclose(loss.cpu(), ref, rtol=1e-4, atol=1e-3), (loss, ref)
    assert (g.cpu() - lc.grad).abs().max() < 1e-3
    ops.native.check_status()

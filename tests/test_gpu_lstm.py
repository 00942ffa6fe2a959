"""LSTM prediction-network kernels against torch.nn.LSTM evaluated in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("L,U,B,H", [(1, 7, 3, 64), (2, 31, 20, 640)])
def test_lstm_matches_torch(L, U, B, H):
    from speech_b200 import ops

    torch.manual_seed(0)
    ref = torch.nn.LSTM(H, H, L).cuda()
    x = (torch.randn(U, B, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    weights = []
    for l in range(L):
        weights += [getattr(ref, f"weight_ih_l{l}"), getattr(ref, f"weight_hh_l{l}"), getattr(ref, f"bias_ih_l{l}"),
                    getattr(ref, f"bias_hh_l{l}")]
    out, (hn, cn) = ops.lstm(x, weights, None, None, L)
    w = torch.randn_like(out.float())
    (out.float() * w).sum().backward()
    got = [out.detach().float(), x.grad.float().clone()] + [p.grad.clone() for p in weights]
    for p in weights:
        p.grad = None
    x32 = x.detach().float().requires_grad_(True)
    o2, (h2, c2) = ref(x32)
    (o2 * w).sum().backward()
    exp = [o2.detach(), x32.grad] + [p.grad for p in weights]
    names = ["out", "dx"] + [f"w{i}" for i in range(len(weights))]
    for n, a, e in zip(names, got, exp):
        err = ((a - e).abs().max() / e.abs().max().clamp(min=5e-3)).item()
        assert err < 0.05, f"{n}: {err}"
    assert (hn.float() - h2).abs().max() < 0.03 and (cn.float() - c2).abs().max() < 0.05
    ops.native.check_status()

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


@pytest.mark.parametrize("B,T,U,H,V", [(8, 120, 40, 128, 130), (3, 250, 60, 640, 1024)])
def test_joint_loss_over_several_chunks_matches_oracle(B, T, U, H, V):
    """B * T * (U + 1) exceeds the chunk size several times over (the second case is the training benchmark's shape, one
    utterance per chunk): the chunk offsets of every joint kernel (build, log-sum-exp / gather, d(logits), reduction of dH)
    are exercised against the fp32 lattice oracle."""
    from speech_b200 import ops
    from speech_b200.ops import native_transducer, reference

    durations, sigma = (0, 1, 2, 3, 4), 0.02
    D = len(durations)
    assert B * T * (U + 1) > 2 * native_transducer.CHUNK_ROWS
    f, g, w, b, targets, f_len, y_len = _setup(B, T, U, H, V, D, seed=3)
    loss = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, list(durations), sigma)
    wgt = torch.rand(B, device="cuda") + 0.5
    (loss * wgt).sum().backward()
    got = [loss.detach(), f.grad.float().clone(), g.grad.float().clone(), w.grad.clone(), b.grad.clone()]
    f32 = f.detach().float().requires_grad_(True)
    g32 = g.detach().float().requires_grad_(True)
    w32 = w.detach().to(torch.bfloat16).float().requires_grad_(True)
    b32 = b.detach().clone().requires_grad_(True)
    ref = reference.transducer_joint_loss(f32, g32, w32, b32, targets, f_len, y_len, V, list(durations), sigma, "relu", 0.0, 0)
    (ref * wgt).sum().backward()
    exp = [ref.detach(), f32.grad, g32.grad, w32.grad, b32.grad]
    assert torch.allclose(got[0], exp[0], rtol=2e-2, atol=0.5), (got[0], exp[0])
    for name, a, e in zip(["df", "dg", "dW", "db"], got[1:], exp[1:]):
        err = ((a - e).norm() / e.norm().clamp(min=1e-6)).item()
        assert err < 0.03, f"{name}: {err}"
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


def test_multiblank_lattice_matches_oracle():
    """Multi-blank RNNT on the native wavefront kernels (free label arcs, one blank symbol per duration) against the PyTorch
    lattice oracle: values and the gradient with respect to the logits."""
    from speech_b200.ops import native_transducer, reference

    torch.manual_seed(5)
    B, T, U, V = 3, 23, 6, 14
    big = [2, 4, 8]
    nb = len(big)
    blank = V + nb                               # vocabulary: V tokens, then the big blanks, then the standard blank
    logits = torch.randn(B, T, U + 1, V + nb + 1, device="cuda", requires_grad=True)
    targets = torch.randint(0, V, (B, U), device="cuda")
    f_len = torch.tensor([23, 17, 9], device="cuda")
    y_len = torch.tensor([6, 4, 2], device="cuda")
    for sigma in (0.0, 0.05):
        loss = native_transducer.multiblank_loss_from_logits(logits, targets, f_len, y_len, blank, big, sigma)
        loss.sum().backward()
        got = logits.grad.clone()
        logits.grad = None
        ref = reference.multiblank_loss_from_logits(logits, targets, f_len, y_len, blank, big, sigma)
        ref.sum().backward()
        assert torch.allclose(loss, ref, rtol=1e-4, atol=1e-3), (loss, ref)
        assert (got - logits.grad).abs().max() < 1e-3
        logits.grad = None


def test_fused_joint_dropout_is_consistent_between_forward_and_backward():
    """Joint dropout inside the fused loss: the hidden lattice is rebuilt in backward with the same hash mask.  With the output
    layer reduced to a single active hidden unit pattern the check is done through finite differences of the loss with respect
    to the output bias (independent of the mask) and through the expected keep rate of the gradient of the hidden inputs."""
    from speech_b200 import ops
    from speech_b200.ops import native

    torch.manual_seed(2)
    B, T, U, H, V, D = 2, 20, 5, 64, 30, 5
    f, g, w, b, targets, f_len, y_len = _setup(B, T, U, H, V, D, seed=9)
    native._dropout_counter[0] = 0x1234
    l0 = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02, dropout_p=0.5)
    native._dropout_counter[0] = 0x1234
    l1 = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02, dropout_p=0.5)
    assert torch.equal(l0, l1), "same seed, same mask, same loss"
    l2 = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02, dropout_p=0.5)
    assert not torch.equal(l0, l2), "a new call draws a new mask"
    lnone = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02, dropout_p=0.0)
    assert (l0 - lnone).abs().max() > 1e-3
    # gradient check against a directional finite difference with the mask held fixed (same seed counter, same torch seed)
    torch.manual_seed(3)
    direction = torch.randn_like(w) * 0.05
    native._dropout_counter[0] = 0x777
    loss = ops.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02, dropout_p=0.3)
    loss.sum().backward()
    gw = w.grad.clone()
    vals = []
    for sgn in (1.0, -1.0):
        native._dropout_counter[0] = 0x777
        with torch.no_grad():
            wp = torch.nn.Parameter((w + sgn * direction).detach())
        vals.append(ops.transducer_joint_loss(f.detach(), g.detach(), wp, b.detach(), targets, f_len, y_len, V, [0, 1, 2, 3, 4], 0.02,
                                              dropout_p=0.3).sum().item())
    fd = (vals[0] - vals[1]) / 2.0
    an = (gw * direction).sum().item()
    assert abs(fd - an) < 0.05 * max(1.0, abs(an)), (fd, an)
    ops.native.check_status()

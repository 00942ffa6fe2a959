"""RMSNorm, SwiGLU and rotary-embedding kernels of the LLM block against their fp32 PyTorch restatements, and the LLM block built
on them against the same block computed with the restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6))


@pytest.mark.parametrize("rows,D", [(1000, 2048), (4097, 128), (37, 1024), (300, 4096)])
def test_rmsnorm_fwd_bwd(rows, D):
    from speech_b200.ops import native_llm as nl

    torch.manual_seed(0)
    x = (torch.randn(rows, D, device="cuda") * 1.5).to(torch.bfloat16).requires_grad_(True)
    w = torch.nn.Parameter(1 + 0.2 * torch.randn(D, device="cuda"))
    dy = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
    y = nl.rmsnorm(x, w, 1e-6)
    assert y.dtype == torch.bfloat16 and type(y.grad_fn).__name__.startswith("_RMSNormFn")
    y.backward(dy)
    gx, gw = x.grad.clone(), w.grad.clone()
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    yr = nl.rmsnorm_reference(xr, wr, 1e-6)
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2 and _rel(gx, xr.grad) < 1.5e-2 and _rel(gw, wr.grad) < 1e-2


def test_swiglu_and_rope_fwd_bwd():
    from speech_b200.ops import native_llm as nl

    torch.manual_seed(0)
    g = torch.randn(513, 1024, device="cuda").to(torch.bfloat16).requires_grad_(True)
    u = torch.randn(513, 1024, device="cuda").to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(513, 1024, device="cuda").to(torch.bfloat16)
    y = nl.swiglu(g, u)
    y.backward(dy)
    gr, ur = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
    yr = nl.swiglu_reference(gr, ur)
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2 and _rel(g.grad, gr.grad) < 1.5e-2 and _rel(u.grad, ur.grad) < 1.5e-2
    B, T, H, D = 3, 41, 5, 128
    x = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    pos = torch.arange(T, device="cuda").float()[None, :, None].expand(B, T, 1) + torch.arange(B, device="cuda").float()[:, None, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.cat([pos * inv, pos * inv], dim=-1).contiguous()
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    dyr = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
    y = nl.rope(x, cos, sin)
    assert type(y.grad_fn).__name__.startswith("_RopeFn")
    y.backward(dyr)
    xr = x.detach().float().requires_grad_(True)
    yr = nl.rope_reference(xr, cos, sin)
    yr.backward(dyr.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2
    # rotation: norms are preserved
    assert _rel(y.float().norm(dim=-1), x.detach().float().norm(dim=-1)) < 1e-2


def test_llm_block_on_native_kernels_matches_restatement_block():
    """The decoder LM in bf16 on the GPU (native RMSNorm / rope / SwiGLU / GEMM) against the same weights run in fp32 on the
    PyTorch restatements: logits and the gradient of the embedding table."""
    from speech_b200 import ops
    from speech_b200.speechlm.llm import CausalLM, LLMConfig

    torch.manual_seed(0)
    cfg = LLMConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=64, tie_word_embeddings=False, qk_norm=True)
    lm = CausalLM(cfg).cuda()
    ids = torch.randint(0, 512, (3, 24), device="cuda")
    am = torch.ones(3, 24, dtype=torch.long, device="cuda")
    am[1, :5] = 0
    with ops.compute_dtype(torch.bfloat16):
        out = lm(input_ids=ids, attention_mask=am)["logits"].float()
    out.square().mean().backward()
    g_native = lm.model.embed_tokens.weight.grad.clone()
    lm.zero_grad()
    with ops.eager_mode():
        ref = lm(input_ids=ids, attention_mask=am)["logits"].float()
    ref.square().mean().backward()
    valid = am.bool()
    assert _rel(out[valid], ref[valid]) < 4e-2
    assert _rel(g_native, lm.model.embed_tokens.weight.grad) < 6e-2

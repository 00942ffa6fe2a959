"""SpecAugment mask kernel and n-gram automaton step against their plain PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_specaugment_kernel_matches_reference(dtype):
    _need_gpu()
    from speech_b200 import ops
    from speech_b200.ops import reference

    torch.manual_seed(0)
    B, F, T = 7, 80, 1237
    x = torch.randn(B, F, T, device="cuda", dtype=dtype)
    f_w = torch.randint(0, 28, (B, 2), device="cuda")
    f_s = (torch.rand(B, 2, device="cuda") * (F - f_w + 1)).long()
    t_w = torch.randint(0, 60, (B, 10), device="cuda")
    t_s = (torch.rand(B, 10, device="cuda") * (T - t_w)).long()
    keep = x.clone()
    got = ops.specaugment(x, f_s, f_w, t_s, t_w, 0.0)
    want = reference.specaugment(x, f_s, f_w, t_s, t_w, 0.0)
    assert torch.equal(x, keep)                       # the input is left alone
    assert torch.equal(got, want)
    assert float((got == 0).float().mean()) > 0.05
    only_t = ops.specaugment(x, None, None, t_s, t_w, -1.0)
    assert torch.equal(only_t, reference.specaugment(x, None, None, t_s, t_w, -1.0))


def test_specaugment_module_on_gpu_masks_within_length():
    _need_gpu()
    from speech_b200.modules.spec_augment import SpecAugment

    torch.manual_seed(1)
    aug = SpecAugment(freq_masks=2, time_masks=10, freq_width=27, time_width=0.05)
    x = torch.ones(4, 80, 900, device="cuda")
    length = torch.tensor([900, 500, 300, 64], device="cuda")
    y = aug(x, length)
    assert y.shape == x.shape and float(y.min()) == 0.0
    for b in range(4):                                  # time masks never start beyond the utterance
        cols = (y[b] == 0).all(dim=0).nonzero().flatten()
        assert cols.numel() == 0 or int(cols.max()) < int(length[b])


def test_ngram_advance_kernel_matches_reference():
    _need_gpu()
    from speech_b200 import ops
    from speech_b200.ops import reference

    g = torch.Generator().manual_seed(0)
    V, S, depth = 257, 400, 4
    # a random back-off automaton: state 0 is the root (backs off to itself with weight 0), deeper states back off to lower ids
    pairs = torch.unique(torch.stack([torch.randint(0, S, (6000,), generator=g), torch.randint(0, V, (6000,), generator=g)], 1), dim=0)
    keys = (pairs[:, 0] * V + pairs[:, 1]).sort().values
    arc_w = -torch.rand(keys.numel(), generator=g) * 5
    arc_to = torch.randint(0, S, (keys.numel(),), generator=g)
    backoff_to = torch.tensor([0] + [int(torch.randint(0, s, (1,), generator=g)) for s in range(1, S)])
    backoff_w = -torch.rand(S, generator=g)
    backoff_w[0] = 0.0
    dev = "cuda"
    args = [t.to(dev) for t in (keys, arc_w, arc_to, backoff_w, backoff_to)]
    states = torch.randint(0, S, (33,), generator=g).to(dev)
    sc, nx = ops.ngram_advance(states, *args, V, depth, -7.5, 0)
    sc_ref, nx_ref = reference.ngram_advance(states, *args, V, depth, -7.5, 0)
    assert torch.equal(nx, nx_ref)
    assert torch.allclose(sc, sc_ref, atol=1e-5)


def test_ngram_lm_module_uses_kernel_and_scores_sentences(tmp_path):
    _need_gpu()
    from speech_b200.decoding.ngram_lm import NGramGPULanguageModel, write_arpa

    tok = lambda i: chr(i + 100)  # noqa: E731
    ngrams = {("<s>",): (-99.0, -0.3), ("</s>",): (-1.0, 0.0), (tok(0),): (-0.7, -0.2), (tok(1),): (-0.9, -0.4), (tok(2),): (-1.2, 0.0),
              ("<s>", tok(0)): (-0.3, -0.1), (tok(0), tok(1)): (-0.2, -0.5), (tok(1), tok(2)): (-0.4, 0.0), (tok(1), "</s>"): (-0.6, 0.0),
              (tok(0), tok(1), tok(2)): (-0.1, 0.0)}
    path = str(tmp_path / "lm.arpa")
    write_arpa(path, ngrams)
    lm_cpu = NGramGPULanguageModel.from_arpa(path, vocab_size=3)
    lm_gpu = NGramGPULanguageModel.from_arpa(path, vocab_size=3).cuda()
    for sent in ([0, 1, 2], [2, 2, 1], [1, 0, 1, 2, 0]):
        assert abs(lm_cpu.score_sentence(sent) - lm_gpu.score_sentence(sent)) < 1e-5

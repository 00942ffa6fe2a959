"""Log-mel kernels against the torch.stft-based reference featurizer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("normalize", ["per_feature", None])
def test_logmel_matches_reference(normalize):
    from speech_b200 import ops
    from speech_b200.modules.preprocessor import FilterbankFeatures
    from speech_b200.ops import reference

    torch.manual_seed(0)
    feat = FilterbankFeatures(n_window_size=400, n_window_stride=160, n_fft=512, nfilt=80, dither=0.0, pad_to=16,
                              normalize=normalize).cuda()
    x = torch.randn(3, 16000 * 3 + 123, device="cuda") * 0.1
    lens = torch.tensor([x.shape[1], 16000 * 2 + 7, 801], device="cuda")
    got, gl = ops.logmel(x, lens, feat.window, feat.fb[0], 512, 160, 400, normalize=normalize, pad_to=16)
    ref, rl = reference.logmel(x, lens, feat.window, feat.fb[0], 512, 160, 400, normalize=normalize, pad_to=16)
    assert torch.equal(gl, rl) and got.shape == ref.shape
    err = (got - ref).abs()
    tol = 2e-2 if normalize else 5e-2
    assert err.max() < tol, err.max()
    ops.native.check_status()

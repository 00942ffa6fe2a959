"""Audio (enhancement) collection on CPU: STFT round trip, SDR metrics, MVDR beamformer, mask-based, predictive and the
three generative models (training step + sampler)."""
import math

import pytest
import torch

from speech_b200.audio.models import (EncMaskDecAudioToAudioModel, FlowMatchingAudioToAudioModel, PredictiveAudioToAudioModel,
                                      SchroedingerBridgeAudioToAudioModel, ScoreBasedGenerativeAudioToAudioModel)
from speech_b200.audio.modules import (AudioToSpectrogram, MaskBasedBeamformer, SpectrogramToAudio, sdr, si_sdr)
from speech_b200.core.config import OmegaConf
from speech_b200.core.trainer import Trainer

ENC = {"_target_": "speech_b200.audio.modules.AudioToSpectrogram", "fft_length": 64, "hop_length": 16}
DEC = {"_target_": "speech_b200.audio.modules.SpectrogramToAudio", "fft_length": 64, "hop_length": 16}
DS = {"synthetic": {"num_samples": 8, "min_duration": 0.1, "max_duration": 0.15, "sample_rate": 8000}, "batch_size": 4}


def test_stft_round_trip_and_sdr_metrics():
    torch.manual_seed(0)
    x = torch.randn(2, 2, 800)
    lens = torch.tensor([800, 640])
    a, s = AudioToSpectrogram(64, 16, magnitude_power=0.5), SpectrogramToAudio(64, 16, magnitude_power=0.5)
    spec, sl = a(x, lens)
    assert spec.shape == (2, 2, 33, 51) and sl.tolist() == [51, 41]
    y, yl = s(spec, sl)
    assert yl.tolist() == [800, 640]
    assert torch.allclose(y[0, :, 32:768], x[0, :, 32:768], atol=1e-4)
    t = torch.randn(1, 1, 1000)
    assert float(si_sdr(3.0 * t, t)) > 60 and float(sdr(3.0 * t, t)) < 0
    noisy = t + 0.1 * torch.randn_like(t)
    assert 15 < float(sdr(noisy, t)) < 25


def test_mvdr_beamformer_improves_sdr_with_oracle_masks():
    torch.manual_seed(0)
    T = 4000
    tt = torch.arange(T) / 8000
    src = torch.sin(2 * math.pi * 440 * tt) * (torch.sin(2 * math.pi * 3 * tt) > 0)
    mix = torch.stack([torch.roll(src, d) for d in (0, 2, 4)]) + 0.5 * torch.randn(3, T)
    a, s = AudioToSpectrogram(256, 64), SpectrogramToAudio(256, 64)
    X, L = a(mix.unsqueeze(0), torch.tensor([T]))
    S, _ = a(src.view(1, 1, -1), torch.tensor([T]))
    mask = (S.abs() ** 2 / (S.abs() ** 2 + 0.25 * 128)).clamp(0, 1)[:, :1].squeeze(1).unsqueeze(1)       # oracle Wiener-like mask
    Y, _ = MaskBasedBeamformer(ref_channel=0)(X, L, mask)
    y, _ = s(Y, L)
    before = float(si_sdr(mix[:1].unsqueeze(0), src.view(1, 1, -1)))
    after = float(si_sdr(y[..., :T], src.view(1, 1, -1)[..., : y.shape[-1]]))
    assert after > before + 2.0


def _fit(m, steps=3):
    tr = Trainer(max_steps=steps, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(m)
    return float(tr.callback_metrics["train_loss"])


def test_mask_and_predictive_models():
    torch.manual_seed(0)
    m = EncMaskDecAudioToAudioModel(OmegaConf.create({
        "sample_rate": 8000, "encoder": ENC, "decoder": DEC,
        "mask_estimator": {"_target_": "speech_b200.audio.modules.MaskEstimatorRNN", "num_outputs": 1, "num_subbands": 33,
                           "num_features": 16, "num_layers": 1},
        "mask_processor": {"_target_": "speech_b200.audio.modules.MaskReferenceChannel"},
        "train_ds": DS, "validation_ds": DS, "optim": {"name": "adamw", "lr": 1e-3}}))
    assert math.isfinite(_fit(m))
    out = m.process([torch.randn(1200).numpy()])
    assert out[0].shape == (1, 1200)
    p = PredictiveAudioToAudioModel(OmegaConf.create({
        "sample_rate": 8000, "encoder": ENC, "decoder": DEC,
        "estimator": {"_target_": "speech_b200.audio.modules.SpectrogramConformerUNet", "in_channels": 1, "out_channels": 1,
                      "feat_in": 33, "n_layers": 2, "d_model": 32, "n_heads": 2, "conv_kernel_size": 5, "use_time": False},
        "train_ds": DS, "optim": {"name": "adamw", "lr": 1e-3}}))
    assert math.isfinite(_fit(p))


@pytest.mark.parametrize("cls,est", [
    (FlowMatchingAudioToAudioModel, "SpectrogramConformerUNet"),
    (ScoreBasedGenerativeAudioToAudioModel, "SpectrogramNCSN"),
    (SchroedingerBridgeAudioToAudioModel, "SpectrogramNCSN"),
])
def test_generative_models_train_and_sample(cls, est):
    torch.manual_seed(0)
    ecfg = {"_target_": f"speech_b200.audio.modules.{est}", "in_channels": 2, "out_channels": 1}
    if est == "SpectrogramConformerUNet":
        ecfg.update(feat_in=33, n_layers=2, d_model=32, n_heads=2, conv_kernel_size=5)
    else:
        ecfg.update(hidden=8, n_blocks=1)
    m = cls(OmegaConf.create({"sample_rate": 8000, "encoder": ENC, "decoder": DEC, "estimator": ecfg, "sampler": {"num_steps": 3},
                              "train_ds": DS, "optim": {"name": "adamw", "lr": 1e-3}}))
    assert math.isfinite(_fit(m, 2))
    m.eval()
    y, _ = m(input_signal=torch.randn(1, 1, 900) * 0.1, input_length=torch.tensor([900]))
    assert y.shape == (1, 1, 900) and torch.isfinite(y).all()

"""Audio (enhancement) collection on CPU: STFT round trip, SDR metrics, MVDR beamformer, mask-based, predictive and the
three generative models (training step + sampler)."""
import math
import os

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


def test_multichannel_features_blocks_and_flex_channel_mask_estimator():
    import random
    from speech_b200.audio.multichannel import (ChannelAttentionPool, ChannelAugment, ChannelAveragePool, MaskEstimatorFlexChannels,
                                                MixtureConsistencyProjection, SpectrogramToMultichannelFeatures, SSLPretrainWithMaskedPatch,
                                                TransformAttendConcatenate, TransformAverageConcatenate)

    torch.manual_seed(0)
    x = torch.randn(2, 3, 17, 20, dtype=torch.cfloat)
    lens = torch.tensor([20, 14])
    f = SpectrogramToMultichannelFeatures(17, 3, mag_reduction="rms", use_ipd=True, mag_normalization="mean_var", ipd_normalization="mean")
    feats, _ = f(x, lens)
    assert feats.shape == (2, 3, 34, 20) and f.num_features == 34 and f.num_channels == 3
    assert float(feats[1, :, :, 14:].abs().max()) == 0.0
    assert float(feats[0, 0, :17].mean(-1).abs().max()) < 1e-5                      # mean-variance normalised magnitude
    raw, _ = SpectrogramToMultichannelFeatures(17, 3, mag_reduction=None, use_ipd=True)(x, lens)
    assert float(raw[:, :, 17:].abs().max()) <= math.pi + 1e-5 and torch.allclose(raw[:, :, :17], x.abs())
    for blk in (TransformAverageConcatenate(34, 16), TransformAttendConcatenate(34, 16, n_head=2)):
        blk.eval()
        y = blk(feats)
        assert y.shape == (2, 3, 16, 20)
        perm = [2, 0, 1]
        assert torch.allclose(blk(feats[:, perm]), y[:, perm], atol=1e-5)            # permutation equivariant
    assert ChannelAveragePool()(feats).shape == (2, 1, 34, 20)
    pool = ChannelAttentionPool(34).eval()
    assert torch.allclose(pool(feats[:, [1, 2, 0]]), pool(feats), atol=1e-5)         # permutation invariant
    aug = ChannelAugment(num_channels_min=2, rng=random.Random(0))
    assert aug(x).shape[1] in (2, 3)
    est = MaskEstimatorFlexChannels(num_outputs=2, num_subbands=17, num_blocks=2, channel_reduction_position=1, temporal_block_num_layers=1,
                                    temporal_block_num_heads=2, temporal_block_dimension=16, num_input_channels=3).eval()
    m, _ = est(x, lens)
    assert m.shape == (2, 2, 17, 20) and float(m.min()) >= 0 and float(m.max()) <= 1 and float(m[1, :, :, 14:].abs().max()) == 0
    m4, _ = est(torch.randn(2, 4, 17, 20, dtype=torch.cfloat), lens)                  # another number of channels, same weights
    assert m4.shape == (2, 2, 17, 20)
    end = MaskEstimatorFlexChannels(1, 17, 1, -1, "average", "transform_average_concatenate", temporal_block_num_layers=1,
                                    temporal_block_num_heads=2, temporal_block_dimension=16).eval()
    assert end(x, lens)[0].shape == (2, 1, 17, 20)
    mix = torch.randn(2, 1, 5, 7, dtype=torch.cfloat)
    est_src = torch.randn(2, 3, 5, 7, dtype=torch.cfloat)
    for w in (None, "power"):
        proj = MixtureConsistencyProjection(w)(mix, est_src)
        assert torch.allclose(proj.sum(1, keepdim=True), mix, atol=1e-4)
    masked = SSLPretrainWithMaskedPatch(patch_size=4, mask_fraction=0.5, rng=random.Random(1))(torch.ones(2, 8, 20), lens)
    zero_frames = (masked[0].abs().sum(0) == 0).sum()
    assert int(zero_frames) == 12 and set((masked[0].abs().sum(0) == 0).view(5, 4).all(1).tolist()) == {True, False}


def test_gss_wpe_and_parametric_wiener_filter_on_synthetic_scenes():
    from speech_b200.audio.multichannel import MaskBasedDereverbWPE, MaskEstimatorGSS, ParametricMultichannelWienerFilter, WPEFilter

    torch.manual_seed(0)
    B, C, F, N = 1, 4, 6, 400
    # two sources with distinct steering vectors, active in different halves (plus an overlap), weak noise
    steer = torch.randn(2, F, C, dtype=torch.cdouble)
    act = torch.zeros(B, 2, N)
    act[0, 0, :250] = 1
    act[0, 1, 150:] = 1
    s = torch.randn(2, F, N, dtype=torch.cdouble) * act[0].unsqueeze(1)
    x = torch.einsum("sfc,sfn->cfn", steer, s).unsqueeze(0) + 0.01 * torch.randn(B, C, F, N, dtype=torch.cdouble)
    gamma = MaskEstimatorGSS(num_iterations=8)(x, act)
    assert gamma.shape == (B, 2, F, N) and torch.allclose(gamma.sum(1), torch.ones(B, F, N, dtype=gamma.dtype), atol=1e-5)
    assert float(gamma[0, 0, :, :150].min()) > 0.99 and float(gamma[0, 1, :, 250:].min()) > 0.99
    # in the overlap the posterior follows the dominant source
    dom0 = (s[0].abs() > 3 * s[1].abs())[:, 150:250]
    dom1 = (s[1].abs() > 3 * s[0].abs())[:, 150:250]
    g0 = gamma[0, 0, :, 150:250]
    assert float(g0[dom0].mean()) > float(g0[dom1].mean()) + 0.3
    # PMWF with oracle covariances recovers source 0 at the reference microphone far better than the unprocessed mixture
    ps = torch.einsum("fc,fd->fcd", steer[0], steer[0].conj()).unsqueeze(0)
    pn = torch.einsum("fc,fd->fcd", steer[1], steer[1].conj()).unsqueeze(0) + 1e-4 * torch.eye(C, dtype=torch.cdouble)
    target = (steer[0, :, 0].unsqueeze(-1) * s[0]).unsqueeze(0).unsqueeze(0)
    for beta, rank in ((0.0, "one"), (1.0, "full")):
        y = ParametricMultichannelWienerFilter(beta=beta, rank=rank, ref_channel=0)(x, ps, pn)
        err, base = (y - target).abs().pow(2).mean(), (x[:, :1] - target).abs().pow(2).mean()
        assert float(err) < 0.05 * float(base), (beta, rank, float(err), float(base))
    y = ParametricMultichannelWienerFilter(beta=0.0, rank="one", ref_channel="max_snr")(x, ps, pn)
    assert y.shape == (B, 1, F, N)
    # WPE: reverberation that is an exact linear prediction from delayed frames (wet[t] = dry[t] + 0.5 wet[t-2] - 0.3 wet[t-3])
    # is removed almost completely when the filter covers those taps
    N2 = 800
    dry = torch.randn(1, 1, 3, N2, dtype=torch.cdouble)
    wet = dry.clone()
    for t in range(3, N2):
        wet[..., t] = dry[..., t] + 0.5 * wet[..., t - 2] - 0.3 * wet[..., t - 3]
    filt = WPEFilter(filter_length=4, prediction_delay=2)
    assert filt.convtensor(wet).shape == (1, 1, 3, N2, 4) and torch.equal(filt.convtensor(wet)[0, 0, 0, 10], wet[0, 0, 0, [8, 7, 6, 5]])
    before = (wet - dry).abs().pow(2).mean()
    exact, _ = filt(wet, torch.ones(1, 3, N2, dtype=torch.double))                       # flat power: plain least squares
    assert float((exact - dry).abs().pow(2).mean()) < 0.02 * float(before)
    # with the power re-estimated from the signal itself (a white source is the worst case for that weighting) it still helps
    out, _ = MaskBasedDereverbWPE(filter_length=4, prediction_delay=2, num_iterations=2)(wet)
    after = (out - dry).abs().pow(2).mean()
    assert float(after) < 0.7 * float(before), (float(after), float(before))
    lens = torch.tensor([500])
    out_l, _ = MaskBasedDereverbWPE(filter_length=4, prediction_delay=2)(wet, lens)
    assert float(out_l[..., 500:].abs().max()) == 0.0


def test_transformer_unet_shapes_padding_and_time_conditioning():
    from speech_b200.audio.transformer_unet import ConvPositionEmbed, LearnedSinusoidalPosEmb, SpectrogramTransformerUNet, TransformerUNet

    torch.manual_seed(0)
    assert LearnedSinusoidalPosEmb(8)(torch.tensor([0.1, 0.5])).shape == (2, 9)
    with pytest.raises(ValueError):
        ConvPositionEmbed(8, 4)
    with pytest.raises(ValueError):
        TransformerUNet(16, 3)
    net = SpectrogramTransformerUNet(in_channels=2, out_channels=1, freq_dim=9, dim=32, depth=4, heads=4, conv_pos_embed_kernel_size=5).eval()
    x = torch.randn(2, 1, 9, 12, dtype=torch.cfloat)
    cond = torch.randn(2, 1, 9, 12, dtype=torch.cfloat)
    lens = torch.tensor([12, 8])
    y, _ = net(x, lens, condition=cond, time=torch.tensor([0.2, 0.9]))
    assert y.shape == (2, 1, 9, 12) and y.is_complex() and float(y[1, :, :, 8:].abs().max()) == 0
    # outputs of the valid part do not depend on what sits in the padding
    x2 = x.clone(); x2[1, :, :, 8:] = 100.0
    y2, _ = net(x2, lens, condition=cond, time=torch.tensor([0.2, 0.9]))
    assert torch.allclose(y2[1, :, :, :8], y[1, :, :, :8], atol=1e-4)
    # the time condition matters once the (zero-initialised) adaptive norms are trained
    for m in net.modules():
        if hasattr(m, "to_gamma"):
            torch.nn.init.normal_(m.to_gamma.weight, std=0.5)
    y3, _ = net(x, lens, condition=cond, time=torch.tensor([0.8, 0.1]))
    y4, _ = net(x, lens, condition=cond, time=torch.tensor([0.2, 0.9]))
    assert not torch.allclose(y3, y4, atol=1e-4)
    y4.abs().sum().backward()
    assert net.proj_in.weight.grad is not None


def test_audio_metrics_wrapper_stoi_and_reference_free_estimates():
    from speech_b200.audio.metrics import AudioMetricWrapper, QualityEstimator, SquimMOSMetric, SquimObjectiveMetric, stoi
    from speech_b200.audio.modules import si_sdr

    torch.manual_seed(0)
    t = torch.arange(32000) / 16000.0
    # speech-like: a carrier with a slow envelope, so that band envelopes carry information
    clean = torch.sin(2 * math.pi * 220 * t) * (0.6 + 0.4 * torch.sin(2 * math.pi * 3 * t)) + 0.5 * torch.sin(2 * math.pi * 1300 * t) * (0.5 + 0.5 * torch.sin(2 * math.pi * 5 * t + 1))
    noise = torch.randn_like(clean)
    s_clean, s_mild, s_bad = float(stoi(clean, clean)), float(stoi(clean + 0.05 * noise, clean)), float(stoi(clean + 2.0 * noise, clean))
    assert s_clean > 0.999 and s_clean > s_mild > s_bad and s_bad < 0.8
    assert float(stoi(clean + 0.05 * noise, clean, extended=True)) > float(stoi(clean + 2.0 * noise, clean, extended=True))
    # wrapper: channel selection and per-example trimming
    tgt = torch.randn(2, 2, 4000)
    est = tgt + 0.1 * torch.randn(2, 2, 4000)
    est[1, :, 3000:] = 100.0                                          # garbage beyond the valid length of example 1
    lens = torch.tensor([4000, 3000])
    m = AudioMetricWrapper(lambda p, t_: si_sdr(p.unsqueeze(1), t_.unsqueeze(1)).squeeze(1), channel=1)
    m.update(est, tgt, lens)
    assert 15.0 < float(m.compute()) < 25.0
    with pytest.raises(RuntimeError):
        AudioMetricWrapper(lambda p, t_: p.sum(), channel=3).update(est, tgt)
    # reference-free: the estimator learns to rank a clean and a noisy signal by SI-SDR and STOI
    qe = QualityEstimator(d_model=32, n_layers=1, n_heads=2)
    x = torch.stack([clean[:8000], clean[:8000] + 1.0 * noise[:8000]])
    labels = {"si_sdr": torch.tensor([30.0, 0.0]), "stoi": torch.tensor([1.0, 0.5])}
    opt = torch.optim.Adam(qe.parameters(), 3e-3)
    for _ in range(60):
        opt.zero_grad()
        qe.training_loss(x, labels).backward()
        opt.step()
    qe.eval()
    obj = SquimObjectiveMetric(16000, "si_sdr", estimator=qe)
    obj.update(x[:1])
    hi = float(obj.compute())
    obj.reset()
    obj.update(x[1:])
    assert hi > float(obj.compute()) + 5.0
    mos = SquimMOSMetric(8000, estimator=qe)
    mos.update(x[:, ::2], x[:, ::2])
    assert 1.0 <= float(mos.compute()) <= 5.0 and mos.state_dict() == {}
    with pytest.raises(ValueError):
        SquimObjectiveMetric(16000, "mos")


def test_audio_utils_coherence_alignment_targets_covariance():
    import numpy as np

    from speech_b200.audio import utils as U

    rng = np.random.default_rng(0)
    pos = np.array([[0, 0, 0], [0.05, 0, 0], [0.2, 0, 0]], dtype=float)
    g = U.theoretical_coherence(pos, 16000, "spherical", 256)
    assert g.shape == (129, 3, 3) and np.allclose(g[:, 0, 0], 1) and np.allclose(g[0], 1) and abs(g[100, 0, 2]) < abs(g[100, 0, 1])
    assert U.theoretical_coherence(pos, 16000, "cylindrical", 256)[10, 0, 1] == pytest.approx(0.92, abs=0.01)          # J0(2 pi 625 Hz 0.05 m / c)
    noise = rng.standard_normal((64000, 3))
    field = U.generate_approximate_noise_field(pos, noise, 16000, "spherical", 256)
    S = torch.stft(torch.tensor(field.T), 256, 64, 256, torch.hann_window(256, dtype=torch.float64), return_complex=True).numpy().transpose(1, 2, 0)
    est = U.estimated_coherence(S)
    lo = slice(5, 40)
    assert np.abs(np.real(est[lo, 0, 1]) - g[lo, 0, 1]).mean() < 0.1 and np.abs(np.real(est[lo, 0, 2]) - g[lo, 0, 2]).mean() < 0.12
    with pytest.raises(RuntimeError):
        U.transform_to_match_coherence(np.stack([noise[:, 0]] * 3, 1), g, fft_length=256)
    x = rng.standard_normal(4000)
    assert U.get_segment_start(x, x[1234:1800]) == 1234
    h = np.array([1.0, 0.5, -0.25])
    M = U.convmtx_numpy(x[:50], 3)
    assert np.allclose(M @ h, np.convolve(x[:50], h)[:50]) and np.allclose(U.convmtx_numpy(x[:50], 3, delay=2)[2:] @ h, (M @ h)[:-2])
    assert U.convmtx_mc_numpy(np.stack([x[:50], x[50:100]], 1), 3).shape == (50, 6)
    filtered = np.convolve(x, [0.8, 0.3, 0.1])[:4000]
    assert U.calculate_sdr_numpy(filtered, x) < 12 and U.calculate_sdr_numpy(filtered, x, convolution_invariant=True, convolution_filter_length=8) > 40
    assert U.calculate_sdr_numpy(3 * x, x, scale_invariant=True) > 60 and U.calculate_sdr_numpy(3 * x, x) < 0
    assert U.calculate_sdr_numpy(x, x, sdr_max=20) == pytest.approx(20.0, abs=0.01)
    assert float(U.mag2db(10.0)) == pytest.approx(20.0) and float(U.db2mag(-20.0)) == pytest.approx(0.1) and float(U.pow2db(100.0)) == pytest.approx(20.0)
    t = U.toeplitz(torch.tensor([1.0 + 0j, 2 + 1j, 3 - 1j]))
    assert t[1, 0] == 2 + 1j and t[0, 1] == 2 - 1j and t[2, 0] == 3 - 1j and torch.allclose(t, t.conj().T)
    X = torch.randn(2, 3, 5, 40, dtype=torch.complex64)
    C = U.covariance_matrix(X)
    assert C.shape == (2, 5, 3, 3) and torch.allclose(C, C.conj().transpose(-1, -2), atol=1e-5)
    m = torch.zeros(2, 5, 40)
    m[..., :10] = 1
    assert torch.allclose(U.covariance_matrix(X, m), U.covariance_matrix(X[..., :10]), atol=1e-5)
    assert torch.allclose(U.wrap_to_pi(torch.tensor([3.5, -3.5, 0.5])), torch.tensor([3.5 - 2 * math.pi, -3.5 + 2 * math.pi, 0.5]), atol=1e-6)


def test_array_geometry_and_room_mix_generator(tmp_path):
    import json

    import numpy as np

    from speech_b200.audio.simulation import ArrayGeometry, RIRMixGenerator, calculate_drr, convolve_rir, scaled_disturbance, simultaneously_active_rms, wrap_to_180
    from speech_b200.audio.utils import rms

    arr = ArrayGeometry([[-0.05, 0, 0], [0.05, 0, 0], [0, 0.05, 0]])
    assert arr.num_mics == 3 and arr.radius == pytest.approx(np.hypot(0.05, 1 / 60), abs=1e-6)
    moved = arr.translate([2, 3, 1.5]).rotate(yaw=90)
    assert np.allclose(moved.centroid, [2, 3, 1.5]) and np.allclose(moved.positions[1] - moved.positions[0], [0, 0.1, 0], atol=1e-9)
    p = moved.new_point(1.0, 0.0, 0.0)                                  # "straight ahead" of an array turned by 90 degrees is +y
    assert np.allclose(p, [2, 4, 1.5], atol=1e-9)
    r, az, el = moved.spherical_relative_to_array([2, 3, 2.5])
    assert (r, el) == (pytest.approx(1.0), pytest.approx(90.0)) and wrap_to_180(270) == -90.0
    rir = np.zeros((1, 400))
    rir[0, 20], rir[0, 200] = 1.0, 0.1
    assert calculate_drr(rir, 16000)[0] == pytest.approx(20.0, abs=0.1)
    sig = np.random.default_rng(0).standard_normal(2000)
    assert np.allclose(convolve_rir(sig, rir)[:, 0], np.convolve(sig, rir[0])[:2000], atol=1e-9)
    d = scaled_disturbance(sig, 5 * np.random.default_rng(1).standard_normal(2000), 10.0)
    assert 20 * np.log10(rms(sig) / rms(d)) == pytest.approx(10.0, abs=1e-6)
    gated = sig.copy()
    gated[1000:] = 0
    a, b = simultaneously_active_rms(gated, sig, 1000, window_len_ms=100)
    assert a == pytest.approx(rms(sig[:1000]), rel=1e-6) and b == pytest.approx(rms(sig[:1000]), rel=1e-6)
    rng = np.random.default_rng(2)
    gen = RIRMixGenerator(arr, room_dim_range=((4, 5), (4, 5), (2.5, 3)), rt60_range=(0.2, 0.3), num_interferers=(1, 1), rsnr_range=(10, 10), rsir_range=(5, 5),
                          sample_rate=8000, max_order=3, seed=3)
    speech = lambda: (rng.standard_normal(8000) * (np.sin(np.arange(8000) / 400) > 0)).astype(np.float64)  # noqa: E731
    out = gen.mix(speech(), [speech()], rng.standard_normal(8000))
    assert out["mix"].shape == (8000, 3) and set(out) >= {"mix", "target_reverberant", "target_anechoic", "interference", "noise", "metadata"}
    assert np.allclose(out["mix"], out["target_reverberant"] + out["interference"] + out["noise"], atol=1e-9)
    assert 20 * np.log10(rms(out["target_reverberant"][:, 0]) / rms(out["noise"][:, 0])) == pytest.approx(10.0, abs=1e-6)
    md = out["metadata"]
    assert 0.5 <= md["target_range"] <= 2.5 and md["num_interferers"] == 1 and rms(out["target_anechoic"]) < rms(out["target_reverberant"])
    man = gen.generate(str(tmp_path / "sim"), [speech(), speech()], [speech()], [rng.standard_normal(8000)])
    rows = [json.loads(l) for l in open(man)]
    assert len(rows) == 2 and os.path.exists(rows[1]["mix_filepath"]) and rows[0]["duration"] == 1.0


def test_audio_losses_and_time_domain_denoiser():
    from speech_b200.audio.losses import CombinedLoss, MAELoss, MSELoss, temporal_mean
    from speech_b200.audio.models import BNR2

    torch.manual_seed(0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 100.0]], [[2.0, 2.0, 2.0, 2.0]]])
    assert temporal_mean(x, torch.tensor([3, 4])).flatten().tolist() == pytest.approx([2.0, 2.0])
    est, tgt = torch.zeros(2, 2, 4), torch.ones(2, 2, 4)
    tgt[:, 1] = 3.0
    assert float(MSELoss()(est, tgt)) == pytest.approx(5.0) and float(MAELoss()(est, tgt)) == pytest.approx(2.0)
    assert float(MSELoss(weight=[0.75, 0.25])(est, tgt)) == pytest.approx(3.0)
    e2 = est.clone()
    e2[0, :, 2:] = 50.0
    assert float(MAELoss()(e2, tgt, input_length=torch.tensor([2, 4]))) == pytest.approx(2.0)         # the corrupted tail lies beyond the length
    spec_e, spec_t = torch.zeros(1, 1, 3, 5, dtype=torch.complex64), torch.full((1, 1, 3, 5), 1 + 1j)
    assert float(MSELoss(ndim=4)(spec_e, spec_t)) == pytest.approx(2.0)
    with pytest.raises(ValueError):
        MSELoss(weight=[0.5, 0.6])
    feats = torch.nn.Conv1d(1, 4, 64, stride=32)
    for p_ in feats.parameters():
        p_.requires_grad_(False)
    cl = CombinedLoss(16000, fft_length=256, hop_length=64, num_mels=20, feature_extractor=lambda a, l: feats(a.unsqueeze(1)))
    clean = torch.sin(torch.arange(4000) * 0.05)[None].repeat(2, 1)
    noisy = (clean + 0.3 * torch.randn(2, 4000)).requires_grad_(True)
    l_noisy, l_clean = cl(noisy, clean), cl(clean + 1e-4 * torch.randn(2, 4000), clean)
    assert float(l_clean) < float(l_noisy)
    l_noisy.backward()
    assert noisy.grad.abs().sum() > 0
    m = BNR2(OmegaConf.create({"sample_rate": 16000, "seasr": {"hidden_nodes": 8, "kernel_size": 64, "f1": 32, "f2": 16, "stride": 32},
                               "loss": {"fft_length": 256, "hop_length": 64, "num_mels": 20, "asr_loss_weight": 0.0}}))
    lens = torch.tensor([4000, 3000])
    out, _ = m(noisy.detach().unsqueeze(1), lens)
    assert out.shape == (2, 1, 4000) and float(out[1, :, 3000:].abs().sum()) == 0.0 and float(out.abs().max()) <= 1.0
    loss = m.training_step((noisy.detach().unsqueeze(1), lens, clean.unsqueeze(1), lens), 0)["loss"]
    loss.backward()
    assert torch.isfinite(loss) and m.seasr.analysis.weight.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        BNR2(OmegaConf.create({"sample_rate": 8000}))


def test_multi_signal_audio_datasets_sync_async_embedding_and_channel_selection(tmp_path):
    import json

    import numpy as np
    import torch

    from speech_b200.audio import data_extra as D
    from speech_b200.data.audio_to_text import save_wav

    sr = 8000
    t = np.arange(sr * 2) / sr
    clean = (0.5 * np.sin(2 * np.pi * 5 * t)).astype(np.float32)               # slow sine: sample index is recoverable from the phase
    noisy2 = np.stack([clean * 0.5, -clean * 0.5], axis=1).astype(np.float32)  # two channels
    from scipy.io import wavfile

    wavfile.write(str(tmp_path / "noisy.wav"), sr, noisy2)
    save_wav(str(tmp_path / "clean.wav"), clean, sr)
    save_wav(str(tmp_path / "extra.wav"), clean * 0.25, sr)
    save_wav(str(tmp_path / "ref.wav"), np.linspace(-0.5, 0.5, sr * 3).astype(np.float32), sr)
    np.save(tmp_path / "emb.npy", np.arange(6, dtype=np.float32))
    man = tmp_path / "m.json"
    rows = [{"noisy": "noisy.wav", "clean": "clean.wav", "both": ["clean.wav", "extra.wav"], "ref": "ref.wav", "emb": "emb.npy", "duration": 2.0},
            {"noisy": "noisy.wav", "clean": "clean.wav", "both": ["clean.wav", "extra.wav"], "ref": "ref.wav", "emb": "emb.npy", "duration": 2.0, "offset": 0.5}]
    man.write_text("".join(json.dumps(r) + "\n" for r in rows))

    ds = D.AudioToTargetDataset(str(man), sr, "noisy", "clean")
    ex = ds[0]
    assert ex["input_signal"].shape == (2, 2 * sr) and ex["target_signal"].shape == (1, 2 * sr) and ds.num_channels("input_signal") == 2
    assert torch.allclose(ex["input_signal"][0] * 2, ex["target_signal"][0], atol=1e-3)
    sel = D.AudioToTargetDataset(str(man), sr, "noisy", "both", input_channel_selector=1, target_channel_selector="average", normalization_signal="input_signal")[0]
    assert sel["input_signal"].shape == (1, 2 * sr) and float(sel["input_signal"].abs().max()) == pytest.approx(1.0, abs=1e-3)
    assert torch.allclose(sel["target_signal"][0], -sel["input_signal"][0] * (0.625 / 0.5), atol=1e-2)           # mean of (1, 0.25) × clean vs −0.5 × clean, same scale

    rnd = D.AudioToTargetDataset(str(man), sr, "noisy", "clean", audio_duration=0.5, random_offset=True, seed=3)
    a, b = rnd[0], rnd[0]
    assert a["input_signal"].shape == (2, sr // 2) and torch.allclose(a["input_signal"][0] * 2, a["target_signal"][0], atol=1e-3)     # input and target stay aligned
    assert not torch.equal(a["target_signal"], b["target_signal"])                                                                 # a new segment each time
    fixed = D.AudioToTargetDataset(str(man), sr, "noisy", "clean", audio_duration=0.25)[1]
    assert torch.allclose(fixed["target_signal"][0], torch.from_numpy(clean[sr // 2: sr // 2 + sr // 4]), atol=1e-3)                # the manifest offset

    batch = ds.collate_fn([ds[0], rnd[0]])
    assert batch.input_signal.shape == (2, 2, 2 * sr) and batch.input_length.tolist() == [2 * sr, sr // 2] and batch.target_signal.shape == (2, 1, 2 * sr)

    ref = D.AudioToTargetWithReferenceDataset(str(man), sr, "noisy", "clean", "ref", reference_is_synchronized=False, reference_duration=1.0, seed=1)
    r = ref[0]
    assert r["reference_signal"].shape == (1, sr) and r["input_signal"].shape == (2, 2 * sr)
    ramp = r["reference_signal"][0]
    assert float(ramp[1000] - ramp[0]) == pytest.approx(1000.0 / (3 * sr), rel=0.01) and float(ramp[0]) > -0.5                            # a random stretch of the ramp
    rb = ref.collate_fn([ref[0], ref[1]])
    assert rb.reference_signal.shape == (2, 1, sr) and rb.reference_length.tolist() == [sr, sr]
    sync = D.get_audio_dataset_from_config({"manifest_filepath": str(man), "sample_rate": sr, "input_key": "noisy", "target_key": "clean", "reference_key": "clean",
                                            "audio_duration": 0.5, "random_offset": True})
    s0 = sync[0]
    assert isinstance(sync, D.AudioToTargetWithReferenceDataset) and torch.equal(s0["reference_signal"], s0["target_signal"])

    emb = D.get_audio_dataset_from_config({"manifest_filepath": str(man), "sample_rate": sr, "input_key": "noisy", "target_key": "clean", "embedding_key": "emb"})
    eb = emb.collate_fn([emb[0], emb[1]])
    assert eb.embedding_vector.shape == (2, 6) and eb.embedding_length.tolist() == [6, 6] and eb.embedding_vector[0].tolist() == [0, 1, 2, 3, 4, 5]
    assert D.get_audio_dataset_from_config({"manifest_filepath": None}) is None
    with pytest.raises(RuntimeError):
        D.ASRAudioProcessor.list_to_multichannel([np.zeros((10, 1)), np.zeros((12, 1))])


def test_audio_transforms_spectrogram_mel_db_mfcc_resample():
    import math

    import numpy as np
    import torch
    from scipy.signal import resample_poly

    from speech_b200.audio import transforms as T

    torch.manual_seed(0)
    sr = 16000
    t = torch.arange(sr) / sr
    x = torch.sin(2 * math.pi * 1000 * t)[None, :]
    spec = T.Spectrogram(n_fft=512, hop_length=128)(x)
    assert spec.shape == (1, 257, 126) and int(spec[0, :, 60].argmax()) == 32                        # 1 kHz → bin 1000 / (16000 / 512)
    cplx = T.Spectrogram(n_fft=512, hop_length=128, power=None)(x)
    assert cplx.is_complex() and torch.allclose(cplx.abs() ** 2, spec, rtol=1e-4, atol=1e-3)
    fb = T.melscale_fbanks(257, 0.0, 8000.0, 40, sr)
    assert fb.shape == (257, 40) and bool((fb >= 0).all()) and bool((fb.sum(0) > 0).all())
    peaks = fb.argmax(0)
    assert bool((peaks[1:] > peaks[:-1]).all())                                                        # centre frequencies increase
    slaney = T.melscale_fbanks(257, 0.0, 8000.0, 40, sr, norm="slaney", mel_scale="slaney")
    assert float(slaney[:, 0].max()) > float(slaney[:, -1].max())                                      # unit area: narrow low filters are taller
    mel = T.MelSpectrogram(sr, n_fft=512, hop_length=128, n_mels=40)(x)
    assert mel.shape == (1, 40, 126) and torch.allclose(mel, T.MelScale(40, sr, n_stft=257)(spec), atol=1e-4)
    db = T.AmplitudeToDB("power", top_db=60.0)(mel)
    assert float(db.max() - db.min()) <= 60.0 + 1e-4 and float(db.max()) == pytest.approx(10 * math.log10(float(mel.max())), abs=1e-3)
    assert torch.allclose(T.AmplitudeToDB("magnitude")(torch.tensor([[10.0, 1.0]])), torch.tensor([[20.0, 0.0]]))
    dct = T.create_dct(13, 40)
    assert torch.allclose(dct.t() @ dct, torch.eye(13), atol=1e-5)                                     # orthonormal rows
    mf = T.MFCC(sr, n_mfcc=13, melkwargs={"n_fft": 512, "hop_length": 128, "n_mels": 40})(x)
    assert mf.shape == (1, 13, 126)
    with pytest.raises(ValueError):
        T.MFCC(sr, n_mfcc=50, melkwargs={"n_mels": 40})

    sig = torch.sin(2 * math.pi * 440 * t) + 0.5 * torch.sin(2 * math.pi * 3000 * t)
    down = T.Resample(16000, 8000)(sig[None])
    ref = resample_poly(sig.numpy().astype(np.float64), 1, 2)
    assert down.shape == (1, 8000) and float((down[0, 200:-200] - torch.from_numpy(ref[200:-200]).float()).abs().max()) < 0.02
    sharp_down = T.Resample(16000, 8000, lowpass_filter_width=64)(sig[None])
    up = T.Resample(8000, 16000, resampling_method="sinc_interp_kaiser", lowpass_filter_width=64)(sharp_down)
    assert up.shape == (1, 16000) and float((up[0, 400:-400] - sig[400:-400]).abs().max()) < 0.03    # both tones are below 4 kHz: with sharp filters the round trip is near-lossless
    odd = T.Resample(16000, 22050)(sig[None, :1600])
    assert odd.shape == (1, 2205) and T.Resample(16000, 16000)(sig[None]) is not None
    batch = T.Resample(16000, 8000)(torch.stack([sig, -sig]).reshape(2, 1, -1))
    assert batch.shape == (2, 1, 8000) and torch.allclose(batch[0], -batch[1], atol=1e-6)

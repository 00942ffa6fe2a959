"""Waveform -> log-mel features.

``AudioToMelSpectrogramPreprocessor`` wraps ``FilterbankFeatures`` and always runs in fp32 under
``no_grad`` (reference: ``nemo/collections/asr/modules/audio_preprocessing.py:83-92,100-288``;
``parts/preprocessing/features.py:239-494``).  Buffers are named ``featurizer.window`` and
``featurizer.fb`` so reference checkpoints load.  On a GPU the whole pipeline (pre-emphasis,
framing, windowed FFT, power, mel projection, log, per-feature normalisation, masking) runs in
the hand-written ``logmel`` kernels; on the CPU it is ``torch.stft`` based.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..core.module import NeuralModule
from ..core.neural_types import AudioSignal, LengthsType, MelSpectrogramType, NeuralType, typecheck


def _hz_to_mel_slaney(f):
    f = np.asarray(f, dtype=np.float64)
    f_sp = 200.0 / 3
    mels = f / f_sp
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    return np.where(f >= min_log_hz, min_log_mel + np.log(np.maximum(f, 1e-10) / min_log_hz) / logstep, mels)


def _mel_to_hz_slaney(m):
    m = np.asarray(m, dtype=np.float64)
    f_sp = 200.0 / 3
    freqs = f_sp * m
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    return np.where(m >= min_log_mel, min_log_hz * np.exp(logstep * (m - min_log_mel)), freqs)


def mel_filterbank(sr: int, n_fft: int, n_mels: int, fmin: float = 0.0, fmax: Optional[float] = None,
                   norm: Optional[str] = "slaney", htk: bool = False) -> np.ndarray:
    """Triangular mel filterbank [n_mels, n_fft//2+1]; Slaney scale and area normalisation by default."""
    fmax = fmax if fmax is not None else sr / 2
    fft_freqs = np.linspace(0, sr / 2, n_fft // 2 + 1)
    if htk:
        mel_pts = np.linspace(2595.0 * np.log10(1 + fmin / 700.0), 2595.0 * np.log10(1 + fmax / 700.0), n_mels + 2)
        mel_f = 700.0 * (10.0 ** (mel_pts / 2595.0) - 1.0)
    else:
        mel_f = _mel_to_hz_slaney(np.linspace(_hz_to_mel_slaney(fmin), _hz_to_mel_slaney(fmax), n_mels + 2))
    fdiff = np.diff(mel_f)
    ramps = mel_f[:, None] - fft_freqs[None, :]
    weights = np.zeros((n_mels, n_fft // 2 + 1), dtype=np.float64)
    for i in range(n_mels):
        lower = -ramps[i] / fdiff[i]
        upper = ramps[i + 2] / fdiff[i + 1]
        weights[i] = np.maximum(0, np.minimum(lower, upper))
    if norm == "slaney":
        enorm = 2.0 / (mel_f[2: n_mels + 2] - mel_f[:n_mels])
        weights *= enorm[:, None]
    return weights.astype(np.float32)


class FilterbankFeatures(torch.nn.Module):
    def __init__(self, sample_rate=16000, n_window_size=320, n_window_stride=160, window="hann", normalize="per_feature",
                 n_fft=None, preemph=0.97, nfilt=64, lowfreq=0, highfreq=None, log=True, log_zero_guard_type="add",
                 log_zero_guard_value=2 ** -24, dither=1e-5, pad_to=16, max_duration=16.7, frame_splicing=1,
                 exact_pad=False, pad_value=0, mag_power=2.0, use_grads=False, rng=None, nb_augmentation_prob=0.0,
                 nb_max_freq=4000, mel_norm="slaney", stft_exact_pad=False, stft_conv=False):
        super().__init__()
        if exact_pad and n_window_stride % 2 == 1:
            raise NotImplementedError(f"{self} received exact_pad == True, but hop_size was odd.")
        self.log_zero_guard_value = log_zero_guard_value
        if n_window_size is None or n_window_stride is None or n_window_size <= 0 or n_window_stride <= 0:
            raise ValueError(f"{self} got an invalid value for either n_window_size or n_window_stride.")
        self.sample_rate = sample_rate
        self.win_length = n_window_size
        self.hop_length = n_window_stride
        self.n_fft = n_fft or 2 ** math.ceil(math.log2(self.win_length))
        self.stft_pad_amount = (self.n_fft - self.hop_length) // 2 if exact_pad else None
        self.exact_pad = exact_pad
        win_fn = {"hann": torch.hann_window, "hamming": torch.hamming_window, "blackman": torch.blackman_window,
                  "bartlett": torch.bartlett_window, "none": None, None: None}[window]
        w = win_fn(self.win_length, periodic=False) if win_fn else torch.ones(self.win_length)
        self.register_buffer("window", w)
        self.normalize = normalize
        self.log = log
        self.dither = dither
        self.frame_splicing = frame_splicing
        self.nfilt = nfilt
        self.preemph = preemph
        self.pad_to = pad_to
        highfreq = highfreq or sample_rate / 2
        fb = torch.tensor(mel_filterbank(sample_rate, self.n_fft, nfilt, lowfreq, highfreq, norm=mel_norm)).unsqueeze(0)
        self.register_buffer("fb", fb)
        max_length = self.get_seq_len(torch.tensor(max_duration * sample_rate, dtype=torch.float))
        max_pad = pad_to - (max_length % pad_to) if pad_to > 0 else 0
        self.max_length = max_length + max_pad
        self.pad_value = pad_value
        self.mag_power = mag_power
        if log_zero_guard_type not in ("add", "clamp"):
            raise ValueError("log_zero_guard_type must be 'add' or 'clamp'")
        self.log_zero_guard_type = log_zero_guard_type
        self.use_grads = use_grads

    def log_zero_guard_value_fn(self, x):
        v = self.log_zero_guard_value
        if isinstance(v, str):
            return {"tiny": torch.finfo(x.dtype).tiny, "eps": torch.finfo(x.dtype).eps}[v]
        return v

    def get_seq_len(self, seq_len):
        pad_amount = self.stft_pad_amount * 2 if self.stft_pad_amount is not None else self.n_fft // 2 * 2
        return torch.floor_divide((seq_len + pad_amount - self.n_fft), self.hop_length).to(dtype=torch.long)

    @property
    def filter_banks(self):
        return self.fb

    def forward(self, x, seq_len, linear_spec: bool = False):
        ctx = torch.enable_grad() if self.use_grads else torch.no_grad()
        with ctx, torch.autocast(x.device.type, enabled=False):
            dither = self.dither if self.training else 0.0
            mel, out_len = ops.logmel(
                x.float(), seq_len, self.window, self.fb[0], self.n_fft, self.hop_length, self.win_length,
                preemph=self.preemph or 0.0, mag_power=self.mag_power, log_zero_guard=float(self.log_zero_guard_value_fn(x)),
                normalize=self.normalize, pad_to=self.pad_to, pad_value=float(self.pad_value), dither=dither, log=self.log)
        return mel, out_len


class AudioToMelSpectrogramPreprocessor(NeuralModule):
    def __init__(self, sample_rate=16000, window_size=0.02, window_stride=0.01, n_window_size=None, n_window_stride=None,
                 window="hann", normalize="per_feature", n_fft=None, preemph=0.97, features=64, lowfreq=0, highfreq=None,
                 log=True, log_zero_guard_type="add", log_zero_guard_value=2 ** -24, dither=1e-5, pad_to=16,
                 frame_splicing=1, exact_pad=False, pad_value=0, mag_power=2.0, rng=None, nb_augmentation_prob=0.0,
                 nb_max_freq=4000, use_torchaudio: bool = False, mel_norm="slaney", stft_exact_pad=False, stft_conv=False):
        super().__init__()
        self._sample_rate = sample_rate
        if window_size and n_window_size:
            raise ValueError(f"{self} received both window_size and n_window_size. Only one should be specified.")
        if window_stride and n_window_stride:
            raise ValueError(f"{self} received both window_stride and n_window_stride. Only one should be specified.")
        if window_size:
            n_window_size = int(window_size * sample_rate)
        if window_stride:
            n_window_stride = int(window_stride * sample_rate)
        self.win_length, self.hop_length = n_window_size, n_window_stride
        self.featurizer = FilterbankFeatures(
            sample_rate=sample_rate, n_window_size=n_window_size, n_window_stride=n_window_stride, window=window,
            normalize=normalize, n_fft=n_fft, preemph=preemph, nfilt=features, lowfreq=lowfreq, highfreq=highfreq, log=log,
            log_zero_guard_type=log_zero_guard_type, log_zero_guard_value=log_zero_guard_value, dither=dither,
            pad_to=pad_to, frame_splicing=frame_splicing, exact_pad=exact_pad, pad_value=pad_value, mag_power=mag_power,
            mel_norm=mel_norm)

    @property
    def input_types(self):
        return {"input_signal": NeuralType(("B", "T"), AudioSignal(freq=self._sample_rate)),
                "length": NeuralType(("B",), LengthsType())}

    @property
    def output_types(self):
        return {"processed_signal": NeuralType(("B", "D", "T"), MelSpectrogramType()),
                "processed_length": NeuralType(("B",), LengthsType())}

    @typecheck()
    @torch.no_grad()
    def forward(self, input_signal, length):
        if input_signal.dtype != torch.float32:
            input_signal = input_signal.float()
        return self.featurizer(input_signal, length)

    def get_features(self, input_signal, length):
        return self.featurizer(input_signal, length)

    @property
    def filter_banks(self):
        return self.featurizer.filter_banks


class AudioToMFCCPreprocessor(NeuralModule):
    """MFCC features: log-mel followed by an orthonormal DCT-II (reference: ``audio_preprocessing.py:291``)."""

    def __init__(self, sample_rate=16000, window_size=0.02, window_stride=0.01, n_window_size=None, n_window_stride=None,
                 window="hann", n_fft=None, lowfreq=0.0, highfreq=None, n_mels=64, n_mfcc=64, dct_type=2, norm="ortho",
                 log=True):
        super().__init__()
        self.mel = AudioToMelSpectrogramPreprocessor(sample_rate=sample_rate, window_size=window_size,
                                                     window_stride=window_stride, n_window_size=n_window_size,
                                                     n_window_stride=n_window_stride, window=window, normalize=None,
                                                     n_fft=n_fft, preemph=None, features=n_mels, lowfreq=lowfreq,
                                                     highfreq=highfreq, log=log, dither=0.0, pad_to=0)
        n = torch.arange(n_mels, dtype=torch.float32)
        k = torch.arange(n_mfcc, dtype=torch.float32).unsqueeze(1)
        dct = torch.cos(math.pi / n_mels * (n + 0.5) * k)
        if norm == "ortho":
            dct[0] *= 1.0 / math.sqrt(2.0)
            dct *= math.sqrt(2.0 / n_mels)
        self.register_buffer("dct", dct, persistent=False)

    def forward(self, input_signal, length):
        mel, ln = self.mel(input_signal=input_signal, length=length)
        return torch.matmul(self.dct.to(mel.dtype), mel), ln

"""Signal transforms as modules, with the interface of the torchaudio transforms they stand in for (torchaudio is not a dependency):
``Spectrogram``, ``MelScale``, ``MelSpectrogram``, ``AmplitudeToDB``, ``MFCC`` and a windowed-sinc polyphase ``Resample``.
Reference: ``audio/parts/utils/transforms.py``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch import nn


def _hz_to_mel(f: float, scale: str) -> float:
    if scale == "htk":
        return 2595.0 * math.log10(1.0 + f / 700.0)
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    return f / f_sp if f < min_log_hz else min_log_hz / f_sp + math.log(f / min_log_hz) / (math.log(6.4) / 27.0)


def _mel_to_hz(m: torch.Tensor, scale: str) -> torch.Tensor:
    if scale == "htk":
        return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel = min_log_hz / f_sp
    return torch.where(m >= min_log_mel, min_log_hz * torch.exp((math.log(6.4) / 27.0) * (m - min_log_mel)), f_sp * m)


def melscale_fbanks(n_freqs: int, f_min: float, f_max: float, n_mels: int, sample_rate: int, norm: Optional[str] = None, mel_scale: str = "htk") -> torch.Tensor:
    """Triangular filters ``[n_freqs, n_mels]``; ``norm='slaney'`` divides each by its bandwidth (unit area)."""
    if norm not in (None, "slaney"):
        raise ValueError("norm must be None or 'slaney'")
    freqs = torch.linspace(0, sample_rate // 2, n_freqs)
    pts = _mel_to_hz(torch.linspace(_hz_to_mel(f_min, mel_scale), _hz_to_mel(f_max, mel_scale), n_mels + 2), mel_scale)
    diff = pts[1:] - pts[:-1]
    slopes = pts[None, :] - freqs[:, None]
    fb = torch.clamp(torch.minimum(-slopes[:, :-2] / diff[:-1], slopes[:, 2:] / diff[1:]), min=0.0)
    if norm == "slaney":
        fb = fb * (2.0 / (pts[2:] - pts[:-2]))[None, :]
    return fb


class Spectrogram(nn.Module):
    """``[..., T]`` → ``[..., n_fft // 2 + 1, frames]``: magnitude ** ``power`` (``power=None`` keeps the complex STFT)."""

    def __init__(self, n_fft: int = 400, win_length: Optional[int] = None, hop_length: Optional[int] = None, pad: int = 0, window_fn: Callable = torch.hann_window,
                 power: Optional[float] = 2.0, normalized: bool = False, center: bool = True, pad_mode: str = "reflect", onesided: bool = True):
        super().__init__()
        self.n_fft, self.win_length = n_fft, win_length or n_fft
        self.hop_length = hop_length or self.win_length // 2
        self.pad, self.power, self.normalized, self.center, self.pad_mode, self.onesided = pad, power, normalized, center, pad_mode, onesided
        self.register_buffer("window", window_fn(self.win_length), persistent=False)

    def forward(self, waveform: torch.Tensor) -> torch.Tensor:
        if self.pad > 0:
            waveform = F.pad(waveform, (self.pad, self.pad))
        shape = waveform.shape
        s = torch.stft(waveform.reshape(-1, shape[-1]).float(), self.n_fft, self.hop_length, self.win_length, self.window.float(), center=self.center,
                       pad_mode=self.pad_mode, normalized=False, onesided=self.onesided, return_complex=True)
        s = s.reshape(shape[:-1] + s.shape[-2:])
        if self.normalized:
            s = s / self.window.float().pow(2).sum().sqrt()
        if self.power is None:
            return s
        return s.abs() if self.power == 1.0 else s.abs().pow(self.power)


class MelScale(nn.Module):
    """``[..., n_stft, frames]`` → ``[..., n_mels, frames]``."""

    def __init__(self, n_mels: int = 128, sample_rate: int = 16000, f_min: float = 0.0, f_max: Optional[float] = None, n_stft: int = 201,
                 norm: Optional[str] = None, mel_scale: str = "htk"):
        super().__init__()
        f_max = float(sample_rate // 2) if f_max is None else f_max
        if f_min > f_max:
            raise ValueError(f"f_min ({f_min}) above f_max ({f_max})")
        self.register_buffer("fb", melscale_fbanks(n_stft, f_min, f_max, n_mels, sample_rate, norm, mel_scale), persistent=False)

    def forward(self, specgram: torch.Tensor) -> torch.Tensor:
        return torch.matmul(specgram.transpose(-1, -2), self.fb.to(specgram.dtype)).transpose(-1, -2)


class MelSpectrogram(nn.Module):
    def __init__(self, sample_rate: int = 16000, n_fft: int = 400, win_length: Optional[int] = None, hop_length: Optional[int] = None, f_min: float = 0.0,
                 f_max: Optional[float] = None, pad: int = 0, n_mels: int = 128, window_fn: Callable = torch.hann_window, power: float = 2.0,
                 normalized: bool = False, center: bool = True, pad_mode: str = "reflect", norm: Optional[str] = None, mel_scale: str = "htk"):
        super().__init__()
        self.spectrogram = Spectrogram(n_fft, win_length, hop_length, pad, window_fn, power, normalized, center, pad_mode)
        self.mel_scale = MelScale(n_mels, sample_rate, f_min, f_max, n_fft // 2 + 1, norm, mel_scale)

    def forward(self, waveform: torch.Tensor) -> torch.Tensor:
        return self.mel_scale(self.spectrogram(waveform))


class AmplitudeToDB(nn.Module):
    """``10 log10`` for power, ``20 log10`` for magnitude input, floored at 1e-10; ``top_db`` clamps each spectrogram to that many dB below its peak."""

    def __init__(self, stype: str = "power", top_db: Optional[float] = None):
        super().__init__()
        if top_db is not None and top_db < 0:
            raise ValueError("top_db must be positive")
        if stype not in ("power", "magnitude"):
            raise ValueError("stype must be 'power' or 'magnitude'")
        self.multiplier, self.top_db, self.amin = (10.0 if stype == "power" else 20.0), top_db, 1e-10

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        db = self.multiplier * torch.log10(torch.clamp(x, min=self.amin))
        if self.top_db is not None:
            lead = db.shape[:-2] if db.dim() > 2 else ()
            peak = db.reshape(lead + (-1,)).amax(-1) if lead else db.max()
            floor = (peak - self.top_db).reshape(lead + (1, 1)) if lead else peak - self.top_db
            db = torch.maximum(db, floor)
        return db


def create_dct(n_mfcc: int, n_mels: int, norm: Optional[str] = "ortho") -> torch.Tensor:
    """DCT-II matrix ``[n_mels, n_mfcc]``."""
    n = torch.arange(n_mels, dtype=torch.float32)
    k = torch.arange(n_mfcc, dtype=torch.float32)[:, None]
    dct = torch.cos(math.pi / n_mels * (n + 0.5) * k)
    if norm is None:
        dct = dct * 2.0
    else:
        dct[0] *= 1.0 / math.sqrt(2.0)
        dct = dct * math.sqrt(2.0 / n_mels)
    return dct.t()


class MFCC(nn.Module):
    def __init__(self, sample_rate: int = 16000, n_mfcc: int = 40, dct_type: int = 2, norm: str = "ortho", log_mels: bool = False, melkwargs: Optional[dict] = None):
        super().__init__()
        if dct_type != 2:
            raise ValueError("only DCT type 2 is supported")
        self.mel = MelSpectrogram(sample_rate=sample_rate, **dict(melkwargs or {}))
        n_mels = self.mel.mel_scale.fb.shape[1]
        if n_mfcc > n_mels:
            raise ValueError("cannot select more MFCC coefficients than mel bins")
        self.register_buffer("dct_mat", create_dct(n_mfcc, n_mels, norm), persistent=False)
        self.log_mels, self.to_db = log_mels, AmplitudeToDB("power", 80.0)

    def forward(self, waveform: torch.Tensor) -> torch.Tensor:
        m = self.mel(waveform)
        m = torch.log(m + 1e-6) if self.log_mels else self.to_db(m)
        return torch.matmul(m.transpose(-1, -2), self.dct_mat).transpose(-1, -2)


class Resample(nn.Module):
    """Band-limited resampling by a rational factor: a bank of ``new / gcd`` windowed-sinc filters applied as one strided convolution
    (``lowpass_filter_width`` zero crossings, cut-off ``rolloff`` × the lower Nyquist frequency)."""

    def __init__(self, orig_freq: int = 16000, new_freq: int = 16000, resampling_method: str = "sinc_interp_hann", lowpass_filter_width: int = 6,
                 rolloff: float = 0.99, beta: Optional[float] = None, dtype: torch.dtype = torch.float32):
        super().__init__()
        if resampling_method not in ("sinc_interp_hann", "sinc_interp_kaiser"):
            raise ValueError("resampling_method must be sinc_interp_hann or sinc_interp_kaiser")
        g = math.gcd(int(orig_freq), int(new_freq))
        self.orig, self.new = int(orig_freq) // g, int(new_freq) // g
        if self.orig != self.new:
            base = min(self.orig, self.new) * rolloff
            width = math.ceil(lowpass_filter_width * self.orig / base)
            idx = torch.arange(-width, width + self.orig, dtype=torch.float64)[None, :] / self.orig
            t = (torch.arange(0, -self.new, -1, dtype=torch.float64)[:, None] / self.new + idx) * base
            t = t.clamp(-lowpass_filter_width, lowpass_filter_width)
            if resampling_method == "sinc_interp_hann":
                window = torch.cos(t * math.pi / lowpass_filter_width / 2) ** 2
            else:
                beta = 14.769656459379492 if beta is None else beta
                window = torch.i0(beta * torch.sqrt(1 - (t / lowpass_filter_width) ** 2)) / torch.i0(torch.tensor(float(beta), dtype=torch.float64))
            t = t * math.pi
            kernel = torch.where(t == 0, torch.ones_like(t), torch.sin(t) / t) * window * (base / self.orig)
            self.register_buffer("kernel", kernel.to(dtype)[:, None, :], persistent=False)
            self.width = width

    def forward(self, waveform: torch.Tensor) -> torch.Tensor:
        if self.orig == self.new:
            return waveform
        shape = waveform.shape
        x = F.pad(waveform.reshape(-1, 1, shape[-1]).to(self.kernel.dtype), (self.width, self.width + self.orig))
        y = F.conv1d(x, self.kernel, stride=self.orig)                       # [N, new, frames]
        y = y.transpose(1, 2).reshape(y.shape[0], -1)
        n = math.ceil(self.new * shape[-1] / self.orig)
        return y[:, :n].reshape(shape[:-1] + (n,)).to(waveform.dtype)

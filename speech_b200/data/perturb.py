"""Waveform container and on-the-fly waveform perturbations for training-data augmentation.

``AudioSegment`` holds float32 samples with their rate and does loading (whole file or a window), channel selection,
resampling, gain and padding.  Perturbations change a segment in place and are composed by ``AudioAugmentor``, which applies
each with its own probability; ``process_augmentations`` builds the augmentor from the ``augmentor:`` block of a dataset config.

Reference: ``asr/parts/preprocessing/segment.py`` (``AudioSegment.from_file`` / ``segment_from_file``, ``gain_db``, ``pad``,
``subsegment``), ``asr/parts/preprocessing/perturb.py`` (speed, time-stretch, gain, impulse response, shift, noise with SNR
range and optional foreground-duration limit, white noise, RIR + noise, codec transcoding, silence; ``perturbation_types``,
``AudioAugmentor``, ``process_augmentations``).
"""
from __future__ import annotations

import json
import math
import random
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


def resample(x: np.ndarray, orig_sr: int, target_sr: int) -> np.ndarray:
    """Band-limited (windowed-sinc polyphase) resampling."""
    if orig_sr == target_sr or x.size == 0:
        return x.astype(np.float32)
    from scipy.signal import resample_poly

    g = math.gcd(int(orig_sr), int(target_sr))
    return resample_poly(x, int(target_sr) // g, int(orig_sr) // g, axis=0).astype(np.float32)


class AudioSegment:
    def __init__(self, samples, sample_rate: int, target_sr: Optional[int] = None, trim: bool = False, trim_db: float = 60.0,
                 orig_sr: Optional[int] = None, channel_selector=None, offset: float = 0.0, audio_file: Optional[str] = None):
        s = np.asarray(samples)
        if np.issubdtype(s.dtype, np.integer):
            s = s.astype(np.float32) / float(1 << (8 * s.dtype.itemsize - 1))
        s = s.astype(np.float32)
        if s.ndim == 2:
            if channel_selector in (None, "average"):
                s = s.mean(axis=1) if channel_selector == "average" or s.shape[1] == 1 else s
            elif isinstance(channel_selector, int):
                s = s[:, channel_selector]
            else:
                s = s[:, list(channel_selector)]
        if target_sr is not None and target_sr != sample_rate:
            s = resample(s, sample_rate, target_sr)
            sample_rate = target_sr
        if trim and s.ndim == 1 and s.size:
            thr = np.abs(s).max() * 10 ** (-trim_db / 20.0)
            idx = np.nonzero(np.abs(s) > thr)[0]
            if idx.size:
                s = s[idx[0]: idx[-1] + 1]
        self._samples, self._sample_rate = s, sample_rate
        self._orig_sr = orig_sr if orig_sr is not None else sample_rate
        self.offset, self.audio_file = offset, audio_file

    @classmethod
    def from_file(cls, audio_file, target_sr=None, int_values=False, offset: float = 0.0, duration: float = 0.0, trim=False, trim_db=60,
                  channel_selector=None, **_):
        from .audio_to_text import load_audio_file

        x, sr = load_audio_file(audio_file)
        a = int(offset * sr)
        b = a + int(duration * sr) if duration and duration > 0 else x.shape[0]
        return cls(x[a:b], sr, target_sr=target_sr, trim=trim, trim_db=trim_db, orig_sr=sr, channel_selector=channel_selector, offset=offset,
                   audio_file=audio_file if isinstance(audio_file, str) else None)

    @classmethod
    def segment_from_file(cls, audio_file, target_sr=None, n_segments: int = 0, trim=False, channel_selector=None, offset=None, **_):
        """A random (or ``offset``-positioned) window of ``n_segments`` samples (at the target rate), zero padded if short."""
        seg = cls.from_file(audio_file, target_sr=target_sr, trim=trim, channel_selector=channel_selector)
        n = seg.num_samples
        if n_segments > 0:
            if n > n_segments:
                start = random.randint(0, n - n_segments) if offset is None else int(offset * seg.sample_rate)
                seg._samples = seg._samples[start:start + n_segments]
            elif n < n_segments:
                seg.pad(n_segments - n, symmetric=False)
        return seg

    samples = property(lambda self: self._samples.copy())
    sample_rate = property(lambda self: self._sample_rate)
    num_samples = property(lambda self: self._samples.shape[0])
    num_channels = property(lambda self: 1 if self._samples.ndim == 1 else self._samples.shape[1])
    duration = property(lambda self: self._samples.shape[0] / float(self._sample_rate))
    orig_sr = property(lambda self: self._orig_sr)

    @property
    def rms_db(self) -> float:
        return 10.0 * math.log10(max(float(np.mean(self._samples ** 2)), 1e-20))

    def gain_db(self, gain: float) -> None:
        self._samples = self._samples * (10.0 ** (gain / 20.0))

    def pad(self, pad_size: int, symmetric: bool = False) -> None:
        w = ((pad_size, pad_size) if symmetric else (0, pad_size),) + ((0, 0),) * (self._samples.ndim - 1)
        self._samples = np.pad(self._samples, w)

    def subsegment(self, start_time: Optional[float] = None, end_time: Optional[float] = None) -> None:
        a = 0.0 if start_time is None else start_time
        b = self.duration if end_time is None else end_time
        if a < 0:
            a += self.duration
        if b < 0:
            b += self.duration
        if not 0 <= a <= b <= self.duration + 1e-9:
            raise ValueError(f"The slice ({a}, {b}) is out of bounds for a segment of {self.duration} s")
        self._samples = self._samples[int(round(a * self._sample_rate)): int(round(b * self._sample_rate))]


# ---------------------------------------------------------------------------------------------- perturbations
class Perturbation:
    def max_augmentation_length(self, length: int) -> int:
        return length

    def perturb(self, data: AudioSegment) -> None:
        raise NotImplementedError


class SpeedPerturbation(Perturbation):
    """Resample by a random factor (changes both tempo and pitch); ``num_rates`` > 0 draws from a fixed grid."""

    def __init__(self, sr: int = 16000, resample_type: str = "kaiser_fast", min_speed_rate: float = 0.9, max_speed_rate: float = 1.1,
                 num_rates: int = 5, rng=None):
        if min_speed_rate <= 0:
            raise ValueError("Sampling speed below 0 is not possible")
        self._rates = list(np.linspace(min_speed_rate, max_speed_rate, num_rates)) if num_rates > 0 else None
        self._min, self._max, self._rng = min_speed_rate, max_speed_rate, random.Random(rng)

    def max_augmentation_length(self, length):
        return int(math.ceil(length / self._min))

    def perturb(self, data):
        rate = self._rng.choice(self._rates) if self._rates else self._rng.uniform(self._min, self._max)
        if abs(rate - 1.0) < 1e-6:
            return
        data._samples = resample(data._samples, int(round(data.sample_rate * rate * 1000)), data.sample_rate * 1000)


class TimeStretchPerturbation(Perturbation):
    """Tempo change at constant pitch by a phase vocoder."""

    def __init__(self, min_speed_rate: float = 0.9, max_speed_rate: float = 1.1, num_rates: int = 5, n_fft: int = 512, rng=None):
        self._rates = list(np.linspace(min_speed_rate, max_speed_rate, num_rates)) if num_rates > 0 else None
        self._min, self._max, self._n_fft, self._rng = min_speed_rate, max_speed_rate, n_fft, random.Random(rng)

    def max_augmentation_length(self, length):
        return int(math.ceil(length / self._min))

    def perturb(self, data):
        rate = self._rng.choice(self._rates) if self._rates else self._rng.uniform(self._min, self._max)
        if abs(rate - 1.0) < 1e-6 or data.num_samples < self._n_fft:
            return
        n_fft, hop = self._n_fft, self._n_fft // 4
        x = torch.from_numpy(data._samples)
        win = torch.hann_window(n_fft)
        S = torch.stft(x, n_fft, hop, window=win, return_complex=True)                     # [F, T]
        steps = torch.arange(0, S.shape[1] - 1, rate)
        i0 = steps.floor().long()
        frac = (steps - i0).unsqueeze(0)
        mag = (1 - frac) * S[:, i0].abs() + frac * S[:, i0 + 1].abs()
        dphi = torch.angle(S[:, i0 + 1]) - torch.angle(S[:, i0])
        omega = torch.linspace(0, math.pi * hop, S.shape[0]).unsqueeze(1)
        dphi = dphi - omega
        dphi = dphi - 2 * math.pi * torch.round(dphi / (2 * math.pi)) + omega
        phase = torch.cat([torch.angle(S[:, :1]), torch.angle(S[:, :1]) + torch.cumsum(dphi, dim=1)[:, :-1]], dim=1)
        y = torch.istft(torch.polar(mag, phase), n_fft, hop, window=win)
        data._samples = y.numpy().astype(np.float32)


class GainPerturbation(Perturbation):
    def __init__(self, min_gain_dbfs: float = -10, max_gain_dbfs: float = 10, rng=None):
        self._min, self._max, self._rng = min_gain_dbfs, max_gain_dbfs, random.Random(rng)

    def perturb(self, data):
        data.gain_db(self._rng.uniform(self._min, self._max))


class ShiftPerturbation(Perturbation):
    def __init__(self, min_shift_ms: float = -5.0, max_shift_ms: float = 5.0, rng=None):
        self._min, self._max, self._rng = min_shift_ms, max_shift_ms, random.Random(rng)

    def perturb(self, data):
        n = int(self._rng.uniform(self._min, self._max) * data.sample_rate / 1000)
        if abs(n) >= data.num_samples or n == 0:
            return
        s = data._samples
        data._samples = np.concatenate([np.zeros(n, np.float32), s[:-n]]) if n > 0 else np.concatenate([s[-n:], np.zeros(-n, np.float32)])


class WhiteNoisePerturbation(Perturbation):
    def __init__(self, min_level: float = -90, max_level: float = -46, rng=None):
        self.min_level, self.max_level = int(min_level), int(max_level)
        self._rng = np.random.RandomState(rng) if rng is not None else np.random.mtrand._rand

    def perturb(self, data):
        level = self._rng.randint(self.min_level, self.max_level, dtype="int32")
        data._samples = data._samples + self._rng.randn(data.num_samples).astype(np.float32) * (10.0 ** (level / 20.0))


def _read_manifest_items(path) -> List[Dict[str, Any]]:
    paths = path.split(",") if isinstance(path, str) else list(path)
    items = []
    for p in paths:
        with open(p, encoding="utf-8") as f:
            items += [json.loads(l) for l in f if l.strip()]
    return items


class NoisePerturbation(Perturbation):
    """Adds a random excerpt of a noise recording at a random SNR in ``[min_snr_db, max_snr_db]`` (full overlap; the noise is
    tiled when shorter than the utterance)."""

    def __init__(self, manifest_path=None, min_snr_db: float = 10, max_snr_db: float = 50, max_gain_db: float = 300.0, rng=None,
                 audio_tar_filepaths=None, shuffle_n=100, orig_sr: int = 16000, noise_items: Optional[Sequence[Dict[str, Any]]] = None):
        self._items = list(noise_items) if noise_items is not None else _read_manifest_items(manifest_path)
        self._min, self._max, self._max_gain, self._rng = min_snr_db, max_snr_db, max_gain_db, random.Random(rng)

    def get_one_noise_sample(self, target_sr: int) -> AudioSegment:
        it = self._rng.choice(self._items)
        if "samples" in it:
            return AudioSegment(it["samples"], it.get("sample_rate", target_sr), target_sr=target_sr)
        return AudioSegment.from_file(it["audio_filepath"], target_sr=target_sr, offset=it.get("offset", 0.0) or 0.0, duration=it.get("duration", 0.0) or 0.0)

    def perturb(self, data, ref_mic: int = 0):
        self.perturb_with_input_noise(data, self.get_one_noise_sample(data.sample_rate))

    def perturb_with_input_noise(self, data, noise: AudioSegment, data_rms: Optional[float] = None):
        snr = self._rng.uniform(self._min, self._max)
        gain = min((data.rms_db if data_rms is None else data_rms) - noise.rms_db - snr, self._max_gain)
        n = noise._samples
        if n.shape[0] == 0:
            return
        if n.shape[0] < data.num_samples:
            n = np.tile(n, int(math.ceil(data.num_samples / n.shape[0])))
        start = self._rng.randint(0, n.shape[0] - data.num_samples)
        data._samples = data._samples + n[start:start + data.num_samples] * (10.0 ** (gain / 20.0))


class ImpulsePerturbation(Perturbation):
    """Convolves with a room impulse response (peak-normalised, optionally aligned so the direct path keeps its position)."""

    def __init__(self, manifest_path=None, audio_tar_filepaths=None, shuffle_n=128, normalize_impulse: bool = False, shift_impulse: bool = False,
                 rng=None, impulse_items: Optional[Sequence[Dict[str, Any]]] = None):
        self._items = list(impulse_items) if impulse_items is not None else _read_manifest_items(manifest_path)
        self._normalize, self._shift, self._rng = normalize_impulse, shift_impulse, random.Random(rng)

    def perturb(self, data):
        it = self._rng.choice(self._items)
        h = (AudioSegment(it["samples"], it.get("sample_rate", data.sample_rate), target_sr=data.sample_rate) if "samples" in it
             else AudioSegment.from_file(it["audio_filepath"], target_sr=data.sample_rate))._samples
        if h.size == 0:
            return
        h = h / max(float(np.abs(h).max()), 1e-8) if not self._normalize else h / max(float(np.sqrt((h ** 2).sum())), 1e-8)
        peak = int(np.argmax(np.abs(h))) if self._shift else 0
        n = data.num_samples
        L = 1 << int(math.ceil(math.log2(n + h.shape[0])))
        y = np.fft.irfft(np.fft.rfft(data._samples, L) * np.fft.rfft(h, L), L)[peak:peak + n]
        m = float(np.abs(y).max())
        data._samples = (y / m * float(np.abs(data._samples).max()) if m > 0 else y).astype(np.float32)


class RirAndNoisePerturbation(Perturbation):
    """Reverberate, then add foreground / background noise (each optional, each with its own probability)."""

    def __init__(self, rir_manifest_path=None, rir_prob: float = 0.5, noise_manifest_paths=None, noise_prob: float = 1.0, min_snr_db=0, max_snr_db=50,
                 bg_noise_manifest_paths=None, bg_min_snr_db=10, bg_max_snr_db=50, apply_noise_rir: bool = False, rng=None,
                 rir=None, noise=None, bg_noise=None, **_):
        self._rng = random.Random(rng)
        self._rir = rir if rir is not None else (ImpulsePerturbation(rir_manifest_path, rng=rng) if rir_manifest_path else None)
        self._noise = noise if noise is not None else (NoisePerturbation(noise_manifest_paths, min_snr_db, max_snr_db, rng=rng) if noise_manifest_paths else None)
        self._bg = bg_noise if bg_noise is not None else (NoisePerturbation(bg_noise_manifest_paths, bg_min_snr_db, bg_max_snr_db, rng=rng)
                                                          if bg_noise_manifest_paths else None)
        self._rir_prob, self._noise_prob = rir_prob, noise_prob

    def perturb(self, data):
        if self._rir is not None and self._rng.random() < self._rir_prob:
            self._rir.perturb(data)
        rms = data.rms_db
        if self._noise is not None and self._rng.random() < self._noise_prob:
            self._noise.perturb_with_input_noise(data, self._noise.get_one_noise_sample(data.sample_rate), data_rms=rms)
        if self._bg is not None:
            self._bg.perturb_with_input_noise(data, self._bg.get_one_noise_sample(data.sample_rate), data_rms=rms)


class TranscodePerturbation(Perturbation):
    """Telephone-codec simulation: band-limit to 300-3400 Hz at 8 kHz and pass through mu-law (G.711) or A-law companding."""

    def __init__(self, codecs: Optional[List[str]] = None, rng=None):
        self._codecs = list(codecs or ["g711", "amr-nb", "ogg"])
        for c in self._codecs:
            if c not in ("g711", "amr-nb", "ogg"):
                raise ValueError(f"TranscodePerturbation - {c} codec is not supported. Use one of ['g711', 'amr-nb', 'ogg']")
        self._rng = random.Random(rng)

    def perturb(self, data):
        codec = self._rng.choice(self._codecs)
        sr = data.sample_rate
        x = resample(data._samples, sr, 8000)
        X = np.fft.rfft(x)
        f = np.fft.rfftfreq(x.shape[0], 1 / 8000.0)
        X[(f < 300) | (f > 3400)] = 0
        x = np.fft.irfft(X, x.shape[0])
        peak = max(float(np.abs(x).max()), 1e-8)
        x = x / peak
        mu = 255.0 if codec == "g711" else 87.6
        bits = 8 if codec == "g711" else 7
        y = np.sign(x) * np.log1p(mu * np.abs(x)) / np.log1p(mu)
        y = np.round((y + 1) / 2 * (2 ** bits - 1)) / (2 ** bits - 1) * 2 - 1
        x = np.sign(y) * ((1 + mu) ** np.abs(y) - 1) / mu * peak
        out = resample(x.astype(np.float32), 8000, sr)
        n = data.num_samples
        data._samples = np.pad(out, (0, max(0, n - out.shape[0])))[:n].astype(np.float32)


class SilencePerturbation(Perturbation):
    """Pads random amounts of silence (``value``) before and after the utterance."""

    def __init__(self, min_start_silence_secs: float = 0, max_start_silence_secs: float = 0, min_end_silence_secs: float = 0,
                 max_end_silence_secs: float = 0, rng=None, value: float = 0):
        self._s, self._e, self._value, self._rng = (min_start_silence_secs, max_start_silence_secs), (min_end_silence_secs, max_end_silence_secs), value, random.Random(rng)

    def perturb(self, data):
        a = int(self._rng.uniform(*self._s) * data.sample_rate)
        b = int(self._rng.uniform(*self._e) * data.sample_rate)
        data._samples = np.concatenate([np.full(a, self._value, np.float32), data._samples, np.full(b, self._value, np.float32)])


perturbation_types: Dict[str, Callable[..., Perturbation]] = {
    "speed": SpeedPerturbation, "time_stretch": TimeStretchPerturbation, "gain": GainPerturbation, "silence": SilencePerturbation,
    "impulse": ImpulsePerturbation, "shift": ShiftPerturbation, "noise": NoisePerturbation, "white_noise": WhiteNoisePerturbation,
    "rir_noise_aug": RirAndNoisePerturbation, "transcode_aug": TranscodePerturbation,
}


def register_perturbation(name: str, perturbation: Callable[..., Perturbation]) -> None:
    if name in perturbation_types:
        raise KeyError(f"Perturbation with the name {name} exists. Type of perturbation : {perturbation_types[name]}.")
    perturbation_types[name] = perturbation


class AudioAugmentor:
    def __init__(self, perturbations: Optional[List[Tuple[float, Perturbation]]] = None, rng=None):
        self._pipeline = list(perturbations or [])
        self._rng = random.Random(rng)

    def perturb(self, segment: AudioSegment) -> None:
        for prob, p in self._pipeline:
            if self._rng.random() < prob:
                p.perturb(segment)

    def max_augmentation_length(self, length: int) -> int:
        for _, p in self._pipeline:
            length = p.max_augmentation_length(length)
        return length

    def __call__(self, samples, sample_rate: int):
        seg = AudioSegment(samples, sample_rate)
        self.perturb(seg)
        return seg._samples


def process_augmentations(augmenter, global_rank: int = 0, world_size: int = 1) -> Optional[AudioAugmentor]:
    """``{"speed": {"prob": 0.5, "min_speed_rate": 0.9, ...}, "noise": {...}}`` -> ``AudioAugmentor``."""
    if augmenter is None or isinstance(augmenter, AudioAugmentor):
        return augmenter
    cfg = {k: dict(v) for k, v in dict(augmenter).items()}
    pipeline = []
    for name, kw in cfg.items():
        if name not in perturbation_types:
            raise ValueError(f"{name} augmentation is not supported; known: {sorted(perturbation_types)}")
        prob = float(kw.pop("prob", 1.0))
        if not 0.0 <= prob <= 1.0:
            raise ValueError(f"{name} augmentation probability {prob} must be in [0, 1]")
        pipeline.append((prob, perturbation_types[name](**kw)))
    return AudioAugmentor(pipeline)

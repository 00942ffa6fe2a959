"""The rest of the TTS data stack: weighted multi-manifest datasets, the vocoder / codec audio dataset, MagpieTTS datasets with
voice context (training, preference pairs, chunked long-form inference), acoustic featurizers (mel, energy, pitch) with on-disk
caches, feature processors, and silence trimming.

References: ``tts/data/vocoder_dataset.py``, ``tts/data/text_to_speech_dataset.py`` (``MagpieTTSDataset``, ``MagpieTTSDatasetDPO``,
``ChunkedTTSInferenceDataset``), ``tts/parts/preprocessing/{features,feature_processors,audio_trimming}.py``,
``tts/parts/utils/tts_dataset_utils.py``.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset, WeightedRandomSampler

from ..data.audio_to_text import load_audio

__all__ = ["BetaBinomialInterpolator", "ChunkedTTSInferenceDataset", "DatasetMeta", "EnergyAudioTrimmer", "EnergyFeaturizer", "FeatureScaler",
           "LanguageThresholds", "LogCompression", "MagpieTTSDataset", "MagpieTTSDatasetDPO", "MeanVarianceNormalization",
           "MeanVarianceSpeakerNormalization", "MelSpectrogramFeaturizer", "PitchFeaturizer", "VadAudioTrimmer", "VocoderDataset", "audio_collate_fn",
           "filter_dataset_by_duration", "get_weighted_sampler", "normalize_volume", "preprocess_manifests", "sample_audio", "stack_tensors"]


# ------------------------------------------------------------------------------------------------ small utilities
def normalize_volume(audio: np.ndarray, volume_level: float = 0.95) -> np.ndarray:
    if not 0.0 <= volume_level <= 1.0:
        raise ValueError(f"volume_level must be in [0, 1], got {volume_level}")
    peak = float(np.abs(audio).max()) if audio.size else 0.0
    return audio if peak == 0.0 else audio * (volume_level / peak)


def stack_tensors(tensors: Sequence[torch.Tensor], max_lens: Sequence[int], pad_value: float = 0.0) -> torch.Tensor:
    """Pads every tensor's leading dimensions up to ``max_lens`` and stacks them."""
    out = []
    for t in tensors:
        pad = []
        for d, m in zip(reversed(range(len(max_lens))), reversed(list(max_lens))):
            pad += [0, int(m) - t.shape[d]]
        pad = [0, 0] * (t.dim() - len(max_lens)) + pad
        out.append(torch.nn.functional.pad(t, pad, value=pad_value))
    return torch.stack(out)


def filter_dataset_by_duration(entries: List[Dict[str, Any]], min_duration: float, max_duration: float):
    """``(kept entries, total hours, kept hours)``."""
    kept, total, kept_h = [], 0.0, 0.0
    for e in entries:
        d = float(e["duration"])
        total += d
        if (min_duration is None or d >= min_duration) and (max_duration is None or d <= max_duration):
            kept.append(e)
            kept_h += d
    return kept, total / 3600.0, kept_h / 3600.0


def get_weighted_sampler(sample_weights: Sequence[float], batch_size: int, world_size: int = 1, num_steps: Optional[int] = None) -> WeightedRandomSampler:
    n = (num_steps * batch_size * world_size) if num_steps else len(sample_weights)
    return WeightedRandomSampler(torch.as_tensor(list(sample_weights), dtype=torch.double), num_samples=n, replacement=True)


def sample_audio(audio: np.ndarray, n_samples: int, rng: np.random.Generator, trim_threshold: Optional[float] = None) -> np.ndarray:
    """A random crop of ``n_samples`` (zero padded when the signal is shorter); with ``trim_threshold`` a crop whose peak is below
    it (silence) is redrawn a few times."""
    if len(audio) <= n_samples:
        return np.pad(audio, (0, n_samples - len(audio)))
    for _ in range(8):
        s = int(rng.integers(0, len(audio) - n_samples + 1))
        seg = audio[s:s + n_samples]
        if trim_threshold is None or np.abs(seg).max() >= trim_threshold:
            return seg
    return seg


class BetaBinomialInterpolator:
    """Alignment priors for (text length, mel length) pairs are computed on a rounded grid, cached, and resized to the requested
    shape: priors of neighbouring lengths are nearly the same picture."""

    def __init__(self, round_mel_len_to: int = 50, round_text_len_to: int = 10, cache_size: int = 500, scaling_factor: float = 1.0):
        self.rm, self.rt, self.scale, self.cache_size = round_mel_len_to, round_text_len_to, scaling_factor, cache_size
        self._cache: Dict[Tuple[int, int], torch.Tensor] = {}

    @staticmethod
    def _round(v: int, to: int) -> int:
        return max(to, int(np.round(v / to)) * to)

    def __call__(self, mel_len: int, text_len: int) -> torch.Tensor:
        from .magpietts import beta_binomial_prior

        key = (self._round(mel_len, self.rm), self._round(text_len, self.rt))
        if key not in self._cache:
            if len(self._cache) >= self.cache_size:
                self._cache.pop(next(iter(self._cache)))
            self._cache[key] = beta_binomial_prior(key[1], key[0], self.scale)
        p = self._cache[key]
        out = torch.nn.functional.interpolate(p[None, None], size=(mel_len, text_len), mode="bilinear", align_corners=False)[0, 0]
        return out / out.sum(dim=1, keepdim=True).clamp(min=1e-12)


# ------------------------------------------------------------------------------------------------ manifests with weights
@dataclass
class DatasetMeta:
    manifest_path: str
    audio_dir: str = ""
    feature_dir: str = ""
    sample_weight: float = 1.0
    tokenizer_names: Optional[List[str]] = None


def preprocess_manifests(dataset_meta: Dict[str, Any], min_duration: Optional[float] = None, max_duration: Optional[float] = None,
                         weighted: bool = False) -> Tuple[List[Dict[str, Any]], List[float]]:
    """Reads every manifest of ``{name: DatasetMeta or dict}``; entries get ``dataset_name`` / ``audio_dir`` / ``feature_dir``.  With
    ``weighted`` a sample's weight is ``dataset weight / dataset size``, so that datasets are drawn in proportion to their weights
    whatever their sizes."""
    samples, weights = [], []
    for name, meta in dataset_meta.items():
        meta = meta if isinstance(meta, DatasetMeta) else DatasetMeta(**dict(meta))
        entries = [json.loads(l) for l in open(meta.manifest_path, encoding="utf-8") if l.strip()]
        entries, _, _ = filter_dataset_by_duration(entries, min_duration, max_duration) if entries and "duration" in entries[0] else (entries, 0, 0)
        for e in entries:
            e = dict(e, dataset_name=name, audio_dir=meta.audio_dir, feature_dir=meta.feature_dir, tokenizer_names=meta.tokenizer_names)
            samples.append(e)
            weights.append(meta.sample_weight / max(1, len(entries)) if weighted else 1.0)
    return samples, weights


def _audio_path(entry: Dict[str, Any], key: str = "audio_filepath") -> str:
    p = entry[key]
    return p if os.path.isabs(p) or not entry.get("audio_dir") else os.path.join(entry["audio_dir"], p)


def audio_collate_fn(batch: List[dict], resample_rates: Optional[Sequence[int]] = None) -> Dict[str, Any]:
    lens = torch.tensor([b["audio"].shape[0] for b in batch])
    out = {"dataset_names": [b["dataset_name"] for b in batch], "audio_filepaths": [b["audio_filepath"] for b in batch],
           "audio": stack_tensors([b["audio"] for b in batch], [int(lens.max())]), "audio_lens": lens}
    for r in resample_rates or ():
        k = f"audio_{r}"
        l = torch.tensor([b[k].shape[0] for b in batch])
        out[k], out[f"audio_lens_{r}"] = stack_tensors([b[k] for b in batch], [int(l.max())]), l
    return out


class VocoderDataset(Dataset):
    """Audio-only examples for vocoder / codec training: a random crop of ``n_samples`` per item (the whole file when ``None``),
    optional peak normalisation, extra copies at other sample rates, extra features through ``feature_processors``."""

    def __init__(self, dataset_meta: Dict[str, Any], sample_rate: int, weighted_sampling_steps_per_epoch: Optional[int] = None,
                 n_samples: Optional[int] = None, resample_rates: Optional[Sequence[int]] = None, feature_processors: Optional[Dict[str, Any]] = None,
                 min_duration: Optional[float] = None, max_duration: Optional[float] = None, trunc_duration: Optional[float] = None,
                 volume_norm: bool = False, trim_threshold: Optional[float] = None, seed: int = 0):
        self.sr, self.n_samples, self.rates, self.steps = sample_rate, n_samples, list(resample_rates or []), weighted_sampling_steps_per_epoch
        self.procs = list((feature_processors or {}).values())
        self.trunc, self.volume_norm, self.trim_threshold = trunc_duration, volume_norm, trim_threshold
        self.samples, self.weights = preprocess_manifests(dataset_meta, min_duration, max_duration, weighted=bool(weighted_sampling_steps_per_epoch))
        self.rng = np.random.default_rng(seed)

    def get_sampler(self, batch_size: int, world_size: int = 1):
        return get_weighted_sampler(self.weights, batch_size, world_size, self.steps) if self.steps else None

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        e = self.samples[i]
        path = _audio_path(e)
        a = np.asarray(load_audio(path, target_sr=self.sr, offset=float(e.get("offset", 0) or 0), duration=self.trunc or e.get("duration")), dtype=np.float32)
        if self.n_samples:
            a = sample_audio(a, self.n_samples, self.rng, self.trim_threshold)
        if self.volume_norm:
            a = normalize_volume(a)
        ex = {"dataset_name": e["dataset_name"], "audio_filepath": path, "audio": torch.from_numpy(np.ascontiguousarray(a))}
        for r in self.rates:
            n = int(round(len(a) * r / self.sr))
            ex[f"audio_{r}"] = torch.nn.functional.interpolate(ex["audio"][None, None], size=n, mode="linear", align_corners=False)[0, 0]
        for p in self.procs:
            p.process(ex)
        return ex

    def collate_fn(self, batch):
        return audio_collate_fn(batch, self.rates)


# ------------------------------------------------------------------------------------------------ featurizers with caches
def _feature_path(entry: Dict[str, Any], feature_dir: str, name: str) -> Path:
    rel = Path(entry["audio_filepath"])
    rel = rel.relative_to(rel.anchor) if rel.is_absolute() else rel
    return Path(feature_dir) / name / rel.with_suffix(".pt")


class MelSpectrogramFeaturizer:
    def __init__(self, feature_name: str = "mel_spec", sample_rate: int = 22050, mel_dim: int = 80, win_length: int = 1024, hop_length: int = 256,
                 lowfreq: float = 0.0, highfreq: Optional[float] = None, log_guard: float = 1e-5, volume_norm: bool = False):
        from ..modules.preprocessor import mel_filterbank

        self.name, self.sr, self.win, self.hop, self.guard, self.volume_norm = feature_name, sample_rate, win_length, hop_length, log_guard, volume_norm
        self.fb = torch.as_tensor(mel_filterbank(sample_rate, win_length, mel_dim, fmin=lowfreq, fmax=highfreq), dtype=torch.float32)

    def _audio(self, entry, audio_dir):
        a = np.asarray(load_audio(_audio_path(dict(entry, audio_dir=audio_dir)), target_sr=self.sr), dtype=np.float32)
        return torch.from_numpy(normalize_volume(a) if self.volume_norm else a)

    def magnitude(self, audio: torch.Tensor) -> torch.Tensor:
        w = torch.hann_window(self.win)
        return torch.stft(audio, self.win, self.hop, self.win, w, return_complex=True).abs()

    def compute(self, audio: torch.Tensor) -> torch.Tensor:
        """[T] -> log-mel [mel_dim, frames]."""
        return torch.log((self.fb @ self.magnitude(audio)).clamp(min=self.guard))

    def compute_mel_spec(self, entry, audio_dir="") -> torch.Tensor:
        return self.compute(self._audio(entry, audio_dir))

    def save(self, entry, audio_dir, feature_dir, overwrite: bool = True):
        p = _feature_path(entry, feature_dir, self.name)
        if p.exists() and not overwrite:
            return
        p.parent.mkdir(parents=True, exist_ok=True)
        torch.save(self.compute_mel_spec(entry, audio_dir), p)

    def load(self, entry, audio_dir, feature_dir) -> Dict[str, torch.Tensor]:
        return {self.name: torch.load(_feature_path(entry, feature_dir, self.name))}

    def collate_fn(self, batch: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        xs = [b[self.name] for b in batch]
        m = max(x.shape[-1] for x in xs)
        return {self.name: torch.stack([torch.nn.functional.pad(x, (0, m - x.shape[-1])) for x in xs])}


class EnergyFeaturizer:
    """Frame energy = L2 norm of the magnitude spectrum over frequency."""

    def __init__(self, spec_featurizer: MelSpectrogramFeaturizer, feature_name: str = "energy"):
        self.spec, self.name = spec_featurizer, feature_name

    def compute(self, audio: torch.Tensor) -> torch.Tensor:
        return self.spec.magnitude(audio).norm(dim=0)

    def save(self, entry, audio_dir, feature_dir, overwrite: bool = True):
        p = _feature_path(entry, feature_dir, self.name)
        if p.exists() and not overwrite:
            return
        p.parent.mkdir(parents=True, exist_ok=True)
        torch.save(self.compute(self.spec._audio(entry, audio_dir)), p)

    def load(self, entry, audio_dir, feature_dir):
        return {self.name: torch.load(_feature_path(entry, feature_dir, self.name))}

    def collate_fn(self, batch):
        xs = [b[self.name] for b in batch]
        m = max(x.shape[-1] for x in xs)
        return {self.name: torch.stack([torch.nn.functional.pad(x, (0, m - x.shape[-1])) for x in xs])}


class PitchFeaturizer:
    """Frame-wise fundamental frequency by normalised autocorrelation: for every frame the lag in ``[sr / pitch_fmax, sr / pitch_fmin]``
    with the highest normalised autocorrelation (parabolic refinement); frames whose peak is under ``voiced_threshold`` are
    unvoiced (pitch 0).  Returns pitch, a voiced mask and the peak value as voicing probability."""

    def __init__(self, sample_rate: int = 22050, win_length: int = 1024, hop_length: int = 256, pitch_fmin: float = 65.0, pitch_fmax: float = 2093.0,
                 voiced_threshold: float = 0.5, pitch_feature_name: str = "pitch", voiced_mask_feature_name: str = "voiced_mask",
                 voiced_prob_feature_name: str = "voiced_prob"):
        self.sr, self.win, self.hop, self.fmin, self.fmax, self.thr = sample_rate, win_length, hop_length, pitch_fmin, pitch_fmax, voiced_threshold
        self.names = (pitch_feature_name, voiced_mask_feature_name, voiced_prob_feature_name)

    def compute_pitch(self, audio: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        x = torch.nn.functional.pad(audio.float(), (self.win // 2, self.win // 2))
        fr = x.unfold(0, self.win, self.hop)
        fr = fr - fr.mean(dim=1, keepdim=True)
        n = 2 * self.win
        spec = torch.fft.rfft(fr, n=n)
        ac = torch.fft.irfft(spec * spec.conj(), n=n)[:, : self.win]
        # normalise by the energy of the two overlapping parts (so that a pure tone scores 1 at its period)
        e = torch.cumsum(fr.pow(2), dim=1)
        tot = e[:, -1:]
        lags = torch.arange(self.win)
        head = torch.cat([torch.zeros_like(tot), e[:, :-1]], dim=1)      # energy of the first `lag` samples
        e1 = tot - head                                                  # energy of x[lag:]
        e2 = e.flip(1)                                                   # energy of x[:win-lag]
        nac = ac / (e1 * e2).clamp(min=1e-10).sqrt()
        lo, hi = max(2, int(self.sr / self.fmax)), min(self.win - 2, int(self.sr / self.fmin))
        seg = nac[:, lo:hi + 1]
        best = seg.max(dim=1).values
        # a periodic signal scores alike at every multiple of its period: take the shortest lag that is a local maximum and
        # within a few percent of the best score
        local = (seg >= nac[:, lo - 1:hi]) & (seg >= nac[:, lo + 1:hi + 2])
        cand = local & (seg >= 0.93 * best[:, None])
        idx = torch.where(cand.any(dim=1), cand.int().argmax(dim=1), seg.argmax(dim=1))
        peak = seg.gather(1, idx[:, None])[:, 0]
        lag = (idx + lo).float()
        a, b, c = nac.gather(1, (idx + lo - 1)[:, None])[:, 0], peak, nac.gather(1, (idx + lo + 1)[:, None])[:, 0]
        lag = lag + 0.5 * (a - c) / (a - 2 * b + c).clamp(max=-1e-8)
        voiced = peak >= self.thr
        pitch = torch.where(voiced, self.sr / lag.clamp(min=1.0), torch.zeros_like(lag))
        return pitch, voiced, peak.clamp(0, 1)

    def save(self, entry, audio_dir, feature_dir, overwrite: bool = True):
        a = torch.from_numpy(np.asarray(load_audio(_audio_path(dict(entry, audio_dir=audio_dir)), target_sr=self.sr), dtype=np.float32))
        vals = self.compute_pitch(a)
        for name, v in zip(self.names, vals):
            if name:
                p = _feature_path(entry, feature_dir, name)
                if p.exists() and not overwrite:
                    continue
                p.parent.mkdir(parents=True, exist_ok=True)
                torch.save(v, p)

    def load(self, entry, audio_dir, feature_dir):
        return {n: torch.load(_feature_path(entry, feature_dir, n)) for n in self.names if n}

    def collate_fn(self, batch):
        out = {}
        for n in self.names:
            if n and n in batch[0]:
                xs = [b[n] for b in batch]
                m = max(x.shape[-1] for x in xs)
                out[n] = torch.stack([torch.nn.functional.pad(x, (0, m - x.shape[-1])) for x in xs])
        return out


# ------------------------------------------------------------------------------------------------ feature processors
class FeatureScaler:
    def __init__(self, field: str, add_value: float = 0.0, div_value: float = 1.0):
        self.field, self.add, self.div = field, add_value, div_value

    def process(self, ex: dict) -> None:
        ex[self.field] = (ex[self.field] + self.add) / self.div


class LogCompression:
    def __init__(self, field: str, log_zero_guard_type: str = "add", log_zero_guard_value: float = 1.0):
        if log_zero_guard_type not in ("add", "clamp"):
            raise ValueError(f"unsupported log zero guard type {log_zero_guard_type!r}")
        self.field, self.kind, self.val = field, log_zero_guard_type, log_zero_guard_value

    def process(self, ex: dict) -> None:
        f = ex[self.field]
        ex[self.field] = torch.log(f + self.val if self.kind == "add" else f.clamp(min=self.val))


class MeanVarianceNormalization:
    """``stats_path``: JSON ``{"default": {"<field>_mean": m, "<field>_std": s}}``; only positions where ``mask_field`` is set are
    normalised, the rest are zeroed."""

    def __init__(self, field: str, stats_path: str, mask_field: Optional[str] = "voiced_mask"):
        st = json.load(open(stats_path, encoding="utf-8"))["default"]
        self.field, self.mask_field, self.mean, self.std = field, mask_field, float(st[f"{field}_mean"]), float(st[f"{field}_std"])

    def process(self, ex: dict) -> None:
        f = (ex[self.field] - self.mean) / self.std
        if self.mask_field:
            f = torch.where(ex[self.mask_field].bool(), f, torch.zeros_like(f))
        ex[self.field] = f


class MeanVarianceSpeakerNormalization:
    """As above with statistics per speaker (``{"<speaker>": {...}, "default": {...}}``; unknown speakers use ``default``)."""

    def __init__(self, field: str, stats_path: str, speaker_field: str = "speaker", mask_field: Optional[str] = "voiced_mask", fallback_to_default: bool = True):
        self.stats = json.load(open(stats_path, encoding="utf-8"))
        self.field, self.spk, self.mask_field, self.fallback = field, speaker_field, mask_field, fallback_to_default

    def process(self, ex: dict) -> None:
        key = str(ex[self.spk])
        if key not in self.stats:
            if not self.fallback:
                raise ValueError(f"no statistics for speaker {key}")
            key = "default"
        st = self.stats[key]
        f = (ex[self.field] - float(st[f"{self.field}_mean"])) / float(st[f"{self.field}_std"])
        if self.mask_field:
            f = torch.where(ex[self.mask_field].bool(), f, torch.zeros_like(f))
        ex[self.field] = f


# ------------------------------------------------------------------------------------------------ trimming
def _pad_indices(start: int, end: int, max_sample: int, pad: int) -> Tuple[int, int]:
    return max(0, start - pad), min(max_sample, end + pad)


class EnergyAudioTrimmer:
    """Speech starts at the first run of ``speech_frame_threshold`` frames whose level is within ``db_threshold`` dB of the
    loudest frame (and ends at the last such run); ``pad_seconds`` of margin is kept on both sides."""

    def __init__(self, db_threshold: float = 50.0, ref_amplitude: Optional[float] = None, speech_frame_threshold: int = 1, trim_win_length: int = 2048,
                 trim_hop_length: int = 512, pad_seconds: float = 0.1, volume_norm: bool = True):
        self.db, self.ref, self.k, self.win, self.hop, self.pad, self.volume_norm = db_threshold, ref_amplitude, speech_frame_threshold, trim_win_length, trim_hop_length, pad_seconds, volume_norm

    def trim_audio(self, audio: np.ndarray, sample_rate: int, audio_id: str = "") -> Tuple[np.ndarray, int, int]:
        x = normalize_volume(audio) if self.volume_norm else audio
        if len(x) < self.win:
            return audio, 0, len(audio)
        fr = np.lib.stride_tricks.sliding_window_view(np.pad(x, (self.win // 2, self.win // 2)), self.win)[:: self.hop]
        rms = np.sqrt((fr ** 2).mean(axis=1))
        ref = self.ref if self.ref is not None else float(rms.max())
        speech = 20 * np.log10(np.maximum(rms, 1e-10) / max(ref, 1e-10)) > -self.db
        start_f, end_f = get_start_and_end_of_speech_frames(speech, self.k, audio_id)
        s, e = _pad_indices(start_f * self.hop, end_f * self.hop, len(audio), int(self.pad * sample_rate))
        return audio[s:e], s, e


def get_start_and_end_of_speech_frames(is_speech: np.ndarray, speech_frame_threshold: int, audio_id: str = "") -> Tuple[int, int]:
    """First frame of the first run and last frame (exclusive) of the last run of ``speech_frame_threshold`` speech frames; the
    whole range when no such run exists."""
    n, k = len(is_speech), speech_frame_threshold
    runs = np.convolve(is_speech.astype(np.int32), np.ones(k, dtype=np.int32), mode="valid") == k if n >= k else np.zeros(0, dtype=bool)
    if not runs.any():
        return 0, n
    idx = np.nonzero(runs)[0]
    return int(idx[0]), int(idx[-1]) + k


class VadAudioTrimmer:
    """Trimming by a voice-activity model: ``vad(frames [N, win]) -> speech probability [N]`` (any callable, e.g. a MarbleNet
    wrapper) on frames at ``vad_sample_rate``; indices are scaled back to the audio's rate."""

    def __init__(self, vad: Callable[[torch.Tensor], torch.Tensor], vad_sample_rate: int = 16000, vad_threshold: float = 0.5, speech_frame_threshold: int = 1,
                 trim_win_length: int = 4096, trim_hop_length: int = 1024, pad_seconds: float = 0.1, volume_norm: bool = True):
        self.vad, self.vsr, self.thr, self.k, self.win, self.hop, self.pad, self.volume_norm = vad, vad_sample_rate, vad_threshold, speech_frame_threshold, trim_win_length, trim_hop_length, pad_seconds, volume_norm

    def trim_audio(self, audio: np.ndarray, sample_rate: int, audio_id: str = "") -> Tuple[np.ndarray, int, int]:
        x = torch.from_numpy(np.ascontiguousarray(normalize_volume(audio) if self.volume_norm else audio)).float()
        if sample_rate != self.vsr:
            x = torch.nn.functional.interpolate(x[None, None], size=int(round(len(x) * self.vsr / sample_rate)), mode="linear", align_corners=False)[0, 0]
        if len(x) < self.win:
            return audio, 0, len(audio)
        with torch.no_grad():
            prob = self.vad(x.unfold(0, self.win, self.hop))
        start_f, end_f = get_start_and_end_of_speech_frames((prob > self.thr).cpu().numpy(), self.k, audio_id)
        scale = sample_rate / self.vsr
        s, e = int(start_f * self.hop * scale), int(min(len(x), end_f * self.hop + self.win - self.hop) * scale)
        s, e = _pad_indices(s, e, len(audio), int(self.pad * sample_rate))
        return audio[s:e], s, e


# ------------------------------------------------------------------------------------------------ MagpieTTS datasets
class LanguageThresholds:
    """Above how many words (characters for languages written without spaces) a text is synthesised chunk by chunk."""

    words = {"en": 45, "de": 40, "es": 45, "fr": 45, "it": 45, "pt": 45, "nl": 40, "hi": 50, "vi": 50}
    chars = {"zh": 100, "ja": 100, "ko": 120, "th": 150}
    default_words = 45

    def get_word_count(self, text: str, language: str) -> int:
        return len(re.sub(r"\s+", "", text)) if language in self.chars else len(text.split())

    def threshold(self, language: str) -> int:
        return self.chars.get(language, self.words.get(language, self.default_words))

    def exceeds_threshold(self, text: str, language: str) -> bool:
        return self.get_word_count(text, language) > self.threshold(language)


class MagpieTTSDataset(Dataset):
    """Manifest entries: ``text``, ``audio_filepath`` (or ``target_audio_codes_path``: a saved ``[C, T]`` tensor), optional
    ``context_audio_filepath`` (+ ``context_audio_duration``) or ``context_audio_codes_path``, ``speaker``, ``language``.

    The context (voice prompt) is a random slice of ``context_duration_min..max`` seconds of the context audio (all of it when
    shorter); without a context file and with ``use_self_context`` a slice of the target audio itself is used.  ``tokenizers``:
    ``{name: tokenizer}``; an entry picks the tokenizer named after its language (or the first)."""

    def __init__(self, dataset_meta: Dict[str, Any], sample_rate: int, tokenizers: Dict[str, Any], codec_frame_rate: float = 21.5,
                 min_duration: Optional[float] = 0.2, max_duration: Optional[float] = 20.0, context_duration_min: float = 3.0, context_duration_max: float = 10.0,
                 load_cached_codes_if_available: bool = True, use_self_context: bool = True, prior_scaling_factor: Optional[float] = None,
                 weighted_sampling_steps_per_epoch: Optional[int] = None, bos_id: Optional[int] = None, eos_id: Optional[int] = None, volume_norm: bool = True, seed: int = 0):
        self.sr, self.tok, self.frame_rate = sample_rate, dict(tokenizers), codec_frame_rate
        self.cmin, self.cmax, self.cached, self.self_ctx = context_duration_min, context_duration_max, load_cached_codes_if_available, use_self_context
        self.steps, self.volume_norm = weighted_sampling_steps_per_epoch, volume_norm
        self.samples, self.weights = preprocess_manifests(dataset_meta, min_duration, max_duration, weighted=bool(weighted_sampling_steps_per_epoch))
        self.prior = BetaBinomialInterpolator(scaling_factor=prior_scaling_factor) if prior_scaling_factor else None
        first = next(iter(self.tok.values()))
        self.bos = bos_id if bos_id is not None else int(first.vocab_size)
        self.eos = eos_id if eos_id is not None else int(first.vocab_size) + 1
        self.rng = np.random.default_rng(seed)

    def get_sampler(self, batch_size: int, world_size: int = 1):
        return get_weighted_sampler(self.weights, batch_size, world_size, self.steps) if self.steps else None

    def __len__(self):
        return len(self.samples)

    def _tokenizer_for(self, e) -> Tuple[str, Any]:
        names = e.get("tokenizer_names") or []
        lang = e.get("language", "en")
        for n in list(names) + [lang]:
            if n in self.tok:
                return n, self.tok[n]
        n = next(iter(self.tok))
        return n, self.tok[n]

    def _slice_context(self, total_sec: float) -> Tuple[float, float]:
        want = float(self.rng.uniform(self.cmin, self.cmax))
        dur = min(want, total_sec)
        start = float(self.rng.uniform(0.0, max(0.0, total_sec - dur)))
        return start, dur

    def __getitem__(self, i) -> Dict[str, Any]:
        e = self.samples[i]
        name, tok = self._tokenizer_for(e)
        ids = [self.bos] + list(tok.text_to_ids(e.get("normalized_text", e["text"]))) + [self.eos]
        ex: Dict[str, Any] = {"dataset_name": e["dataset_name"], "raw_text": e["text"], "text": torch.tensor(ids, dtype=torch.long), "tokenizer_name": name,
                              "language": e.get("language", "en"), "speaker": e.get("speaker", -1)}
        if self.cached and e.get("target_audio_codes_path"):
            ex["audio_codes"] = torch.load(e["target_audio_codes_path"]).long()
        else:
            a = np.asarray(load_audio(_audio_path(e), target_sr=self.sr, offset=float(e.get("offset", 0) or 0), duration=e.get("duration")), dtype=np.float32)
            ex["audio"] = torch.from_numpy(normalize_volume(a) if self.volume_norm else a)
            ex["audio_filepath"] = _audio_path(e)
        if self.cached and e.get("context_audio_codes_path"):
            c = torch.load(e["context_audio_codes_path"]).long()
            start, dur = self._slice_context(c.shape[-1] / self.frame_rate)
            s, n = int(start * self.frame_rate), max(1, int(dur * self.frame_rate))
            ex["context_audio_codes"] = c[:, s:s + n]
        elif e.get("context_audio_filepath"):
            total = float(e.get("context_audio_duration", 0.0)) or None
            if total is None:
                c = np.asarray(load_audio(_audio_path(e, "context_audio_filepath"), target_sr=self.sr), dtype=np.float32)
                start, dur = self._slice_context(len(c) / self.sr)
                c = c[int(start * self.sr): int((start + dur) * self.sr)]
            else:
                start, dur = self._slice_context(total)
                c = np.asarray(load_audio(_audio_path(e, "context_audio_filepath"), target_sr=self.sr, offset=start, duration=dur), dtype=np.float32)
            ex["context_audio"] = torch.from_numpy(normalize_volume(c) if self.volume_norm else c)
        elif self.self_ctx and "audio" in ex:
            start, dur = self._slice_context(len(ex["audio"]) / self.sr)
            ex["context_audio"] = ex["audio"][int(start * self.sr): int((start + dur) * self.sr)].clone()
        if self.prior is not None:
            n_frames = ex["audio_codes"].shape[-1] if "audio_codes" in ex else max(1, int(round(len(ex["audio"]) / self.sr * self.frame_rate)))
            ex["align_prior"] = self.prior(n_frames, len(ids))
        return ex

    def collate_fn(self, batch: List[Dict[str, Any]]) -> Dict[str, Any]:
        out: Dict[str, Any] = {k: [b[k] for b in batch] for k in ("dataset_name", "raw_text", "tokenizer_name", "language", "speaker")}
        tl = torch.tensor([len(b["text"]) for b in batch])
        out["text"], out["text_lens"] = stack_tensors([b["text"] for b in batch], [int(tl.max())]), tl
        for key in ("audio", "context_audio"):
            if all(key in b for b in batch):
                l = torch.tensor([b[key].shape[0] for b in batch])
                out[key], out[f"{key}_lens"] = stack_tensors([b[key] for b in batch], [int(l.max())]), l
        for key in ("audio_codes", "context_audio_codes"):
            if all(key in b for b in batch):
                l = torch.tensor([b[key].shape[-1] for b in batch])
                out[key] = torch.stack([torch.nn.functional.pad(b[key], (0, int(l.max()) - b[key].shape[-1])) for b in batch])
                out[f"{key}_lens"] = l
        if all("align_prior" in b for b in batch):
            ps = [b["align_prior"] for b in batch]
            out["align_prior_matrix"] = stack_tensors(ps, [max(p.shape[0] for p in ps), max(p.shape[1] for p in ps)])
        return out

    @staticmethod
    def as_model_batch(batch: Dict[str, Any]) -> tuple:
        """``(text, text_len, audio, audio_len[, context_audio, context_audio_len])`` as ``MagpieTTSModel.training_step`` takes it."""
        t = (batch["text"], batch["text_lens"], batch["audio"], batch["audio_lens"])
        return t + (batch["context_audio"], batch["context_audio_lens"]) if "context_audio" in batch else t


class MagpieTTSDatasetDPO(MagpieTTSDataset):
    """Preference pairs: consecutive manifest lines ``2k`` (chosen) and ``2k + 1`` (rejected) share a prompt; each carries ``reward``."""

    def __len__(self):
        return len(self.samples) // 2

    def __getitem__(self, i):
        return {"chosen": super().__getitem__(2 * i), "rejected": super().__getitem__(2 * i + 1),
                "rewards": (float(self.samples[2 * i].get("reward", 1.0)), float(self.samples[2 * i + 1].get("reward", 0.0)))}

    def collate_fn(self, batch):
        return {"chosen": super().collate_fn([b["chosen"] for b in batch]), "rejected": super().collate_fn([b["rejected"] for b in batch]),
                "rewards": torch.tensor([b["rewards"] for b in batch])}


class ChunkedTTSInferenceDataset(MagpieTTSDataset):
    """Inference items whose text is pre-split into sentence chunks when it exceeds the language's threshold; every item carries
    ``chunked_tokens`` (a list of id tensors) and one context for all its chunks."""

    def __init__(self, *a, max_chunk_chars: int = 200, thresholds: Optional[LanguageThresholds] = None, **kw):
        kw.setdefault("min_duration", None)
        kw.setdefault("max_duration", None)
        super().__init__(*a, **kw)
        self.max_chars, self.thr = max_chunk_chars, thresholds or LanguageThresholds()

    def __getitem__(self, i):
        from .magpietts import split_text_for_tts

        e = self.samples[i]
        if "audio_filepath" not in e and "target_audio_codes_path" not in e:          # text-only inference manifests
            name, tok = self._tokenizer_for(e)
            ex = {"dataset_name": e["dataset_name"], "raw_text": e["text"], "tokenizer_name": name, "language": e.get("language", "en"),
                  "speaker": e.get("speaker", -1), "text": torch.tensor([self.bos] + list(tok.text_to_ids(e["text"])) + [self.eos])}
            if e.get("context_audio_filepath"):
                c = np.asarray(load_audio(_audio_path(e, "context_audio_filepath"), target_sr=self.sr), dtype=np.float32)
                ex["context_audio"] = torch.from_numpy(c[: int(self.cmax * self.sr)])
        else:
            ex = super().__getitem__(i)
        _, tok = self._tokenizer_for(e)
        lang = ex["language"]
        parts = split_text_for_tts(e["text"], self.max_chars) if self.thr.exceeds_threshold(e["text"], lang) else [e["text"]]
        ex["chunked_text"] = parts
        ex["chunked_tokens"] = [torch.tensor([self.bos] + list(tok.text_to_ids(p)) + [self.eos], dtype=torch.long) for p in parts]
        return ex

    def collate_fn(self, batch):
        keep = [{k: v for k, v in b.items() if k not in ("chunked_text", "chunked_tokens")} for b in batch]
        out = super().collate_fn(keep)
        out["chunked_text"] = [b["chunked_text"] for b in batch]
        out["chunked_tokens"] = [b["chunked_tokens"] for b in batch]
        return out

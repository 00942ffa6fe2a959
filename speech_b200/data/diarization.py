"""Diarization data: RTTM parsing, frame-level speaker-activity targets, the end-to-end diarization dataset and a
synthetic multi-speaker session generator (reference: ``data/audio_to_diar_label.py``, ``data/data_simulation.py``,
``parts/utils/speaker_utils.py``)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

from .audio_to_text import load_audio, read_manifest


def read_rttm(path: str) -> List[Tuple[float, float, str]]:
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            p = line.split()
            if len(p) >= 8 and p[0] == "SPEAKER":
                out.append((float(p[3]), float(p[3]) + float(p[4]), p[7]))
    return out


def write_rttm(path: str, segments: Sequence[Tuple[float, float, str]], uniq_id: str = "session") -> None:
    with open(path, "w", encoding="utf-8") as f:
        for st, en, spk in segments:
            f.write(f"SPEAKER {uniq_id} 1 {st:.3f} {en - st:.3f} <NA> <NA> {spk} <NA> <NA>\n")


def segments_to_frame_targets(segments: Sequence[Tuple[float, float, str]], num_frames: int, frame_sec: float, num_spks: int,
                              offset: float = 0.0) -> torch.Tensor:
    """[T, S] 0/1 activity; speakers are indexed by order of first appearance."""
    order: Dict[str, int] = {}
    for st, en, spk in sorted(segments):
        if spk not in order and len(order) < num_spks:
            order[spk] = len(order)
    tgt = torch.zeros((num_frames, num_spks))
    for st, en, spk in segments:
        if spk not in order:
            continue
        a = int(round(max(0.0, st - offset) / frame_sec))
        b = int(round(max(0.0, en - offset) / frame_sec))
        tgt[a:min(b, num_frames), order[spk]] = 1.0
    return tgt


def _collate(batch):
    alen = torch.tensor([b[0].shape[0] for b in batch], dtype=torch.long)
    audio = torch.zeros(len(batch), int(alen.max()))
    tlen = torch.tensor([b[1].shape[0] for b in batch], dtype=torch.long)
    tgt = torch.zeros(len(batch), int(tlen.max()), batch[0][1].shape[1])
    for i, (a, t) in enumerate(batch):
        audio[i, : a.shape[0]] = a
        tgt[i, : t.shape[0]] = t
    return audio, alen, tgt, tlen


class AudioToSpeechE2ESpkDiarDataset(Dataset):
    """Manifest lines ``{"audio_filepath", "offset", "duration", "rttm_filepath"}``; sessions are cut into
    ``session_len_sec`` windows."""

    def __init__(self, manifest_filepath, num_spks: int, frame_sec: float, session_len_sec: float = 90.0,
                 sample_rate: int = 16000, **_):
        self.items = []
        for it in read_manifest(manifest_filepath):
            dur = float(it.get("duration") or 0.0)
            off = float(it.get("offset") or 0.0)
            n = max(1, int(np.ceil(dur / session_len_sec))) if dur > 0 else 1
            for k in range(n):
                self.items.append((it, off + k * session_len_sec, min(session_len_sec, dur - k * session_len_sec) if dur else None))
        self.num_spks, self.frame_sec, self.sr = num_spks, frame_sec, sample_rate

    def durations(self):
        return [d or 0.0 for _, _, d in self.items]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, idx):
        it, off, dur = self.items[idx]
        x = torch.as_tensor(load_audio(it["audio_filepath"], target_sr=self.sr, offset=off, duration=dur), dtype=torch.float32)
        T = int(np.ceil(x.numel() / self.sr / self.frame_sec))
        segs = read_rttm(it["rttm_filepath"]) if it.get("rttm_filepath") else []
        return x, segments_to_frame_targets(segs, T, self.frame_sec, self.num_spks, offset=off)

    collate_fn = staticmethod(_collate)


class SyntheticDiarizationDataset(Dataset):
    """Sessions of up to ``num_spks`` "speakers" (tones of distinct pitch with noise) taking turns, sometimes overlapping."""

    def __init__(self, num_samples: int, num_spks: int, frame_sec: float, min_duration: float = 2.0, max_duration: float = 4.0,
                 sample_rate: int = 16000, seed: int = 0, overlap_prob: float = 0.2):
        self.n, self.num_spks, self.frame_sec, self.sr, self.seed = num_samples, num_spks, frame_sec, sample_rate, seed
        g = np.random.default_rng(seed)
        self._dur = g.uniform(min_duration, max_duration, size=num_samples)
        self.overlap_prob = overlap_prob

    def durations(self):
        return self._dur.tolist()

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = np.random.default_rng(self.seed * 7919 + idx)
        n = int(self._dur[idx] * self.sr)
        x = 0.01 * g.standard_normal(n)
        segs = []
        t, k = 0.0, 0
        n_spk = int(g.integers(1, self.num_spks + 1))
        while t < self._dur[idx] - 0.3:
            d = float(g.uniform(0.3, 1.0))
            spk = int(g.integers(0, n_spk))
            st, en = t, min(self._dur[idx], t + d)
            a, b = int(st * self.sr), int(en * self.sr)
            tt = np.arange(b - a) / self.sr
            x[a:b] += 0.3 * np.sin(2 * np.pi * (200.0 + 170.0 * spk) * tt)
            segs.append((st, en, f"s{spk}"))
            t = en - (d * 0.5 if g.random() < self.overlap_prob else -float(g.uniform(0.0, 0.3)))
            k += 1
        T = int(np.ceil(n / self.sr / self.frame_sec))
        return torch.as_tensor(x, dtype=torch.float32), segments_to_frame_targets(segs, T, self.frame_sec, self.num_spks)

    collate_fn = staticmethod(_collate)


def build_diarization_dataset(config, num_spks: int, frame_sec: float):
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn = get("synthetic", None)
    if syn is not None:
        return SyntheticDiarizationDataset(num_spks=num_spks, frame_sec=frame_sec, **dict(syn))
    return AudioToSpeechE2ESpkDiarDataset(get("manifest_filepath"), num_spks=num_spks, frame_sec=frame_sec,
                                          session_len_sec=get("session_len_sec", 90.0), sample_rate=get("sample_rate", 16000))

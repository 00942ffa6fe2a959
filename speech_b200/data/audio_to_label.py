"""Audio → label datasets: utterance-level classification / speaker labels, frame-level labels (VAD), and a synthetic
variant for tests and benchmarks (reference: ``data/audio_to_label.py``, ``audio_to_label_dataset.py``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

from .audio_to_text import load_audio, read_manifest


def _collate_labels(batch, frame_level: bool = False, pad_label: int = 0):
    audio_lens = torch.tensor([b[0].shape[0] for b in batch], dtype=torch.long)
    audio = torch.zeros(len(batch), int(audio_lens.max()), dtype=torch.float32)
    for i, b in enumerate(batch):
        audio[i, : b[0].shape[0]] = b[0]
    if frame_level:
        ll = torch.tensor([len(b[1]) for b in batch], dtype=torch.long)
        labels = torch.full((len(batch), int(ll.max())), pad_label, dtype=torch.long)
        for i, b in enumerate(batch):
            labels[i, : len(b[1])] = torch.as_tensor(b[1], dtype=torch.long)
    else:
        labels = torch.tensor([int(b[1]) for b in batch], dtype=torch.long)
        ll = torch.ones(len(batch), dtype=torch.long)
    return audio, audio_lens, labels, ll


class AudioToClassificationLabelDataset(Dataset):
    """Manifest lines ``{"audio_filepath", "duration", "label"[, "offset"]}``; ``labels`` fixes the class order."""

    def __init__(self, manifest_filepath, labels: Optional[Sequence[str]] = None, sample_rate: int = 16000,
                 min_duration: Optional[float] = 0.1, max_duration: Optional[float] = None, trim: bool = False,
                 is_regression_task: bool = False, cal_labels_occurrence: bool = False, **_):
        self.items = read_manifest(manifest_filepath, min_duration=min_duration, max_duration=max_duration)
        found = sorted({str(it["label"]) for it in self.items})
        self.labels = list(labels) if labels else found
        self.label2id = {l: i for i, l in enumerate(self.labels)}
        self.id2label = {i: l for l, i in self.label2id.items()}
        self.sample_rate = sample_rate
        self.is_regression_task = is_regression_task
        if cal_labels_occurrence:
            counts = np.zeros(len(self.labels))
            for it in self.items:
                counts[self.label2id[str(it["label"])]] += 1
            self.labels_occurrence = counts.tolist()

    @property
    def num_classes(self) -> int:
        return len(self.labels)

    def durations(self) -> List[float]:
        return [float(it.get("duration", 0.0)) for it in self.items]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, idx):
        it = self.items[idx]
        x = load_audio(it["audio_filepath"], target_sr=self.sample_rate, offset=float(it.get("offset", 0.0) or 0.0),
                       duration=it.get("duration"))
        lab = float(it["label"]) if self.is_regression_task else self.label2id[str(it["label"])]
        return torch.as_tensor(x, dtype=torch.float32), lab

    def collate_fn(self, batch):
        return _collate_labels(batch)

    _collate_fn = collate_fn


AudioToSpeechLabelDataset = AudioToClassificationLabelDataset


class AudioToMultiLabelDataset(AudioToClassificationLabelDataset):
    """Frame-level labels: ``label`` is a whitespace-separated sequence of class names, one per output frame."""

    def __getitem__(self, idx):
        it = self.items[idx]
        x = load_audio(it["audio_filepath"], target_sr=self.sample_rate, offset=float(it.get("offset", 0.0) or 0.0),
                       duration=it.get("duration"))
        labs = [self.label2id[t] for t in str(it["label"]).split()]
        return torch.as_tensor(x, dtype=torch.float32), labs

    def collate_fn(self, batch):
        return _collate_labels(batch, frame_level=True)


class SyntheticLabelDataset(Dataset):
    """Deterministic noise-plus-tone utterances whose dominant frequency encodes the class (learnable in a few steps)."""

    def __init__(self, num_samples: int, num_classes: int, min_duration: float = 0.5, max_duration: float = 1.0,
                 sample_rate: int = 16000, seed: int = 0, frame_level: bool = False, frame_hop: float = 0.02):
        self.n, self.num_classes, self.sr = num_samples, num_classes, sample_rate
        self.labels = [str(i) for i in range(num_classes)]
        g = np.random.default_rng(seed)
        self._dur = g.uniform(min_duration, max_duration, size=num_samples)
        self._lab = g.integers(0, num_classes, size=num_samples)
        self.seed, self.frame_level, self.frame_hop = seed, frame_level, frame_hop

    def durations(self):
        return self._dur.tolist()

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = np.random.default_rng(self.seed * 100003 + idx)
        n = int(self._dur[idx] * self.sr)
        t = np.arange(n) / self.sr
        lab = int(self._lab[idx])
        x = 0.3 * np.sin(2 * np.pi * (300.0 + 400.0 * lab) * t) + 0.02 * g.standard_normal(n)
        if self.frame_level:
            return torch.as_tensor(x, dtype=torch.float32), [lab] * max(1, int(self._dur[idx] / self.frame_hop))
        return torch.as_tensor(x, dtype=torch.float32), lab

    def collate_fn(self, batch):
        return _collate_labels(batch, frame_level=self.frame_level)


def build_label_dataset(config, frame_level: bool = False):
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn = get("synthetic", None)
    if syn is not None:
        return SyntheticLabelDataset(frame_level=frame_level, **dict(syn))
    cls = AudioToMultiLabelDataset if frame_level else AudioToClassificationLabelDataset
    return cls(get("manifest_filepath"), labels=get("labels", None), sample_rate=get("sample_rate", 16000),
               min_duration=get("min_duration", 0.1), max_duration=get("max_duration", None),
               is_regression_task=get("is_regression_task", False), cal_labels_occurrence=get("cal_labels_occurrence", False))

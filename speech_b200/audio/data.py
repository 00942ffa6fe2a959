"""Audio-to-target datasets for enhancement / separation: manifests with ``input_filepath`` / ``target_filepath`` (one or
several channels, optional ``embedding`` / ``reference`` keys) or an on-the-fly synthetic mixer (clean tone bursts + noise)
(reference: ``audio/data/audio_to_audio.py``, ``audio_to_audio_dataset.py``, ``data_simulation.py``)."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from ..data.audio_to_text import get_dataloader_from_config, load_audio, read_manifest


def _collate(batch):
    il = torch.tensor([b[0].shape[-1] for b in batch], dtype=torch.long)
    C_in, C_t = batch[0][0].shape[0], batch[0][1].shape[0]
    x = torch.zeros(len(batch), C_in, int(il.max()))
    y = torch.zeros(len(batch), C_t, int(il.max()))
    for i, (a, b) in enumerate(batch):
        x[i, :, : a.shape[-1]] = a
        y[i, :, : b.shape[-1]] = b[..., : a.shape[-1]]
    return x, il, y, il.clone()


class AudioToTargetDataset(Dataset):
    def __init__(self, manifest_filepath, sample_rate: int = 16000, input_key: str = "input_filepath", target_key: str = "target_filepath",
                 audio_duration: Optional[float] = None, random_offset: bool = False, min_duration=None, max_duration=None, **_):
        self.items = read_manifest(manifest_filepath, min_duration=min_duration, max_duration=max_duration)
        self.sr, self.ik, self.tk, self.dur, self.rand = sample_rate, input_key, target_key, audio_duration, random_offset

    def durations(self):
        return [float(it.get("duration", self.dur or 0.0)) for it in self.items]

    def __len__(self):
        return len(self.items)

    def _load(self, path, off, dur):
        x = np.asarray(load_audio(path, target_sr=self.sr, offset=off, duration=dur), dtype=np.float32)
        return torch.as_tensor(x).reshape(1, -1) if x.ndim == 1 else torch.as_tensor(x.T if x.shape[0] > x.shape[1] else x)

    def __getitem__(self, idx):
        it = self.items[idx]
        off = float(it.get("offset", 0.0) or 0.0)
        dur = self.dur or it.get("duration")
        if self.rand and self.dur and it.get("duration") and it["duration"] > self.dur:
            off += float(np.random.uniform(0, it["duration"] - self.dur))
        return self._load(it[self.ik], off, dur), self._load(it[self.tk], off, dur)

    collate_fn = staticmethod(_collate)


class SyntheticNoisyDataset(Dataset):
    def __init__(self, num_samples: int, min_duration: float = 0.5, max_duration: float = 1.0, sample_rate: int = 16000, snr_db: float = 5.0,
                 num_channels: int = 1, seed: int = 0):
        self.n, self.sr, self.snr, self.C, self.seed = num_samples, sample_rate, snr_db, num_channels, seed
        self._dur = np.random.default_rng(seed).uniform(min_duration, max_duration, size=num_samples)

    def durations(self):
        return self._dur.tolist()

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = np.random.default_rng(self.seed * 31337 + idx)
        n = int(self._dur[idx] * self.sr)
        t = np.arange(n) / self.sr
        clean = 0.3 * np.sin(2 * np.pi * g.uniform(200, 900) * t) * (np.sin(2 * np.pi * g.uniform(1, 4) * t) > 0)
        noise = g.standard_normal((self.C, n))
        scale = np.sqrt((clean ** 2).mean() / max((noise ** 2).mean(), 1e-9)) * 10 ** (-self.snr / 20)
        delays = [int(c * 2) for c in range(self.C)]
        mix = np.stack([np.roll(clean, d) for d in delays]) + scale * noise
        return torch.as_tensor(mix, dtype=torch.float32), torch.as_tensor(clean, dtype=torch.float32).reshape(1, -1)

    collate_fn = staticmethod(_collate)


def build_audio_to_target_dataloader(config, rank: int = 0, world_size: int = 1):
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn = get("synthetic", None)
    if syn is None and any(get(k, None) is not None for k in ("input_channel_selector", "target_channel_selector", "normalization_signal", "reference_key", "embedding_key")):
        from .data_extra import get_audio_dataset_from_config          # multi-file signals, channel selection, peak normalisation, reference / embedding

        return get_dataloader_from_config(config, get_audio_dataset_from_config(config), rank, world_size)
    ds = SyntheticNoisyDataset(**dict(syn)) if syn is not None else AudioToTargetDataset(
        get("manifest_filepath"), get("sample_rate", 16000), get("input_key", "input_filepath"), get("target_key", "target_filepath"),
        get("audio_duration", None), get("random_offset", False))
    return get_dataloader_from_config(config, ds, rank, world_size)

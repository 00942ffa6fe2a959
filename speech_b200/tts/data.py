"""TTS datasets: ``(text ids, text length, audio, audio length)`` from NeMo-style manifests
(``{"audio_filepath", "text", "duration"[, "speaker"]}``) or a synthetic generator; the vocoder / codec dataset yields audio
only (reference: ``tts/data/text_to_speech_dataset.py``, ``text_to_speech_dataset_lhotse.py``, ``vocoder_dataset.py``)."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from ..data.audio_to_text import get_dataloader_from_config, load_audio, read_manifest


def _collate(batch):
    tl = torch.tensor([len(b[0]) for b in batch], dtype=torch.long)
    al = torch.tensor([b[1].shape[0] for b in batch], dtype=torch.long)
    text = torch.zeros(len(batch), int(tl.max()), dtype=torch.long)
    audio = torch.zeros(len(batch), int(al.max()))
    for i, (t, a) in enumerate(batch):
        text[i, : len(t)] = torch.as_tensor(t, dtype=torch.long)
        audio[i, : a.shape[0]] = a
    return text, tl, audio, al


class TextToSpeechDataset(Dataset):
    def __init__(self, manifest_filepath, tokenizer, sample_rate: int = 22050, min_duration: float = 0.1,
                 max_duration: Optional[float] = None, add_bos_eos: bool = True):
        self.items = read_manifest(manifest_filepath, min_duration=min_duration, max_duration=max_duration)
        self.tok, self.sr, self.add = tokenizer, sample_rate, add_bos_eos
        self.bos, self.eos = int(tokenizer.vocab_size), int(tokenizer.vocab_size) + 1

    def durations(self):
        return [float(it.get("duration", 0.0)) for it in self.items]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, idx):
        it = self.items[idx]
        ids = list(self.tok.text_to_ids(it.get("normalized_text", it["text"])))
        if self.add:
            ids = [self.bos] + ids + [self.eos]
        x = load_audio(it["audio_filepath"], target_sr=self.sr, offset=float(it.get("offset", 0) or 0), duration=it.get("duration"))
        return ids, torch.as_tensor(x, dtype=torch.float32)

    collate_fn = staticmethod(_collate)


class SyntheticTTSDataset(Dataset):
    """Each "character" is rendered as a short tone of its own pitch, so text and audio are monotonically aligned."""

    def __init__(self, num_samples: int, tokenizer, sample_rate: int = 22050, min_chars: int = 3, max_chars: int = 8,
                 seconds_per_char: float = 0.08, seed: int = 0):
        self.n, self.tok, self.sr, self.spc, self.seed = num_samples, tokenizer, sample_rate, seconds_per_char, seed
        g = np.random.default_rng(seed)
        self._len = g.integers(min_chars, max_chars + 1, size=num_samples)
        self.bos, self.eos = int(tokenizer.vocab_size), int(tokenizer.vocab_size) + 1

    def durations(self):
        return (self._len * self.spc).tolist()

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = np.random.default_rng(self.seed * 9973 + idx)
        chars = g.integers(0, 8, size=int(self._len[idx]))
        text = "".join(chr(ord("a") + int(c)) for c in chars)
        n = int(self.spc * self.sr)
        t = np.arange(n) / self.sr
        x = np.concatenate([0.3 * np.sin(2 * np.pi * (220.0 + 90.0 * int(c)) * t) for c in chars]).astype(np.float32)
        ids = [self.bos] + list(self.tok.text_to_ids(text)) + [self.eos]
        return ids, torch.as_tensor(x)

    collate_fn = staticmethod(_collate)


def _collate_audio_only(batch):
    _, _, audio, al = _collate(batch)
    return audio, al


def build_tts_dataloader(config, tokenizer, sample_rate: int = 22050, audio_only: bool = False):
    """``audio_only``: batches are ``(audio, audio_len)`` (vocoder / codec training) instead of ``(text, text_len, audio, audio_len)``."""
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn = get("synthetic", None)
    ds = SyntheticTTSDataset(tokenizer=tokenizer, sample_rate=sample_rate, **dict(syn)) if syn is not None else \
        TextToSpeechDataset(get("manifest_filepath"), tokenizer, sample_rate, get("min_duration", 0.1), get("max_duration", None))
    if audio_only:
        ds.collate_fn = _collate_audio_only
    return get_dataloader_from_config(config, ds, 0, 1)

"""Multi-signal audio datasets for enhancement / separation / target-speaker extraction.  A manifest entry names one or several files
per signal (input, target, reference, embedding); the processor loads the *synchronous* signals (input, target: same offset and
duration, so they stay aligned) and the *asynchronous* ones (a reference or enrolment clip: its own random segment of a fixed
duration), selects channels per signal, concatenates several files of one signal into channels, optionally scales all signals by
the peak of one of them, and loads embedding vectors from ``.npy`` files.
Reference: ``audio/data/audio_to_audio.py`` (``SignalSetup``, ``ASRAudioProcessor``, ``BaseAudioDataset``, ``AudioToTargetDataset``,
``AudioToTargetWithReferenceDataset``, ``AudioToTargetWithEmbeddingDataset``), ``audio/data/audio_to_audio_dataset.py`` (factories).
"""
from __future__ import annotations

import random
from collections import OrderedDict, namedtuple
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Type, Union

import numpy as np
import torch
from torch.utils.data import Dataset

from ..core.config import DictConfig, to_container
from ..data import collections as manifest_collections
from ..data.audio_to_text import load_audio_file


@dataclass
class SignalSetup:
    signals: List[str]                                               # names of the signals of this group
    duration: Optional[Union[float, List[float]]] = None              # seconds to load (one value, or one per signal for async groups)
    channel_selectors: Optional[List[Any]] = None                      # per signal: None (all), an int, a list of ints, or "average"


def _select_channels(x: np.ndarray, selector) -> np.ndarray:
    """``x``: [n, C] → [n, C']."""
    if selector is None:
        return x
    if selector == "average":
        return x.mean(axis=1, keepdims=True)
    if isinstance(selector, int):
        return x[:, [selector]]
    return x[:, list(selector)]


def _read_segment(path: str, sample_rate: int, offset: float, duration: Optional[float], selector=None) -> np.ndarray:
    """[n, C] float32 at ``sample_rate``; a segment running past the end of the file is zero-padded to ``duration``."""
    x, sr = load_audio_file(path)
    x = x.reshape(len(x), -1)
    a = int(round(offset * sr))
    b = len(x) if duration is None else a + int(round(duration * sr))
    seg = x[a:b]
    if sr != sample_rate:
        from ..data.perturb import resample

        seg = np.stack([resample(seg[:, c], sr, sample_rate) for c in range(seg.shape[1])], axis=1)
    if duration is not None:
        want = int(round(duration * sample_rate))
        seg = seg[:want] if len(seg) >= want else np.concatenate([seg, np.zeros((want - len(seg), seg.shape[1]), dtype=seg.dtype)])
    return _select_channels(seg.astype(np.float32), selector)


def _file_duration(path: str) -> float:
    x, sr = load_audio_file(path)
    return len(x) / float(sr)


class ASRAudioProcessor:
    """``process(example)`` → ``OrderedDict`` signal name → tensor ``[C, T]`` (embeddings: ``[D]``)."""

    def __init__(self, sample_rate: float, random_offset: bool, normalization_signal: Optional[str] = None, eps: float = 1e-8, seed: Optional[int] = None):
        self.sample_rate, self.random_offset, self.normalization_signal, self.eps = int(sample_rate), bool(random_offset), normalization_signal, eps
        self.sync_setup: Optional[SignalSetup] = None
        self.async_setup: Optional[SignalSetup] = None
        self.embedding_setup: Optional[SignalSetup] = None
        self._rng = random.Random(seed)

    # ------------------------------------------------------------------ loading
    @staticmethod
    def list_to_multichannel(signal: Union[np.ndarray, List[np.ndarray]]) -> np.ndarray:
        """Several [n, C_i] arrays of one signal → [n, sum C_i] (all files must have the same number of samples)."""
        if not isinstance(signal, list):
            return signal
        if len({len(s) for s in signal}) != 1:
            raise RuntimeError(f"files of one signal differ in length: {[len(s) for s in signal]}")
        return np.concatenate(signal, axis=1)

    @staticmethod
    def get_duration(audio_files: Union[str, List[str]]) -> List[float]:
        return [_file_duration(f) for f in ([audio_files] if isinstance(audio_files, str) else audio_files)]

    def get_samples(self, audio_file: Union[str, List[str]], offset: float, duration: Optional[float], channel_selector=None) -> np.ndarray:
        files = audio_file if isinstance(audio_file, list) else [audio_file]
        segs = [_read_segment(f, self.sample_rate, offset, duration, None) for f in files]
        return _select_channels(self.list_to_multichannel(segs if len(segs) > 1 else segs[0]), channel_selector)

    def get_samples_synchronized(self, audio_files: List[Union[str, List[str]]], channel_selectors: List[Any], sample_rate: int, duration: Optional[float],
                                 fixed_offset: float = 0.0, random_offset: bool = False) -> List[np.ndarray]:
        """One offset for all signals: the example's own offset, plus (with ``random_offset`` and a fixed duration) a random shift that keeps the
        segment inside the shortest file."""
        offset = fixed_offset
        if duration is not None and random_offset:
            flat = [f for fs in audio_files for f in (fs if isinstance(fs, list) else [fs])]
            shortest = min(self.get_duration(flat))
            room = shortest - fixed_offset - duration
            if room > 0:
                offset += self._rng.uniform(0.0, room)
        return [self.get_samples(f, offset, duration, sel) for f, sel in zip(audio_files, channel_selectors)]

    def load_sync_signals(self, example) -> Dict[str, np.ndarray]:
        s = self.sync_setup
        files = [example.audio_files[name] for name in s.signals]
        sels = s.channel_selectors or [None] * len(files)
        dur = s.duration if s.duration is not None else example.duration
        out = self.get_samples_synchronized(files, sels, self.sample_rate, dur, float(example.offset or 0.0), self.random_offset and s.duration is not None)
        return OrderedDict(zip(s.signals, out))

    def load_async_signals(self, example) -> Dict[str, np.ndarray]:
        s = self.async_setup
        durs = s.duration if isinstance(s.duration, (list, tuple)) else [s.duration] * len(s.signals)
        sels = s.channel_selectors or [None] * len(s.signals)
        out = OrderedDict()
        for name, dur, sel in zip(s.signals, durs, sels):
            f = example.audio_files[name]
            off = 0.0
            if dur is not None:
                room = min(self.get_duration(f)) - dur
                if room > 0:
                    off = self._rng.uniform(0.0, room)
            out[name] = self.get_samples(f, off, dur, sel)
        return out

    @staticmethod
    def load_embedding_vector(filepath: str) -> np.ndarray:
        if not filepath.endswith(".npy"):
            raise RuntimeError(f"embedding files must be .npy, got {filepath}")
        return np.load(filepath).astype(np.float32).reshape(-1)

    def load_embedding(self, example) -> Dict[str, np.ndarray]:
        return OrderedDict((name, self.load_embedding_vector(example.audio_files[name])) for name in self.embedding_setup.signals)

    # ------------------------------------------------------------------ processing
    def process_audio(self, audio: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        if self.normalization_signal:
            scale = 1.0 / (float(np.abs(audio[self.normalization_signal]).max()) + self.eps)
            audio = OrderedDict((k, v * scale) for k, v in audio.items())
        return audio

    def process(self, example) -> Dict[str, torch.Tensor]:
        audio = self.load_sync_signals(example) if self.sync_setup else OrderedDict()
        if self.async_setup:
            audio.update(self.load_async_signals(example))
        audio = self.process_audio(audio)
        out = OrderedDict((k, torch.from_numpy(np.ascontiguousarray(v.T))) for k, v in audio.items())          # [C, T]
        if self.embedding_setup:
            out.update((k, torch.from_numpy(v)) for k, v in self.load_embedding(example).items())
        return out


def _audio_collate_fn(batch: List[Dict[str, torch.Tensor]]) -> Tuple[torch.Tensor, ...]:
    """Per signal ``(padded [B, C, T] (or [B, D] for vectors), lengths [B])``, in the order of the example's keys."""
    out: List[torch.Tensor] = []
    for key in batch[0]:
        items = [b[key] for b in batch]
        lens = torch.tensor([it.shape[-1] for it in items], dtype=torch.long)
        if items[0].dim() == 1:
            out += [torch.stack(items), lens]
            continue
        T = int(lens.max())
        out += [torch.stack([torch.nn.functional.pad(it, (0, T - it.shape[-1])) for it in items]), lens]
    return tuple(out)


class BaseAudioDataset(Dataset):
    def __init__(self, collection, audio_processor: ASRAudioProcessor, output_type: Type[tuple]):
        self.collection, self.audio_processor, self.output_type = collection, audio_processor, output_type

    def num_channels(self, signal_key: str) -> int:
        return int(self[0][signal_key].shape[0]) if self[0][signal_key].dim() > 1 else 1

    def durations(self) -> List[float]:
        return [float(e.duration) for e in self.collection]

    def __len__(self):
        return len(self.collection)

    def __getitem__(self, index: int) -> Dict[str, torch.Tensor]:
        return self.audio_processor.process(self.collection[index])

    def _collate_fn(self, batch):
        return self.output_type(*_audio_collate_fn(batch))

    collate_fn = _collate_fn


def _keys(mapping: Dict[str, Any]) -> Dict[str, Any]:
    return {k: v for k, v in mapping.items() if v is not None}


class AudioToTargetDataset(BaseAudioDataset):
    """Batches ``(input_signal, input_length, target_signal, target_length)``."""

    def __init__(self, manifest_filepath, sample_rate: int, input_key: str, target_key: str, audio_duration: Optional[float] = None, random_offset: bool = False,
                 max_duration: Optional[float] = None, min_duration: Optional[float] = None, max_utts: Optional[int] = 0, input_channel_selector=None,
                 target_channel_selector=None, normalization_signal: Optional[str] = None, seed: Optional[int] = None):
        col = manifest_collections.AudioCollection(manifest_filepath, {"input_signal": input_key, "target_signal": target_key}, min_duration=min_duration,
                                                   max_duration=max_duration, max_number=max_utts or None)
        proc = ASRAudioProcessor(sample_rate, random_offset, normalization_signal, seed=seed)
        proc.sync_setup = SignalSetup(["input_signal", "target_signal"], audio_duration, [input_channel_selector, target_channel_selector])
        super().__init__(col, proc, namedtuple("AudioToTargetExample", "input_signal input_length target_signal target_length"))


class AudioToTargetWithReferenceDataset(BaseAudioDataset):
    """Adds a reference signal: synchronous with the input (e.g. the far-end signal of an echo canceller) or, with
    ``reference_is_synchronized=False``, an independent clip of ``reference_duration`` seconds (e.g. an enrolment utterance)."""

    def __init__(self, manifest_filepath, sample_rate: int, input_key: str, target_key: str, reference_key: str, audio_duration: Optional[float] = None,
                 random_offset: bool = False, max_duration=None, min_duration=None, max_utts: Optional[int] = 0, input_channel_selector=None,
                 target_channel_selector=None, reference_channel_selector=None, reference_is_synchronized: bool = True, reference_duration: Optional[float] = None,
                 normalization_signal: Optional[str] = None, seed: Optional[int] = None):
        col = manifest_collections.AudioCollection(manifest_filepath, {"input_signal": input_key, "target_signal": target_key, "reference_signal": reference_key},
                                                   min_duration=min_duration, max_duration=max_duration, max_number=max_utts or None)
        proc = ASRAudioProcessor(sample_rate, random_offset, normalization_signal, seed=seed)
        if reference_is_synchronized:
            proc.sync_setup = SignalSetup(["input_signal", "target_signal", "reference_signal"], audio_duration,
                                          [input_channel_selector, target_channel_selector, reference_channel_selector])
        else:
            proc.sync_setup = SignalSetup(["input_signal", "target_signal"], audio_duration, [input_channel_selector, target_channel_selector])
            proc.async_setup = SignalSetup(["reference_signal"], [reference_duration], [reference_channel_selector])
        super().__init__(col, proc, namedtuple("AudioToTargetWithReferenceExample", "input_signal input_length target_signal target_length reference_signal reference_length"))


class AudioToTargetWithEmbeddingDataset(BaseAudioDataset):
    """Adds an embedding vector stored as ``.npy`` (e.g. the target speaker's embedding)."""

    def __init__(self, manifest_filepath, sample_rate: int, input_key: str, target_key: str, embedding_key: str, audio_duration: Optional[float] = None,
                 random_offset: bool = False, max_duration=None, min_duration=None, max_utts: Optional[int] = 0, input_channel_selector=None,
                 target_channel_selector=None, normalization_signal: Optional[str] = None, seed: Optional[int] = None):
        col = manifest_collections.AudioCollection(manifest_filepath, {"input_signal": input_key, "target_signal": target_key, "embedding_vector": embedding_key},
                                                   min_duration=min_duration, max_duration=max_duration, max_number=max_utts or None)
        proc = ASRAudioProcessor(sample_rate, random_offset, normalization_signal, seed=seed)
        proc.sync_setup = SignalSetup(["input_signal", "target_signal"], audio_duration, [input_channel_selector, target_channel_selector])
        proc.embedding_setup = SignalSetup(["embedding_vector"])
        super().__init__(col, proc, namedtuple("AudioToTargetWithEmbeddingExample", "input_signal input_length target_signal target_length embedding_vector embedding_length"))


# -------------------------------------------------------------------------------------------------------------- factories
def _c(config) -> dict:
    return to_container(config, resolve=True) if isinstance(config, DictConfig) else dict(config)


_COMMON = ("audio_duration", "random_offset", "max_duration", "min_duration", "max_utts", "input_channel_selector", "target_channel_selector", "normalization_signal")


def get_audio_to_target_dataset(config) -> AudioToTargetDataset:
    c = _c(config)
    return AudioToTargetDataset(c["manifest_filepath"], c["sample_rate"], c["input_key"], c["target_key"], **{k: c[k] for k in _COMMON if k in c})


def get_audio_to_target_with_reference_dataset(config) -> AudioToTargetWithReferenceDataset:
    c = _c(config)
    extra = ("reference_channel_selector", "reference_is_synchronized", "reference_duration")
    return AudioToTargetWithReferenceDataset(c["manifest_filepath"], c["sample_rate"], c["input_key"], c["target_key"], c["reference_key"],
                                             **{k: c[k] for k in _COMMON + extra if k in c})


def get_audio_to_target_with_embedding_dataset(config) -> AudioToTargetWithEmbeddingDataset:
    c = _c(config)
    return AudioToTargetWithEmbeddingDataset(c["manifest_filepath"], c["sample_rate"], c["input_key"], c["target_key"], c["embedding_key"],
                                             **{k: c[k] for k in _COMMON if k in c})


def get_audio_dataset_from_config(config):
    """``reference_key`` → with reference, ``embedding_key`` → with embedding, else input / target only; ``None`` without a manifest."""
    c = _c(config)
    if c.get("manifest_filepath") is None:
        return None
    if c.get("reference_key"):
        return get_audio_to_target_with_reference_dataset(c)
    if c.get("embedding_key"):
        return get_audio_to_target_with_embedding_dataset(c)
    return get_audio_to_target_dataset(c)


class CutAudioToTargetDataset(Dataset):
    """The same batches from mini-batches of cuts: the cut's own audio is the input, the target (and optional reference / embedding) comes from
    the paths stored in the cut's custom fields ``target_key`` / ``reference_key`` / ``embedding_key``."""

    def __init__(self, sample_rate: int = 16000, target_key: str = "target_recording", reference_key: Optional[str] = None, embedding_key: Optional[str] = None):
        self.sample_rate, self.target_key, self.reference_key, self.embedding_key = sample_rate, target_key, reference_key, embedding_key

    def _load(self, src, offset=0.0, duration=None) -> torch.Tensor:
        if isinstance(src, (np.ndarray, torch.Tensor)):
            x = np.asarray(src, dtype=np.float32)
            return torch.from_numpy(x.reshape(1, -1) if x.ndim == 1 else x)
        return torch.from_numpy(np.ascontiguousarray(_read_segment(src, self.sample_rate, offset, duration).T))

    def __getitem__(self, cuts):
        batch = []
        for c in cuts:
            x = np.asarray(c.load_audio(self.sample_rate), dtype=np.float32)
            ex = OrderedDict(input_signal=torch.from_numpy(x.reshape(1, -1) if x.ndim == 1 else x))
            ex["target_signal"] = self._load(c.custom[self.target_key], c.offset, c.duration or None)
            if self.reference_key:
                ex["reference_signal"] = self._load(c.custom[self.reference_key])
            if self.embedding_key:
                ex["embedding_vector"] = torch.from_numpy(ASRAudioProcessor.load_embedding_vector(c.custom[self.embedding_key]))
            batch.append(ex)
        return _audio_collate_fn(batch)

"""Speech-to-text datasets, manifests, duration-bucketed batch sampling and dataloader construction.

* NeMo JSON-lines manifests (``audio_filepath``, ``duration``, ``text``, optional ``offset``, ``lang``, ...),
  also sharded path patterns ``file_{0..9}.json`` (reference readers:
  ``nemo/collections/common/data/lhotse/nemo_adapters.py``, ``asr/data/audio_to_text.py``).
* ``AudioToCharDataset`` / ``AudioToBPEDataset`` with the reference collate layout
  ``(audio [B,L], audio_len [B], tokens [B,U], token_len [B])`` (``asr/data/audio_to_text.py:1389``,
  ``audio_to_text_lhotse.py:28-89``).
* ``DynamicBucketingSampler``: batches bounded by total seconds (``batch_duration``, optional
  ``quadratic_duration`` penalty) or by ``batch_size``, drawn from duration buckets (``num_buckets`` /
  ``bucket_duration_bins``), sharded per data-parallel rank with a shared ``shard_seed`` — the sampling
  options of ``LhotseDataLoadingConfig`` (``common/data/lhotse/dataloader.py:71-256,506-743``).
* ``get_dataloader_from_config`` builds a ``torch.utils.data.DataLoader(batch_size=None)`` because the
  sampler yields whole mini-batches (``dataloader.py:372-377``).
* ``SyntheticSpeechDataset``: seeded Gaussian waveforms + uniform token ids of configurable shape, used by
  benchmarks and plumbing tests.
"""
from __future__ import annotations

import glob
import io
import json
import math
import os
import random
import re
import wave
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset

from ..core.config import DictConfig, cfg_get, to_container
from ..utils.logging import logging


# --------------------------------------------------------------------------- manifests / audio IO
def expand_sharded_filepaths(path: Union[str, Sequence[str]]) -> List[str]:
    if not isinstance(path, str):
        out: List[str] = []
        for p in path:
            out.extend(expand_sharded_filepaths(p))
        return out
    path = path.replace("_OP_", "{").replace("_CL_", "}")
    if "," in path and not os.path.exists(path):
        return expand_sharded_filepaths(path.split(","))
    m = re.search(r"\{(\d+)\.\.(\d+)\}", path)
    if m:
        a, b = m.group(1), m.group(2)
        width = len(a) if a.startswith("0") else 0
        return [f for i in range(int(a), int(b) + 1)
                for f in expand_sharded_filepaths(path[: m.start()] + str(i).zfill(width) + path[m.end():])]
    if any(ch in path for ch in "*?["):
        return sorted(glob.glob(path))
    return [path]


def read_manifest(path: Union[str, Sequence[str]], min_duration: Optional[float] = None,
                  max_duration: Optional[float] = None, max_utts: int = 0) -> List[Dict[str, Any]]:
    items = []
    for p in expand_sharded_filepaths(path):
        base = os.path.dirname(os.path.abspath(p))
        with open(p, encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                it = json.loads(line)
                ap = it.get("audio_filepath", it.get("audio_file"))
                if ap is not None and not os.path.isabs(ap) and not os.path.exists(ap):
                    cand = os.path.join(base, ap)
                    ap = cand if os.path.exists(cand) else ap
                it["audio_filepath"] = ap
                if "text" not in it:
                    if "text_filepath" in it:
                        with open(it["text_filepath"], encoding="utf-8") as tf:
                            it["text"] = tf.read().replace("\n", "")
                    else:
                        it["text"] = it.get("normalized_text", "")
                d = it.get("duration")
                if d is not None and ((min_duration and d < min_duration) or (max_duration and d > max_duration)):
                    continue
                items.append(it)
                if max_utts and len(items) >= max_utts:
                    return items
    return items


def write_manifest(path: str, items: List[Dict[str, Any]]) -> None:
    with open(path, "w", encoding="utf-8") as f:
        for it in items:
            f.write(json.dumps(it, ensure_ascii=False) + "\n")


def load_audio(path: str, target_sr: int = 16000, offset: float = 0.0, duration: Optional[float] = None,
               channel_selector: Union[int, str, None] = None) -> np.ndarray:
    """PCM WAV (8/16/24/32-bit int or 32-bit float) or ``.npy`` -> float32 mono at ``target_sr``.  ``path`` may also be a
    binary file object holding a WAV (members of tarred datasets)."""
    if isinstance(path, str) and path.endswith(".npy"):
        x, sr = np.load(path).astype(np.float32), target_sr
    else:
        try:
            with wave.open(path, "rb") as w:
                sr, nch, sw, n = w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()
                start = int(offset * sr)
                w.setpos(min(start, n))
                cnt = n - start if duration is None else min(n - start, int(duration * sr))
                raw = w.readframes(max(cnt, 0))
            if sw == 2:
                x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
            elif sw == 4:
                x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
            elif sw == 1:
                x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
            elif sw == 3:
                b = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 3).astype(np.int32)
                v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
                x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / float(1 << 23)
            else:
                raise ValueError(f"unsupported sample width {sw}")
            x = x.reshape(-1, nch)
            offset, duration = 0.0, None
        except wave.Error:
            from scipy.io import wavfile

            sr, data = wavfile.read(path)
            x = data.astype(np.float32)
            if data.dtype.kind == "i":
                x /= float(np.iinfo(data.dtype).max) + 1.0
            x = x.reshape(len(x), -1)
        if x.shape[1] > 1:
            if channel_selector in (None, "average"):
                x = x.mean(axis=1)
            else:
                x = x[:, int(channel_selector)]
        else:
            x = x[:, 0]
    if offset:
        x = x[int(offset * sr):]
    if duration is not None:
        x = x[: int(duration * sr)]
    if sr != target_sr:
        from scipy.signal import resample_poly

        g = math.gcd(int(sr), int(target_sr))
        x = resample_poly(x, target_sr // g, sr // g).astype(np.float32)
    return np.ascontiguousarray(x, dtype=np.float32)


def save_wav(path: str, samples: np.ndarray, sr: int = 16000) -> None:
    pcm = np.clip(samples, -1.0, 1.0)
    pcm = (pcm * 32767.0).astype("<i2")
    with wave.open(path, "wb") as w:
        w.setnchannels(1 if pcm.ndim == 1 else pcm.shape[1])          # [n] mono or [n, channels] interleaved on write
        w.setsampwidth(2)
        w.setframerate(sr)
        w.writeframes(pcm.tobytes())


# --------------------------------------------------------------------------- datasets
def speech_collate(batch, pad_id: int = 0):
    """[(audio, audio_len, tokens, token_len[, idx])] -> padded tensors."""
    has_idx = len(batch[0]) == 5
    al = torch.tensor([int(b[1]) for b in batch], dtype=torch.long)
    tl = torch.tensor([int(b[3]) for b in batch], dtype=torch.long)
    A = torch.zeros(len(batch), int(al.max()), dtype=torch.float32)
    T = torch.full((len(batch), max(1, int(tl.max()))), pad_id, dtype=torch.long)
    for i, b in enumerate(batch):
        A[i, : al[i]] = torch.as_tensor(b[0][: al[i]])
        T[i, : tl[i]] = torch.as_tensor(b[2][: tl[i]], dtype=torch.long)
    if has_idx:
        return A, al, T, tl, torch.tensor([int(b[4]) for b in batch], dtype=torch.long)
    return A, al, T, tl


class _BaseAudioText(Dataset):
    def __init__(self, manifest_filepath, sample_rate: int = 16000, min_duration=None, max_duration=None, max_utts=0,
                 trim: bool = False, return_sample_id: bool = False, augmentor: Optional[Callable] = None,
                 channel_selector=None, pad_id: int = 0, **_):
        self.items = read_manifest(manifest_filepath, min_duration, max_duration, max_utts)
        self.sample_rate, self.return_sample_id, self.augmentor = sample_rate, return_sample_id, augmentor
        self.channel_selector, self.pad_id = channel_selector, pad_id

    def __len__(self):
        return len(self.items)

    def durations(self) -> List[float]:
        return [float(it.get("duration", 0.0) or 0.0) for it in self.items]

    def tokenize(self, it: Dict[str, Any]) -> List[int]:
        raise NotImplementedError

    def __getitem__(self, idx):
        it = self.items[idx]
        x = load_audio(it["audio_filepath"], self.sample_rate, it.get("offset", 0.0) or 0.0, it.get("duration"),
                       self.channel_selector)
        if self.augmentor is not None:
            x = self.augmentor(x, self.sample_rate)
        toks = self.tokenize(it)
        out = (torch.from_numpy(x), len(x), torch.tensor(toks, dtype=torch.long), len(toks))
        return out + (idx,) if self.return_sample_id else out

    def collate_fn(self, batch):
        return speech_collate(batch, self.pad_id)

    def _collate_fn(self, batch):
        return self.collate_fn(batch)


class AudioToCharDataset(_BaseAudioText):
    def __init__(self, manifest_filepath, labels: List[str], normalize: bool = True, unk_index: int = -1,
                 blank_index: int = -1, **kw):
        super().__init__(manifest_filepath, **kw)
        self.labels = list(labels)
        self._map = {c: i for i, c in enumerate(self.labels)}
        self.normalize, self.unk_index = normalize, unk_index

    def tokenize(self, it):
        text = it["text"].lower() if self.normalize else it["text"]
        ids = []
        for c in text:
            if c in self._map:
                ids.append(self._map[c])
            elif self.unk_index >= 0:
                ids.append(self.unk_index)
        return ids


class AudioToBPEDataset(_BaseAudioText):
    def __init__(self, manifest_filepath, tokenizer, use_start_end_token: bool = False, **kw):
        super().__init__(manifest_filepath, **kw)
        self.tokenizer = tokenizer
        self.use_start_end_token = use_start_end_token

    def tokenize(self, it):
        tok = self.tokenizer
        if hasattr(tok, "langs") and not isinstance(it.get("text"), list):
            ids = tok.text_to_ids(it["text"], it.get("lang", tok.langs[0]))
        else:
            ids = tok.text_to_ids(it["text"])
        if self.use_start_end_token and getattr(tok, "bos_id", -1) is not None and tok.bos_id >= 0:
            ids = [tok.bos_id] + ids + [tok.eos_id]
        return ids


class SyntheticSpeechDataset(Dataset):
    """Seeded synthetic utterances: waveform i.i.d. N(0, 0.1^2) at 16 kHz, duration uniform in
    [min_duration, max_duration], token ids uniform in [0, vocab_size) with ``tokens_per_second`` labels per
    second (or a fixed-range count)."""

    def __init__(self, num_samples: int, vocab_size: int, min_duration: float = 1.0, max_duration: float = 4.0,
                 sample_rate: int = 16000, tokens_per_second: Optional[float] = 3.0, seed: int = 0,
                 max_tokens_frac_of_frames: Optional[float] = None, subsampling: int = 8, hop: float = 0.01,
                 token_low: int = 0, return_sample_id: bool = False):
        g = np.random.default_rng(seed)
        self.durs = g.uniform(min_duration, max_duration, size=num_samples)
        self.seeds = g.integers(0, 2 ** 31 - 1, size=num_samples)
        self.vocab_size, self.sr, self.tps = vocab_size, sample_rate, tokens_per_second
        self.frac, self.subsampling, self.hop = max_tokens_frac_of_frames, subsampling, hop
        self.token_low, self.return_sample_id = token_low, return_sample_id

    def __len__(self):
        return len(self.durs)

    def durations(self):
        return self.durs.tolist()

    def num_tokens(self, idx: int) -> int:
        d = float(self.durs[idx])
        if self.frac is not None:
            frames = int(d / self.hop) // self.subsampling
            hi = max(2, int(frames * self.frac))
            return int(np.random.default_rng(int(self.seeds[idx]) + 1).integers(2, hi + 1))
        return max(1, int(round(d * (self.tps or 3.0))))

    def __getitem__(self, idx):
        g = np.random.default_rng(int(self.seeds[idx]))
        n = int(self.durs[idx] * self.sr)
        x = (g.standard_normal(n) * 0.1).astype(np.float32)
        u = self.num_tokens(idx)
        t = g.integers(self.token_low, self.vocab_size, size=u)
        out = (torch.from_numpy(x), n, torch.from_numpy(t).long(), u)
        return out + (idx,) if self.return_sample_id else out

    def collate_fn(self, batch):
        return speech_collate(batch, 0)


# --------------------------------------------------------------------------- sampling
class DynamicBucketingSampler:
    """Yields lists of dataset indices forming one mini-batch for *this* rank.

    All ranks build the same global sequence of batches from ``shard_seed`` + epoch and take every
    ``world_size``-th one starting at ``rank``, so ranks never overlap and stay in step
    (same number of batches; the tail is dropped to a multiple of world_size).
    """

    def __init__(self, durations: Sequence[float], batch_duration: Optional[float] = None, batch_size: Optional[int] = None,
                 num_buckets: int = 1, bucket_duration_bins: Optional[Sequence[float]] = None,
                 quadratic_duration: Optional[float] = None, shuffle: bool = True, drop_last: bool = False,
                 shard_seed: int = 0, rank: int = 0, world_size: int = 1, max_batch_size: Optional[int] = None,
                 bucket_batch_size: Optional[Sequence[int]] = None):
        if batch_duration is None and batch_size is None and bucket_batch_size is None:
            raise ValueError("one of batch_duration / batch_size / bucket_batch_size is required")
        self.durs = np.asarray(durations, dtype=np.float64)
        self.batch_duration, self.batch_size = batch_duration, batch_size
        self.quadratic_duration, self.shuffle, self.drop_last = quadratic_duration, shuffle, drop_last
        self.seed, self.rank, self.world_size = shard_seed, rank, world_size
        self.max_batch_size = max_batch_size
        self.bucket_batch_size = list(bucket_batch_size) if bucket_batch_size is not None else None
        if bucket_duration_bins is not None:
            self.bins = np.asarray(list(bucket_duration_bins), dtype=np.float64)
        elif num_buckets > 1:
            self.bins = estimate_duration_bins(self.durs, num_buckets)
        else:
            self.bins = np.asarray([], dtype=np.float64)
        self.bucket_of = np.searchsorted(self.bins, self.durs, side="right")
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def _cost(self, d: float) -> float:
        if self.quadratic_duration:
            return d + d * d / self.quadratic_duration
        return d

    def _global_batches(self) -> List[List[int]]:
        rng = np.random.default_rng(self.seed + 7919 * self.epoch)
        batches: List[List[int]] = []
        for b in range(len(self.bins) + 1):
            idx = np.nonzero(self.bucket_of == b)[0]
            if len(idx) == 0:
                continue
            if self.shuffle:
                rng.shuffle(idx)
            else:
                idx = idx[np.argsort(self.durs[idx], kind="stable")]
            cur: List[int] = []
            longest = 0.0
            fixed = self.bucket_batch_size[b] if self.bucket_batch_size is not None else self.batch_size
            for i in idx:
                d = float(self.durs[i])
                if self.batch_duration is not None and fixed is None:
                    new_longest = max(longest, d)
                    # padded cost: every utterance is padded to the longest one in the batch
                    if cur and self._cost(new_longest) * (len(cur) + 1) > self.batch_duration or \
                            (self.max_batch_size and len(cur) >= self.max_batch_size):
                        batches.append(cur)
                        cur, new_longest = [], d
                    longest = new_longest
                    cur.append(int(i))
                else:
                    cur.append(int(i))
                    if len(cur) >= fixed:
                        batches.append(cur)
                        cur = []
            if cur and not self.drop_last:
                batches.append(cur)
        if self.shuffle:
            order = rng.permutation(len(batches))
            batches = [batches[i] for i in order]
        n = len(batches) // self.world_size * self.world_size
        return batches[:n] if self.world_size > 1 else batches

    def __iter__(self) -> Iterator[List[int]]:
        gb = self._global_batches()
        for k in range(self.rank, len(gb), self.world_size):
            yield gb[k]

    def __len__(self) -> int:
        return len(self._global_batches()) // self.world_size


def estimate_duration_bins(durations: Sequence[float], num_buckets: int) -> np.ndarray:
    """Bin edges that give every bucket roughly the same total audio duration
    (reference: ``scripts/speech_recognition/estimate_duration_bins.py``)."""
    d = np.sort(np.asarray(durations, dtype=np.float64))
    if num_buckets <= 1 or len(d) == 0:
        return np.asarray([], dtype=np.float64)
    csum = np.cumsum(d)
    targets = csum[-1] * np.arange(1, num_buckets) / num_buckets
    return np.unique(d[np.searchsorted(csum, targets).clip(max=len(d) - 1)])


class _BatchedView(Dataset):
    def __init__(self, dataset, batches: Callable[[], Iterator[List[int]]], collate):
        self.dataset, self.collate = dataset, collate
        self._batches = list(batches())

    def __len__(self):
        return len(self._batches)

    def __getitem__(self, k):
        return self.collate([self.dataset[i] for i in self._batches[k]])


class BatchedLoader:
    """Re-creatable iterable over sampler batches with worker processes and pinned memory."""

    def __init__(self, dataset, sampler: DynamicBucketingSampler, collate, num_workers: int = 0, pin_memory: bool = False,
                 prefetch_factor: Optional[int] = None):
        self.dataset, self.sampler, self.collate = dataset, sampler, collate
        self.num_workers, self.pin_memory, self.prefetch_factor = num_workers, pin_memory, prefetch_factor
        self.batch_size = None
        self._epoch = 0

    def __len__(self):
        return len(self.sampler)

    def __iter__(self):
        self.sampler.set_epoch(self._epoch)
        self._epoch += 1
        view = _BatchedView(self.dataset, lambda: iter(self.sampler), self.collate)
        kw = {}
        if self.num_workers > 0 and self.prefetch_factor:
            kw["prefetch_factor"] = self.prefetch_factor
        dl = DataLoader(view, batch_size=None, shuffle=False, num_workers=self.num_workers,
                        pin_memory=self.pin_memory and torch.cuda.is_available(), **kw)
        return iter(dl)


def get_dataloader_from_config(config, dataset, global_rank: int = 0, world_size: int = 1):
    """Build the loader described by a ``train_ds`` / ``validation_ds`` block."""
    c = to_container(config, resolve=True) if isinstance(config, DictConfig) else dict(config)
    durs = dataset.durations() if hasattr(dataset, "durations") else [1.0] * len(dataset)
    collate = getattr(dataset, "collate_fn", None) or speech_collate
    use_bucketing = c.get("batch_duration") is not None or c.get("use_bucketing", False) or c.get("num_buckets", 0) > 1
    if use_bucketing or c.get("use_lhotse", False):
        sampler = DynamicBucketingSampler(
            durs, batch_duration=c.get("batch_duration"), batch_size=c.get("batch_size") if c.get("batch_duration") is None else None,
            num_buckets=c.get("num_buckets", 1) or 1, bucket_duration_bins=c.get("bucket_duration_bins"),
            quadratic_duration=c.get("quadratic_duration"), shuffle=c.get("shuffle", False),
            drop_last=c.get("drop_last", False), shard_seed=c.get("shard_seed", c.get("seed", 0)) if not isinstance(c.get("shard_seed"), str) else 0,
            rank=global_rank, world_size=world_size, max_batch_size=c.get("max_batch_size"),
            bucket_batch_size=c.get("bucket_batch_size"))
    else:
        sampler = DynamicBucketingSampler(durs, batch_size=c.get("batch_size", 1), num_buckets=1,
                                          shuffle=c.get("shuffle", False), drop_last=c.get("drop_last", False),
                                          shard_seed=c.get("seed", 0), rank=global_rank, world_size=world_size)
    return BatchedLoader(dataset, sampler, collate, num_workers=c.get("num_workers", 0), pin_memory=c.get("pin_memory", False),
                         prefetch_factor=c.get("prefetch_factor"))


def build_speech_dataset(config, tokenizer=None, labels=None, global_rank=0, world_size=1):
    """Pick the dataset class from the config: synthetic, BPE (tokenizer given) or character."""
    c = to_container(config, resolve=True) if isinstance(config, DictConfig) else dict(config)
    common = dict(sample_rate=c.get("sample_rate", 16000), min_duration=c.get("min_duration"),
                  max_duration=c.get("max_duration"), max_utts=c.get("max_utts", 0),
                  return_sample_id=c.get("return_sample_id", False), channel_selector=c.get("channel_selector"))
    if c.get("synthetic") is not None:
        s = dict(c["synthetic"])
        return SyntheticSpeechDataset(return_sample_id=c.get("return_sample_id", False), **s)
    if c.get("manifest_filepath") is None:
        return None
    if tokenizer is not None:
        return AudioToBPEDataset(c["manifest_filepath"], tokenizer, use_start_end_token=c.get("use_start_end_token", False), **common)
    return AudioToCharDataset(c["manifest_filepath"], labels=labels or c.get("labels"), normalize=c.get("normalize_transcripts", False)
                              or c.get("normalize", False), unk_index=c.get("unk_index", -1), **common)


def load_audio_file(path) -> Tuple[np.ndarray, int]:
    """Samples at the file's own rate: float32 ``[n]`` (mono) or ``[n, channels]``, and the sample rate."""
    if isinstance(path, str) and path.endswith(".npy"):
        return np.load(path).astype(np.float32), 16000
    from scipy.io import wavfile

    sr, data = wavfile.read(path)
    x = data.astype(np.float32)
    if data.dtype.kind == "i":
        x /= float(np.iinfo(data.dtype).max) + 1.0
    elif data.dtype.kind == "u":
        x = (x - 128.0) / 128.0
    return x, int(sr)

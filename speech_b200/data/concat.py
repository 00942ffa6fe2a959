"""Combining datasets: ``ConcatDataset`` (iterable; round-robin, temperature-weighted or fixed-probability sampling over child
datasets with per-rank / per-worker partitioning), ``ConcatMapDataset`` (map-style with a precomputed index schedule),
``CodeSwitchedDataset`` (utterances of several monolingual corpora joined into one synthetic code-switched utterance), and
``FallbackDataset`` (an item that fails to load is replaced by the previous good one).

References: ``common/data/dataset.py`` (``ConcatDataset``, ``ConcatMapDataset``, ``CodeSwitchedDataset``), ``common/data/fallback.py``.
"""
from __future__ import annotations

from typing import Any, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset, IterableDataset, get_worker_info

__all__ = ["CodeSwitchedDataset", "ConcatDataset", "ConcatMapDataset", "FallbackDataset"]


def _sampling_probabilities(sizes: Sequence[int], technique: str, temperature: float, probabilities: Optional[Sequence[float]]) -> np.ndarray:
    if technique == "temperature":
        p = np.asarray(sizes, dtype=np.float64)
        p = (p / p.sum()) ** (1.0 / temperature)
        return p / p.sum()
    if technique == "random":
        if probabilities is None or len(probabilities) != len(sizes):
            raise ValueError("sampling_technique='random' needs one probability per dataset")
        p = np.asarray(probabilities, dtype=np.float64)
        return p / p.sum()
    raise ValueError(f"unknown sampling technique {technique!r}")


def _schedule(sizes: Sequence[int], technique: str, temperature: float, probabilities, seed: int) -> List[Tuple[int, int]]:
    """``(dataset, item)`` pairs of one epoch.  ``round-robin`` visits the datasets in turn until the largest is exhausted (smaller
    ones wrap around); the sampling techniques draw ``sum(sizes)`` items, each dataset cycling through a permutation of itself."""
    rng = np.random.default_rng(seed)
    if technique == "round-robin":
        n = max(sizes)
        return [(d, k % sizes[d]) for k in range(n) for d in range(len(sizes)) if sizes[d] > 0]
    p = _sampling_probabilities(sizes, technique, temperature, probabilities)
    perms = [rng.permutation(s) for s in sizes]
    pos = [0] * len(sizes)
    out = []
    for d in rng.choice(len(sizes), size=int(sum(sizes)), p=p):
        if pos[d] == sizes[d]:
            perms[d], pos[d] = rng.permutation(sizes[d]), 0
        out.append((int(d), int(perms[d][pos[d]])))
        pos[d] += 1
    return out


class ConcatMapDataset(Dataset):
    def __init__(self, datasets: Sequence[Dataset], sampling_technique: str = "temperature", sampling_temperature: float = 5.0,
                 sampling_probabilities: Optional[Sequence[float]] = None, seed: int = 0):
        self.datasets = list(datasets)
        self.sizes = [len(d) for d in self.datasets]
        self.indices = _schedule(self.sizes, sampling_technique, sampling_temperature, sampling_probabilities, seed)

    def __len__(self):
        return len(self.indices)

    def __getitem__(self, i):
        d, k = self.indices[i]
        return self.datasets[d][k]


class ConcatDataset(IterableDataset):
    """Map-style children are indexed through the schedule; iterable children are consumed in schedule order.  With
    ``global_rank`` / ``world_size`` and data-loader workers, every consumer takes every n-th item of the schedule, so that the
    union over ranks and workers is one epoch."""

    def __init__(self, datasets: Sequence, shuffle: bool = True, sampling_technique: str = "temperature", sampling_temperature: float = 5.0,
                 sampling_scale: int = 1, sampling_probabilities: Optional[Sequence[float]] = None, seed: int = 0, global_rank: int = 0, world_size: int = 1):
        self.datasets, self.shuffle = list(datasets), shuffle
        self.technique, self.temperature, self.scale, self.probs = sampling_technique, sampling_temperature, max(1, sampling_scale), sampling_probabilities
        self.seed, self.rank, self.world = seed, global_rank, world_size
        self.epoch = 0
        self.sizes = [len(d) if hasattr(d, "__len__") else 0 for d in self.datasets]

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        n = (max(self.sizes) * len(self.sizes) if self.technique == "round-robin" else sum(self.sizes)) * self.scale
        return n // self.world

    def __iter__(self) -> Iterator[Any]:
        info = get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        sched = []
        for k in range(self.scale):
            sched += _schedule(self.sizes, self.technique, self.temperature, self.probs, self.seed + 1000 * self.epoch + k)
        stride, offset = self.world * nw, self.rank * nw + wid
        iters = [iter(d) if not hasattr(d, "__getitem__") else None for d in self.datasets]
        for j in range(offset, len(sched), stride):
            d, k = sched[j]
            if iters[d] is None:
                yield self.datasets[d][k]
            else:
                try:
                    yield next(iters[d])
                except StopIteration:
                    iters[d] = iter(self.datasets[d])
                    yield next(iters[d])


class CodeSwitchedDataset(IterableDataset):
    """Children yield ``(audio [T], audio_len, tokens [U], token_len)``.  One output sample joins utterances drawn from the children
    (by ``lang_probs``) until adding another would exceed ``max_duration`` seconds and at least ``min_duration`` is reached (at
    least ``min_monolingual`` of the samples come from a single child); utterances are level-normalised to ``db_norm`` dBFS,
    separated by pauses, and their token sequences are concatenated.  With ``return_lang_ids`` a fifth element holds the child
    index of every token."""

    def __init__(self, datasets: Sequence, lang_probs: Optional[Sequence[float]] = None, shuffle: bool = True, min_duration: float = 4.0, max_duration: float = 20.0,
                 min_monolingual: float = 0.3, db_norm: float = -25.0, pause_start: float = 0.0, pause_join: float = 0.0, pause_end: float = 0.0,
                 sample_rate: int = 16000, seed: int = 0, global_rank: int = 0, world_size: int = 1, return_lang_ids: bool = False, infinity_mode: bool = False):
        self.datasets = list(datasets)
        n = len(self.datasets)
        p = np.asarray(lang_probs if lang_probs is not None else [1.0 / n] * n, dtype=np.float64)
        if len(p) != n or abs(p.sum() - 1.0) > 1e-6:
            raise ValueError("lang_probs needs one probability per dataset and must sum to one")
        self.p, self.min_d, self.max_d, self.mono, self.db = p, min_duration, max_duration, min_monolingual, db_norm
        self.pauses, self.sr, self.seed, self.rank, self.world = (pause_start, pause_join, pause_end), sample_rate, seed, global_rank, world_size
        self.ret_ids, self.infinite = return_lang_ids, infinity_mode
        self.epoch = 0

    def _norm(self, x: torch.Tensor) -> torch.Tensor:
        rms = x.pow(2).mean().sqrt().clamp(min=1e-9)
        return x * (10 ** (self.db / 20.0) / rms)

    def __iter__(self):
        info = get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        rng = np.random.default_rng(self.seed + 7919 * self.epoch + 31 * (self.rank * nw + wid))
        iters = [iter(d) for d in self.datasets]
        live = [True] * len(iters)

        def draw(lang):
            try:
                return next(iters[lang])
            except StopIteration:
                if not self.infinite:
                    live[lang] = False
                    return None
                iters[lang] = iter(self.datasets[lang])
                return next(iters[lang])

        zeros = lambda sec: torch.zeros(int(sec * self.sr))  # noqa: E731
        while any(live):
            mono = rng.random() < self.mono
            fixed = int(rng.choice(len(self.p), p=self.p)) if mono else None
            audio, toks, ids, dur = [zeros(self.pauses[0])], [], [], 0.0
            while dur < self.min_d:
                lang = fixed if fixed is not None else int(rng.choice(len(self.p), p=self.p))
                if not live[lang]:
                    if not any(live):
                        break
                    lang = int(np.nonzero(live)[0][0])
                item = draw(lang)
                if item is None:
                    continue
                a, al, t, tl = item[:4]
                a, t = torch.as_tensor(a)[: int(al)].float(), torch.as_tensor(t)[: int(tl)]
                d = a.numel() / self.sr
                if dur + d > self.max_d and dur > 0:
                    break
                if toks:
                    audio.append(zeros(self.pauses[1]))
                audio.append(self._norm(a))
                toks.append(t)
                ids.append(torch.full_like(t, lang))
                dur += d
            if not toks:
                return
            audio.append(zeros(self.pauses[2]))
            x, y = torch.cat(audio).clamp(-1, 1), torch.cat(toks)
            out = (x, torch.tensor(x.numel()), y, torch.tensor(y.numel()))
            yield out + (torch.cat(ids),) if self.ret_ids else out


class FallbackDataset(Dataset):
    """Wraps a map-style dataset: when loading an item raises (or returns ``None``), the last item that loaded is returned instead,
    and the failure is counted — one broken file should not end a run."""

    def __init__(self, dataset: Dataset):
        self.dataset = dataset
        self._last: Any = None
        self.failures = 0

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, i):
        try:
            item = self.dataset[i]
        except Exception:  # noqa: BLE001  (whatever a decoder throws)
            item = None
        if item is None:
            self.failures += 1
            if self._last is None:
                raise RuntimeError(f"item {i} failed to load and there is no earlier item to fall back to")
            return self._last
        self._last = item
        return item

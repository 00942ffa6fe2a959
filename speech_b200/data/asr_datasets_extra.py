"""The rest of the map-style / iterable ASR datasets and the factory functions that pick one from a dataloader config:
tarred audio (character / BPE / label) with shard scatter or replication and a shuffle buffer, bucketed chains with
per-bucket batch sizes, self-supervised audio+noise items, feature-manifest datasets, datasets over in-memory or
Hugging-Face style records, and the prediction writer that gathers transcripts of a distributed ``predict`` run.
Reference: ``asr/data/audio_to_text.py`` (``_TarredAudioToTextDataset``, ``BucketingDataset``, ``RandomizedChainDataset``),
``asr/data/audio_to_text_dataset.py``, ``asr/data/ssl_dataset.py``, ``asr/data/feature_to_text.py``,
``asr/data/huggingface/hf_audio_to_text.py``, ``asr/data/audio_to_label_dataset.py``.
"""
from __future__ import annotations

import io
import json
import os
import random
import tarfile
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Union

import numpy as np
import torch
from torch.utils.data import ChainDataset, Dataset, IterableDataset

from ..core.config import DictConfig, to_container
from .audio_to_text import (AudioToBPEDataset, AudioToCharDataset, expand_sharded_filepaths, load_audio, read_manifest,
                            speech_collate)
from .concat import CodeSwitchedDataset, ConcatDataset


def _plain(cfg) -> dict:
    return to_container(cfg, resolve=True) if isinstance(cfg, DictConfig) else dict(cfg)


# ---------------------------------------------------------------------------------------------------------------- shards
def shard_filepaths(paths: Union[str, Sequence[str]], shard_strategy: str = "scatter", world_size: int = 1, global_rank: int = 0) -> List[str]:
    """Brace-expanded shard list for this rank: ``scatter`` gives every rank a contiguous, equal slice (the shard count must
    divide by the world size), ``replicate`` gives every rank all shards."""
    files = expand_sharded_filepaths(paths)
    if shard_strategy not in ("scatter", "replicate"):
        raise ValueError(f"shard_strategy must be 'scatter' or 'replicate', got {shard_strategy!r}")
    if shard_strategy == "replicate" or world_size <= 1:
        return files
    if len(files) % world_size != 0:
        raise ValueError(f"{len(files)} shards cannot be scattered evenly over {world_size} ranks")
    per = len(files) // world_size
    return files[global_rank * per:(global_rank + 1) * per]


def shard_manifests_if_needed(manifest_filepaths, shard_strategy: str, shard_manifests: bool, global_rank: int, world_size: int):
    """With one manifest per shard (``shard_manifests``), a rank reads only the manifests of its own shards."""
    if shard_manifests and world_size > 1:
        return shard_filepaths(manifest_filepaths, shard_strategy, world_size, global_rank)
    return manifest_filepaths


class _TarredAudio(IterableDataset):
    """Audio stored as members of tar shards, the transcripts in a JSON-lines manifest keyed by file stem.  A member named
    ``<stem>-sub<k>.<ext>`` repeats the manifest entry ``<stem>`` (how duplicated files appear inside one shard).  Workers of
    a loader split the rank's shards between them; ``shuffle_n`` holds that many samples in a buffer and draws from it at
    random."""

    def __init__(self, audio_tar_filepaths, manifest_filepath, sample_rate: int = 16000, shuffle_n: int = 0, min_duration=None,
                 max_duration=None, max_utts: int = 0, shard_strategy: str = "scatter", shard_manifests: bool = False, global_rank: int = 0,
                 world_size: int = 1, return_sample_id: bool = False, augmentor: Optional[Callable] = None, pad_id: int = 0, seed: int = 0, **_):
        manifest_filepath = shard_manifests_if_needed(manifest_filepath, shard_strategy, shard_manifests, global_rank, world_size)
        self.items = read_manifest(manifest_filepath, min_duration, max_duration, max_utts)
        self.index = {os.path.splitext(os.path.basename(it["audio_filepath"]))[0]: k for k, it in enumerate(self.items)}
        self.tars = shard_filepaths(audio_tar_filepaths, shard_strategy, world_size, global_rank)
        self.sample_rate, self.shuffle_n, self.return_sample_id = sample_rate, int(shuffle_n), return_sample_id
        self.augmentor, self.pad_id, self.seed, self.epoch = augmentor, pad_id, seed + global_rank, 0
        # samples this rank will see: with scattered shards and a full manifest only the entries of its shards count
        self._len = len(self.items) if (shard_strategy == "replicate" or world_size <= 1 or shard_manifests) else len(self.items) // world_size

    def __len__(self):
        return self._len

    def set_epoch(self, epoch: int):
        self.epoch = int(epoch)

    def target(self, it: Dict[str, Any]):
        raise NotImplementedError

    def _build(self, it, x, k):
        if self.augmentor is not None:
            x = self.augmentor(x, self.sample_rate)
        tgt = self.target(it)
        out = (torch.from_numpy(np.ascontiguousarray(x)), len(x), torch.as_tensor(tgt, dtype=torch.long), len(tgt) if hasattr(tgt, "__len__") else 1)
        return out + (k,) if self.return_sample_id else out

    def _stream(self) -> Iterator:
        info = torch.utils.data.get_worker_info()
        tars = self.tars if info is None else self.tars[info.id::info.num_workers]
        for t in tars:
            with tarfile.open(t) as tf:
                for member in tf:
                    if not member.isfile():
                        continue
                    stem = os.path.splitext(os.path.basename(member.name))[0]
                    base = stem.rsplit("-sub", 1)[0] if "-sub" in stem else stem
                    k = self.index.get(base)
                    if k is None:
                        continue
                    it = self.items[k]
                    x = np.asarray(load_audio(io.BytesIO(tf.extractfile(member).read()), self.sample_rate, it.get("offset", 0.0) or 0.0,
                                              it.get("duration") if it.get("offset") else None), dtype=np.float32)
                    yield self._build(it, x, k)

    def __iter__(self):
        if self.shuffle_n <= 1:
            yield from self._stream()
            return
        rng = random.Random(self.seed * 7919 + self.epoch)
        buf: List[Any] = []
        for s in self._stream():
            if len(buf) < self.shuffle_n:
                buf.append(s)
                continue
            j = rng.randrange(len(buf))
            buf[j], s = s, buf[j]
            yield s
        rng.shuffle(buf)
        yield from buf

    def collate_fn(self, batch):
        return speech_collate(batch, self.pad_id)

    _collate_fn = collate_fn


class TarredAudioToCharDataset(_TarredAudio):
    def __init__(self, audio_tar_filepaths, manifest_filepath, labels: Sequence[str], normalize: bool = True, unk_index: int = -1, **kw):
        super().__init__(audio_tar_filepaths, manifest_filepath, **kw)
        self._map = {c: i for i, c in enumerate(labels)}
        self.labels, self.normalize, self.unk_index = list(labels), normalize, unk_index

    def target(self, it):
        text = it["text"].lower() if self.normalize else it["text"]
        return [self._map[c] if c in self._map else self.unk_index for c in text if c in self._map or self.unk_index >= 0]


class TarredAudioToBPEDataset(_TarredAudio):
    def __init__(self, audio_tar_filepaths, manifest_filepath, tokenizer, use_start_end_token: bool = False, **kw):
        super().__init__(audio_tar_filepaths, manifest_filepath, **kw)
        self.tokenizer, self.use_start_end_token = tokenizer, use_start_end_token

    def target(self, it):
        return AudioToBPEDataset.tokenize(self, it)


class TarredAudioToClassificationLabelDataset(_TarredAudio):
    """One class label per file (``label`` field); batches are (audio, lengths, labels, label lengths)."""

    def __init__(self, audio_tar_filepaths, manifest_filepath, labels: Sequence[str], **kw):
        super().__init__(audio_tar_filepaths, manifest_filepath, **kw)
        self.labels = list(labels)
        self._map = {str(c): i for i, c in enumerate(labels)}

    def target(self, it):
        return [self._map[str(it["label"])]]

    def collate_fn(self, batch):
        a, al, t, tl = speech_collate([b[:4] for b in batch], self.pad_id)[:4]
        return a, al, t.reshape(-1), tl


class TarredAudioToSpeechLabelDataset(TarredAudioToClassificationLabelDataset):
    """Speaker-label variant: when ``window_length_in_sec`` is given, a file is cut into windows with ``shift_length_in_sec``
    hop and every window carries the file's label."""

    def __init__(self, *a, window_length_in_sec: Optional[float] = None, shift_length_in_sec: float = 1.0, **kw):
        super().__init__(*a, **kw)
        self.window, self.shift = window_length_in_sec, shift_length_in_sec

    def collate_fn(self, batch):
        if not self.window:
            return super().collate_fn(batch)
        w, h = int(self.window * self.sample_rate), int(self.shift * self.sample_rate)
        xs, ys = [], []
        for b in batch:
            x, y = b[0], int(b[2][0])
            if len(x) < w:
                x = torch.nn.functional.pad(x, (0, w - len(x)))
            for s in range(0, len(x) - w + 1, h):
                xs.append(x[s:s + w])
                ys.append(y)
        n = len(xs)
        return torch.stack(xs), torch.full((n,), w, dtype=torch.long), torch.tensor(ys), torch.ones(n, dtype=torch.long)


# ------------------------------------------------------------------------------------------------------------- bucketing
class BucketingDataset(IterableDataset):
    """Groups the samples of an iterable dataset into lists of ``bucketing_batch_size`` (the loader then runs with batch size 1 and
    the collate function receives one such list)."""

    def __init__(self, dataset: IterableDataset, bucketing_batch_size: int):
        self.wrapped_dataset, self.bucketing_batch_size = dataset, int(bucketing_batch_size)

    def _collate_fn(self, batch):
        return self.wrapped_dataset.collate_fn(batch[0])

    collate_fn = _collate_fn

    def __iter__(self):
        group: List[Any] = []
        for s in self.wrapped_dataset:
            group.append(s)
            if len(group) == self.bucketing_batch_size:
                yield group
                group = []
        if group:
            yield group

    def __len__(self):
        return -(-len(self.wrapped_dataset) // self.bucketing_batch_size)


class RandomizedChainDataset(ChainDataset):
    """Chains the buckets in an order drawn anew from a seeded generator every time it is iterated."""

    def __init__(self, datasets: Iterable[Dataset], rnd_seed: int = 0):
        super().__init__(list(datasets))
        self.rnd_gen = np.random.RandomState(rnd_seed)

    def __iter__(self):
        for k in self.rnd_gen.permutation(len(self.datasets)):
            yield from self.datasets[k]

    def __len__(self):
        return sum(len(d) for d in self.datasets)


def convert_to_config_list(initial) -> List[List[str]]:
    """Manifest / tar paths as a list of lists, one inner list per bucket.  A comma-separated string or a flat list is one bucket."""
    if isinstance(initial, str):
        initial = initial.split(",")
    initial = list(initial) if initial is not None else []
    if not initial:
        raise ValueError("manifest_filepaths and tarred_audio_filepaths must not be empty")
    nested = [isinstance(v, (list, tuple)) or (hasattr(v, "__iter__") and not isinstance(v, str)) for v in initial]
    if any(nested) and not all(nested):
        raise ValueError("paths must be either a list of strings or a list of lists of strings (one per bucket)")
    return [list(v) for v in initial] if all(nested) else [initial]


def calc_bucketing_batch_sizes(ds_config, datasets_len: int) -> List[int]:
    """Per-bucket batch sizes: an integer scales linearly (bucket i of n gets ``(n - i) * size``, shorter audio → larger batch); a
    list assigns them; ``bucketing_weights`` repeats entry i that many times for up-sampled buckets."""
    size, weights = ds_config["bucketing_batch_size"], ds_config.get("bucketing_weights")
    if ds_config["batch_size"] != 1:
        raise ValueError(f"batch_size must be 1 when bucketing_batch_size is set (got {ds_config['batch_size']})")
    if isinstance(size, int):
        n = len(weights) if weights else datasets_len
        per = [(n - i) * size for i in range(n)]
    elif isinstance(size, (list, tuple)) or hasattr(size, "__iter__"):
        per = [int(v) for v in size]
    else:
        raise ValueError(f"bucketing_batch_size must be an int or a list, got {type(size).__name__}")
    out = [b for b, w in zip(per, weights) for _ in range(int(w))] if weights else per
    if len(out) != datasets_len:
        raise ValueError(f"{len(out)} batch sizes for {datasets_len} buckets")
    return out


def get_chain_dataset(datasets: List[Dataset], ds_config, rank: int = 0):
    """One dataset out of the buckets: ``fixed_order`` chains them, ``synced_randomized`` permutes the order with the same seed on
    every rank, ``fully_randomized`` with a seed of its own per rank."""
    datasets = list(datasets)
    if len(datasets) > 1 and ds_config.get("bucketing_batch_size") is not None:
        sizes = calc_bucketing_batch_sizes(ds_config, len(datasets))
        datasets = [BucketingDataset(d, b) for d, b in zip(datasets, sizes)]
    if len(datasets) == 1:
        return datasets[0]
    strategy = ds_config.get("bucketing_strategy", "synced_randomized")
    if strategy == "fixed_order":
        return ChainDataset(datasets)
    if strategy == "synced_randomized":
        return RandomizedChainDataset(datasets, rnd_seed=0)
    if strategy == "fully_randomized":
        return RandomizedChainDataset(datasets, rnd_seed=random.randint(0, 30000) + rank)
    raise ValueError(f"bucketing_strategy={strategy!r}: choose fixed_order, synced_randomized or fully_randomized")


# -------------------------------------------------------------------------------------------------------------- factories
def inject_dataloader_value_from_model_config(model_cfg, dataloader_cfg, key: str) -> None:
    """Copy ``model_cfg[key]`` into the dataloader config when the model defines it (the model's value wins, with a notice if the
    dataloader config held a different one)."""
    if key not in model_cfg or model_cfg[key] is None:
        return
    if key in dataloader_cfg and dataloader_cfg[key] is not None and dataloader_cfg[key] != model_cfg[key]:
        from ..utils.logging import logging

        logging.warning("'%s' is %r in the dataloader config and %r in the model config; the model's value is used", key, dataloader_cfg[key], model_cfg[key])
    dataloader_cfg[key] = model_cfg[key]


def _common(c: dict, augmentor) -> dict:
    return dict(sample_rate=c.get("sample_rate", 16000), min_duration=c.get("min_duration"), max_duration=c.get("max_duration"),
                max_utts=c.get("max_utts", 0), return_sample_id=c.get("return_sample_id", False), channel_selector=c.get("channel_selector"),
                augmentor=augmentor, trim=c.get("trim_silence", False))


def get_char_dataset(config, augmentor=None) -> AudioToCharDataset:
    c = _plain(config)
    if "labels" not in c:
        raise ValueError("a character dataset needs 'labels' in its config")
    return AudioToCharDataset(c["manifest_filepath"], labels=c["labels"], normalize=c.get("normalize_transcripts", c.get("normalize", False)),
                              unk_index=c.get("unk_index", -1), **_common(c, augmentor))


def get_bpe_dataset(config, tokenizer, augmentor=None) -> AudioToBPEDataset:
    c = _plain(config)
    return AudioToBPEDataset(c["manifest_filepath"], tokenizer, use_start_end_token=c.get("use_start_end_token", True), **_common(c, augmentor))


def _concat(make, c: dict, global_rank: int, world_size: int):
    parts = []
    for m in c["manifest_filepath"]:
        parts.append(make({**c, "manifest_filepath": m}))
    return ConcatDataset(parts, shuffle=c.get("concat_shuffle", True), sampling_technique=c.get("concat_sampling_technique", "temperature"),
                         sampling_temperature=c.get("concat_sampling_temperature", 5), sampling_probabilities=c.get("concat_sampling_probabilities"),
                         sampling_scale=c.get("concat_sampling_scale", 1), seed=c.get("concat_sampling_seed") or 0, global_rank=global_rank, world_size=world_size)


def get_concat_char_dataset(config, global_rank: int = 0, world_size: int = 1, augmentor=None):
    c = _plain(config)
    return _concat(lambda cc: get_char_dataset(cc, augmentor), c, global_rank, world_size)


def get_concat_bpe_dataset(config, tokenizer, global_rank: int = 0, world_size: int = 1, augmentor=None):
    c = _plain(config)
    return _concat(lambda cc: get_bpe_dataset(cc, tokenizer, augmentor), c, global_rank, world_size)


def get_tarred_dataset(config, shuffle_n: int, global_rank: int, world_size: int, tokenizer=None, augmentor=None):
    """One tarred dataset per bucket (``tarred_audio_filepaths`` / ``manifest_filepath`` lists of lists), chained per the bucketing
    strategy.  ``bucketing_weights`` repeats a bucket that many times."""
    c = _plain(config)
    tars, mans = convert_to_config_list(c["tarred_audio_filepaths"]), convert_to_config_list(c["manifest_filepath"])
    weights = c.get("bucketing_weights")
    if weights is not None and (len(weights) != len(mans) or any(not isinstance(w, int) or w <= 0 for w in weights)):
        raise ValueError("bucketing_weights needs one positive integer per bucket")
    if len(tars) != len(mans):
        raise ValueError(f"{len(mans)} manifest buckets but {len(tars)} tar buckets")
    if "labels" not in c and tokenizer is None:
        raise ValueError("a tarred character dataset needs 'labels' in its config")
    datasets = []
    for b, (t, m) in enumerate(zip(tars, mans)):
        t = t[0] if len(t) == 1 else t
        m = m[0] if len(m) == 1 else m
        kw = dict(sample_rate=c.get("sample_rate", 16000), shuffle_n=shuffle_n, min_duration=c.get("min_duration"), max_duration=c.get("max_duration"),
                  max_utts=c.get("max_utts", 0), shard_strategy=c.get("tarred_shard_strategy", "scatter"), shard_manifests=c.get("shard_manifests", False),
                  global_rank=global_rank, world_size=world_size, return_sample_id=c.get("return_sample_id", False), augmentor=augmentor)
        if tokenizer is None:
            ds = TarredAudioToCharDataset(t, m, labels=c["labels"], normalize=c.get("normalize_transcripts", False), unk_index=c.get("unk_index", -1), **kw)
        else:
            ds = TarredAudioToBPEDataset(t, m, tokenizer, use_start_end_token=c.get("use_start_end_token", True), **kw)
        datasets.extend([ds] * (weights[b] if weights else 1))
    return get_chain_dataset(datasets, c, rank=global_rank)


def get_concat_tarred_dataset(config, shuffle_n: int, global_rank: int, world_size: int, tokenizer=None, augmentor=None):
    c = _plain(config)
    parts = [get_tarred_dataset({**c, "manifest_filepath": m, "tarred_audio_filepaths": t}, shuffle_n, global_rank, world_size, tokenizer, augmentor)
             for t, m in zip(c["tarred_audio_filepaths"], c["manifest_filepath"])]
    return ConcatDataset(parts, shuffle=False, sampling_technique=c.get("concat_sampling_technique", "temperature"),
                         sampling_temperature=c.get("concat_sampling_temperature", 5), sampling_probabilities=c.get("concat_sampling_probabilities"),
                         sampling_scale=c.get("concat_sampling_scale", 1), seed=c.get("concat_sampling_seed") or 0, global_rank=global_rank, world_size=world_size)


def get_code_switched_dataset(config, shuffle_n: int, global_rank: int, world_size: int, tokenizer=None, augmentor=None):
    c = _plain(config)
    if "manifest_filepath" not in c or not isinstance(c["manifest_filepath"], (list, tuple)):
        raise ValueError("a code-switched dataset needs a list of manifests, one per language")
    cs = dict(c.get("code_switched") or {})
    if not cs:
        raise ValueError("a code-switched dataset needs the 'code_switched' section of the config")
    tarred = c.get("is_tarred", False)
    parts = []
    for k, m in enumerate(c["manifest_filepath"]):
        cc = {**c, "manifest_filepath": m}
        if tarred:
            cc["tarred_audio_filepaths"] = c["tarred_audio_filepaths"][k]
            parts.append(get_tarred_dataset(cc, shuffle_n, global_rank, world_size, tokenizer, augmentor))
        else:
            parts.append(get_char_dataset(cc, augmentor) if tokenizer is None else get_bpe_dataset(cc, tokenizer, augmentor))
    return CodeSwitchedDataset(parts, lang_probs=cs.get("probs"), shuffle=cs.get("shuffle", True), min_duration=cs.get("min_duration", 4),
                               max_duration=cs.get("max_duration", 20), min_monolingual=cs.get("min_monolingual", 0.3), db_norm=cs.get("db_norm", -25.0),
                               pause_start=cs.get("pause_start", 0), pause_join=cs.get("pause_join", 0), pause_end=cs.get("pause_end", 0),
                               seed=cs.get("seed") or 0, global_rank=global_rank, world_size=world_size,
                               sample_rate=c.get("sample_rate", 16000))


def _from_config(config, global_rank, world_size, tokenizer, augmentor):
    c = _plain(config)
    shuffle = c.get("shuffle", False)
    if c.get("is_code_switched", False):
        if c.get("manifest_filepath") is None or (c.get("is_tarred") and c.get("tarred_audio_filepaths") is None):
            return None
        return get_code_switched_dataset(c, c.get("shuffle_n", 4 * c.get("batch_size", 1)) if shuffle else 0, global_rank, world_size, tokenizer, augmentor)
    concat = c.get("is_concat", False)
    if concat and c.get("concat_sampling_technique") == "random" and not c.get("concat_sampling_probabilities"):
        raise ValueError("random concat sampling needs concat_sampling_probabilities")
    if c.get("is_tarred", False):
        if c.get("tarred_audio_filepaths") is None or c.get("manifest_filepath") is None:
            return None
        shuffle_n = c.get("shuffle_n", 4 * c.get("batch_size", 1)) if shuffle else 0
        fn = get_concat_tarred_dataset if concat else get_tarred_dataset
        return fn(c, shuffle_n, global_rank, world_size, tokenizer, augmentor)
    if c.get("manifest_filepath") is None:
        return None
    if concat:
        return (get_concat_char_dataset(c, global_rank, world_size, augmentor) if tokenizer is None
                else get_concat_bpe_dataset(c, tokenizer, global_rank, world_size, augmentor))
    return get_char_dataset(c, augmentor) if tokenizer is None else get_bpe_dataset(c, tokenizer, augmentor)


def get_audio_to_text_char_dataset_from_config(config, local_rank: int = 0, global_rank: int = 0, world_size: int = 1, preprocessor_cfg=None):
    """Dataset for a character model from its dataloader config: code-switched, concatenated, tarred (with buckets) or plain; ``None``
    when the config names no manifest.  ``augmentor`` in the config builds the waveform perturbation chain."""
    return _from_config(config, global_rank, world_size, None, _augmentor_of(config, global_rank, world_size))


def get_audio_to_text_bpe_dataset_from_config(config, local_rank: int = 0, global_rank: int = 0, world_size: int = 1, tokenizer=None, preprocessor_cfg=None):
    if tokenizer is None:
        raise ValueError("a BPE dataset needs a tokenizer")
    return _from_config(config, global_rank, world_size, tokenizer, _augmentor_of(config, global_rank, world_size))


def _augmentor_of(config, global_rank, world_size):
    c = _plain(config)
    if not c.get("augmentor"):
        return None
    from .perturb import process_augmentations

    return process_augmentations(c["augmentor"], global_rank=global_rank, world_size=world_size)


# label datasets --------------------------------------------------------------------------------------------------------
def get_classification_label_dataset(config):
    from .audio_to_label import AudioToClassificationLabelDataset

    c = _plain(config)
    return AudioToClassificationLabelDataset(c["manifest_filepath"], labels=c["labels"], sample_rate=c.get("sample_rate", 16000),
                                             min_duration=c.get("min_duration"), max_duration=c.get("max_duration"))


def get_tarred_classification_label_dataset(config, shuffle_n: int, global_rank: int, world_size: int, speech: bool = False):
    c = _plain(config)
    tars, mans = convert_to_config_list(c["tarred_audio_filepaths"]), convert_to_config_list(c["manifest_filepath"])
    cls = TarredAudioToSpeechLabelDataset if speech else TarredAudioToClassificationLabelDataset
    extra = dict(window_length_in_sec=c.get("window_length_in_sec"), shift_length_in_sec=c.get("shift_length_in_sec", 1.0)) if speech else {}
    ds = [cls(t[0] if len(t) == 1 else t, m[0] if len(m) == 1 else m, labels=c["labels"], sample_rate=c.get("sample_rate", 16000), shuffle_n=shuffle_n,
              min_duration=c.get("min_duration"), max_duration=c.get("max_duration"), shard_strategy=c.get("tarred_shard_strategy", "scatter"),
              global_rank=global_rank, world_size=world_size, **extra) for t, m in zip(tars, mans)]
    return get_chain_dataset(ds, c, rank=global_rank)


def get_tarred_speech_label_dataset(config, shuffle_n: int, global_rank: int, world_size: int):
    return get_tarred_classification_label_dataset(config, shuffle_n, global_rank, world_size, speech=True)


# ------------------------------------------------------------------------------------------------------ prediction writer
class ASRPredictionWriter:
    """Trainer callback for ``predict``: every rank appends the transcripts of its batches to ``<output_file stem>_<rank>.json`` style
    part files as JSON lines carrying the original manifest entry plus ``pred_text``; ``close_output_file`` closes the part and
    returns how many samples were written.  The dataset must return sample ids.
    Reference: ``asr/data/audio_to_text_dataset.py`` ``ASRPredictionWriter``."""

    def __init__(self, dataset, output_file: str):
        self.dataset, self.output_file = dataset, output_file
        self.fh = open(output_file, "w", encoding="utf-8")
        self.samples_num = 0

    def _item(self, sample_id: int) -> Dict[str, Any]:
        items = getattr(self.dataset, "items", None)
        if items is None and hasattr(self.dataset, "get_manifest_sample"):
            return dict(self.dataset.get_manifest_sample(sample_id))
        return dict(items[sample_id])

    def write_on_batch_end(self, trainer=None, pl_module=None, prediction=None, batch_indices=None, batch=None, batch_idx: int = 0, dataloader_idx: int = 0):
        for sample_id, hyp in prediction:
            it = self._item(int(sample_id))
            rec = {k: it[k] for k in ("audio_filepath", "offset", "duration", "text") if k in it}
            if hasattr(hyp, "text"):
                rec["pred_text"] = hyp.text
                if getattr(hyp, "timestamp", None):
                    rec["timestamp"] = hyp.timestamp
                if getattr(hyp, "token_confidence", None) is not None:
                    rec["token_confidence"] = [float(v) for v in hyp.token_confidence]
            else:
                rec["pred_text"] = str(hyp)
            self.fh.write(json.dumps(rec, ensure_ascii=False) + "\n")
            self.samples_num += 1

    on_predict_batch_end_write = write_on_batch_end

    def on_predict_batch_end(self, trainer, model, outputs, batch, batch_idx, dataloader_idx: int = 0):
        if outputs is not None:
            self.write_on_batch_end(trainer, model, outputs)

    def close_output_file(self) -> int:
        self.fh.close()
        return self.samples_num


# --------------------------------------------------------------------------------------------------- self-supervised items
@dataclass
class AudioNoiseItem:
    sample_id: Optional[str] = None
    audio: Optional[torch.Tensor] = None
    audio_len: Optional[torch.Tensor] = None
    noise: Optional[torch.Tensor] = None
    noise_len: Optional[torch.Tensor] = None
    noisy_audio: Optional[torch.Tensor] = None
    noisy_audio_len: Optional[torch.Tensor] = None


@dataclass
class AudioNoiseBatch:
    sample_id: Optional[list] = None
    audio: Optional[torch.Tensor] = None
    audio_len: Optional[torch.Tensor] = None
    noise: Optional[torch.Tensor] = None
    noise_len: Optional[torch.Tensor] = None
    noisy_audio: Optional[torch.Tensor] = None
    noisy_audio_len: Optional[torch.Tensor] = None


def _pad_to(x: torch.Tensor, n: int) -> torch.Tensor:
    return torch.nn.functional.pad(x, (0, n - len(x))) if len(x) < n else x[:n]


def audio_noise_collate(batch: List[AudioNoiseItem], batch_augmentor: Optional[Callable] = None) -> AudioNoiseBatch:
    """Pad clean audio, noise and their sum to the longest clean utterance of the batch; a batch augmentor (e.g. mixing utterances
    of the batch into each other) then rewrites the batch."""
    alen = torch.stack([b.audio_len for b in batch]).reshape(-1)
    n = int(alen.max())
    out = AudioNoiseBatch(sample_id=[b.sample_id for b in batch], audio=torch.stack([_pad_to(b.audio, n) for b in batch]), audio_len=alen,
                          noise=torch.stack([_pad_to(b.noise, n) for b in batch]), noise_len=torch.stack([b.noise_len for b in batch]).reshape(-1).clamp(max=n),
                          noisy_audio=torch.stack([_pad_to(b.noisy_audio, n) for b in batch]), noisy_audio_len=alen.clone())
    return batch_augmentor(out) if batch_augmentor is not None else out


def load_noise_manifest(noise_manifest) -> List[Dict[str, Any]]:
    """Entries of one or several noise manifests (comma-separated string or list); no manifest → no noise."""
    if noise_manifest is None:
        return []
    paths = noise_manifest.split(",") if isinstance(noise_manifest, str) else list(noise_manifest)
    out: List[Dict[str, Any]] = []
    for p in paths:
        out.extend(read_manifest(p.strip()))
    return out


def load_noise_audio(sample: Dict[str, Any], sample_rate: int, max_audio_len: Optional[int] = None, pad_to_max: bool = True,
                     min_white_noise_db: int = -90, max_white_noise_db: int = -46, max_trial: int = 100, rng: Optional[random.Random] = None):
    """A noise clip of at most ``max_audio_len`` samples from a random offset of the file; silent clips are retried, and if the file
    stays silent (or cannot be read) faint white noise stands in.  Returns ``(noise, length)``."""
    rng = rng or random
    dur = float(sample.get("duration") or 0.0)
    want = (max_audio_len or int(dur * sample_rate)) / sample_rate
    x = None
    for _ in range(max_trial):
        off = float(sample.get("offset", 0.0) or 0.0) + (rng.uniform(0.0, dur - want) if dur > want else 0.0)
        try:
            cand = np.asarray(load_audio(sample["audio_filepath"], sample_rate, off, want if dur > want else None), dtype=np.float32)
        except Exception:
            break
        if cand.size and float(np.abs(cand).sum()) > 0:
            x = cand
            break
    if x is None:
        n = max_audio_len or sample_rate
        level = 10.0 ** (rng.uniform(min_white_noise_db, max_white_noise_db) / 20.0)
        x = (np.random.RandomState(rng.randrange(1 << 30)).randn(n) * level).astype(np.float32)
    t = torch.from_numpy(x)
    n = len(t)
    if max_audio_len is not None:
        t = t[:max_audio_len]
        n = len(t)
        if pad_to_max and n < max_audio_len:
            t = torch.nn.functional.pad(t, (0, max_audio_len - n))
    return t, torch.tensor(n, dtype=torch.long)


def sample_noise(noise_data: List[Dict[str, Any]], sample_rate: int, max_audio_len: Optional[int] = None, max_trial: int = 20,
                 rng: Optional[random.Random] = None):
    """Noise from a random manifest entry; with no entries, zeros."""
    rng = rng or random
    if not noise_data:
        n = max_audio_len or sample_rate
        return torch.zeros(n), torch.tensor(n, dtype=torch.long)
    return load_noise_audio(rng.choice(noise_data), sample_rate, max_audio_len, max_trial=max_trial, rng=rng)


def pad_audio(audio: torch.Tensor, min_len: int, pad_audio_mode: str = "repeat") -> torch.Tensor:
    """Lengthen a short clip to ``min_len`` by repetition or by zeros."""
    if len(audio) >= min_len:
        return audio
    if pad_audio_mode == "repeat" and len(audio) > 0:
        return audio.repeat(-(-min_len // len(audio)))[:min_len]
    if pad_audio_mode in ("zero", "repeat"):
        return torch.nn.functional.pad(audio, (0, min_len - len(audio)))
    raise ValueError(f"pad_audio_mode must be 'repeat' or 'zero', got {pad_audio_mode!r}")


class _NoiseMixin:
    def _init_noise(self, noise_manifest, min_audio_len_secs: float, pad_audio_mode: str, batch_augmentor, seed: int = 0):
        self.noise_data = load_noise_manifest(noise_manifest)
        self.min_audio_len_secs, self.pad_audio_mode, self.batch_augmentor = min_audio_len_secs, pad_audio_mode, batch_augmentor
        self._rng = random.Random(seed)

    def _item(self, audio: torch.Tensor, sample_id) -> AudioNoiseItem:
        audio = pad_audio(audio, int(self.min_audio_len_secs * self.sample_rate), self.pad_audio_mode)
        noise, nlen = sample_noise(self.noise_data, self.sample_rate, len(audio), rng=self._rng)
        n = torch.tensor(len(audio), dtype=torch.long)
        return AudioNoiseItem(sample_id=str(sample_id), audio=audio, audio_len=n, noise=noise, noise_len=nlen, noisy_audio=audio + noise, noisy_audio_len=n)

    def _collate_fn(self, batch):
        return audio_noise_collate(batch, self.batch_augmentor)

    collate_fn = _collate_fn


class AudioNoiseDataset(_NoiseMixin, AudioToCharDataset):
    """Clean audio, a noise clip of the same length and their sum for denoising self-supervision; transcripts are ignored."""

    def __init__(self, noise_manifest=None, batch_augmentor=None, min_audio_len_secs: float = 1.0, pad_audio_mode: str = "repeat", seed: int = 0, **kw):
        kw.setdefault("labels", [])
        AudioToCharDataset.__init__(self, **kw)
        self._init_noise(noise_manifest, min_audio_len_secs, pad_audio_mode, batch_augmentor, seed)

    def __getitem__(self, idx):
        it = self.items[idx]
        x = load_audio(it["audio_filepath"], self.sample_rate, it.get("offset", 0.0) or 0.0, it.get("duration"), self.channel_selector)
        if self.augmentor is not None:
            x = self.augmentor(x, self.sample_rate)
        return self._item(torch.from_numpy(np.ascontiguousarray(x)), idx)


class TarredAudioNoiseDataset(_NoiseMixin, TarredAudioToCharDataset):
    def __init__(self, noise_manifest=None, batch_augmentor=None, min_audio_len_secs: float = 1.0, pad_audio_mode: str = "repeat", seed: int = 0, **kw):
        kw.setdefault("labels", [])
        TarredAudioToCharDataset.__init__(self, **kw)
        self._init_noise(noise_manifest, min_audio_len_secs, pad_audio_mode, batch_augmentor, seed)

    def _build(self, it, x, k):
        if self.augmentor is not None:
            x = self.augmentor(x, self.sample_rate)
        return self._item(torch.from_numpy(np.ascontiguousarray(x)), k)


class CutAudioNoiseDataset(Dataset):
    """The same item over mini-batches of cuts (the sampler hands a list of cuts per index)."""

    def __init__(self, noise_manifest=None, batch_augmentor_cfg=None, sample_rate: int = 16000, min_audio_len_secs: float = 1.0, pad_audio_mode: str = "repeat", seed: int = 0):
        self.sample_rate = sample_rate
        self._m = _NoiseMixin()
        self._m.sample_rate = sample_rate
        self._m._init_noise(noise_manifest, min_audio_len_secs, pad_audio_mode, batch_augmentor_cfg, seed)

    def __getitem__(self, cuts) -> AudioNoiseBatch:
        items = [self._m._item(torch.as_tensor(np.asarray(c.load_audio(self.sample_rate) if hasattr(c, "load_audio") else c, dtype=np.float32)), getattr(c, "id", k))
                 for k, c in enumerate(cuts)]
        return audio_noise_collate(items, self._m.batch_augmentor)


def get_audio_noise_dataset_from_config(config, global_rank: int = 0, world_size: int = 1):
    c = _plain(config)
    aug = _augmentor_of(c, global_rank, world_size)
    batch_aug = c.get("batch_augmentor")
    if isinstance(batch_aug, dict):
        from ..core.instantiate import instantiate

        batch_aug = instantiate(batch_aug)
    noise_kw = dict(noise_manifest=c.get("noise_manifest"), batch_augmentor=batch_aug, min_audio_len_secs=c.get("min_audio_len_secs", 1.0),
                    pad_audio_mode=c.get("pad_audio_mode", "repeat"))
    base = dict(sample_rate=c.get("sample_rate", 16000), min_duration=c.get("min_duration"), max_duration=c.get("max_duration"), max_utts=c.get("max_utts", 0),
                augmentor=aug)
    if c.get("is_tarred", False):
        if c.get("tarred_audio_filepaths") is None or c.get("manifest_filepath") is None:
            return None
        shuffle_n = c.get("shuffle_n", 4 * c.get("batch_size", 1)) if c.get("shuffle", False) else 0
        tars, mans = convert_to_config_list(c["tarred_audio_filepaths"]), convert_to_config_list(c["manifest_filepath"])
        ds = [TarredAudioNoiseDataset(audio_tar_filepaths=t[0] if len(t) == 1 else t, manifest_filepath=m[0] if len(m) == 1 else m, shuffle_n=shuffle_n,
                                      shard_strategy=c.get("tarred_shard_strategy", "scatter"), global_rank=global_rank, world_size=world_size, **noise_kw, **base)
              for t, m in zip(tars, mans)]
        return get_chain_dataset(ds, c, rank=global_rank)
    if c.get("manifest_filepath") is None:
        return None
    if c.get("is_concat", False):
        parts = [AudioNoiseDataset(manifest_filepath=m, **noise_kw, **base) for m in c["manifest_filepath"]]
        return ConcatDataset(parts, shuffle=c.get("concat_shuffle", True), sampling_technique=c.get("concat_sampling_technique", "temperature"),
                             sampling_temperature=c.get("concat_sampling_temperature", 5), sampling_probabilities=c.get("concat_sampling_probabilities"),
                             seed=c.get("concat_sampling_seed") or 0, global_rank=global_rank, world_size=world_size)
    return AudioNoiseDataset(manifest_filepath=c["manifest_filepath"], **noise_kw, **base)


# ------------------------------------------------------------------------------------------------------- feature manifests
def _load_feat(path: str) -> torch.Tensor:
    if path.endswith(".npy"):
        return torch.from_numpy(np.load(path)).float()
    return torch.load(path, map_location="cpu").float()


def _rttm_speech_mask(rttm_path: str, n_frames: int, frame_unit_time_secs: float, offset: float = 0.0) -> torch.Tensor:
    mask = torch.zeros(n_frames, dtype=torch.bool)
    with open(rttm_path) as f:
        for line in f:
            p = line.split()
            if len(p) >= 5 and p[0] == "SPEAKER":
                s, d = float(p[3]) - offset, float(p[4])
                a, b = max(0, int(round(s / frame_unit_time_secs))), min(n_frames, int(round((s + d) / frame_unit_time_secs)))
                if b > a:
                    mask[a:b] = True
    return mask


class _FeatureText(Dataset):
    """Pre-computed features ``[D, T]`` (``feature_file``: .npy / .pt) with transcripts.  With ``rttm_filepath`` entries, frames outside
    the RTTM's speech segments are either set to ``zero_spec_db_val`` (``rttm_mode='mask'``) or removed (``'drop'``), which is how
    VAD output gates the ASR input."""

    def __init__(self, manifest_filepath, normalize: bool = False, normalize_type: Union[str, dict] = "per_feature", use_rttm: bool = False,
                 rttm_mode: str = "mask", feat_min_len: int = 4, feat_mask_val: Optional[float] = None, frame_unit_time_secs: float = 0.01,
                 min_duration=None, max_duration=None, max_utts: int = 0, return_sample_id: bool = False, augmentor=None, pad_id: int = 0, **_):
        if rttm_mode not in ("mask", "drop"):
            raise ValueError(f"rttm_mode must be 'mask' or 'drop', got {rttm_mode!r}")
        self.items = read_manifest(manifest_filepath, min_duration, max_duration, max_utts)
        self.normalize, self.normalize_type, self.use_rttm, self.rttm_mode = normalize, normalize_type, use_rttm, rttm_mode
        self.feat_min_len, self.frame_unit_time_secs, self.return_sample_id = feat_min_len, frame_unit_time_secs, return_sample_id
        self.feat_mask_val = -16.635 if feat_mask_val is None else feat_mask_val      # log of the mel floor 2^-24
        self.augmentor, self.pad_id = augmentor, pad_id

    def __len__(self):
        return len(self.items)

    def tokenize(self, it):
        raise NotImplementedError

    def _normalize(self, f: torch.Tensor) -> torch.Tensor:
        if isinstance(self.normalize_type, dict):
            return (f - torch.as_tensor(self.normalize_type["fixed_mean"]).reshape(-1, 1)) / torch.as_tensor(self.normalize_type["fixed_std"]).reshape(-1, 1)
        if self.normalize_type == "per_feature":
            return (f - f.mean(1, keepdim=True)) / (f.std(1, keepdim=True) + 1e-5)
        if self.normalize_type == "all_features":
            return (f - f.mean()) / (f.std() + 1e-5)
        raise ValueError(f"unknown normalize_type {self.normalize_type!r}")

    def __getitem__(self, idx):
        it = self.items[idx]
        f = _load_feat(it.get("feature_file") or it["feature_filepath"])
        if self.use_rttm and it.get("rttm_filepath", it.get("rttm_file")):
            m = _rttm_speech_mask(it.get("rttm_filepath", it.get("rttm_file")), f.shape[1], self.frame_unit_time_secs, float(it.get("offset", 0.0) or 0.0))
            if self.rttm_mode == "mask":
                f = torch.where(m[None, :], f, torch.full_like(f, self.feat_mask_val))
            else:
                f = f[:, m]
                if f.shape[1] < self.feat_min_len:
                    f = torch.nn.functional.pad(f, (0, self.feat_min_len - f.shape[1]), value=self.feat_mask_val)
        if self.augmentor is not None:
            f = self.augmentor(f)
        if self.normalize:
            f = self._normalize(f)
        toks = self.tokenize(it)
        out = (f, f.shape[1], torch.tensor(toks, dtype=torch.long), len(toks))
        return out + (idx,) if self.return_sample_id else out

    def collate_fn(self, batch):
        T, U = max(b[1] for b in batch), max(max(b[3] for b in batch), 1)
        F = torch.full((len(batch), batch[0][0].shape[0], T), self.feat_mask_val if self.use_rttm else 0.0)
        Y = torch.full((len(batch), U), self.pad_id, dtype=torch.long)
        for k, b in enumerate(batch):
            F[k, :, :b[1]] = b[0]
            Y[k, :b[3]] = b[2]
        out = (F, torch.tensor([b[1] for b in batch]), Y, torch.tensor([b[3] for b in batch]))
        return out + (torch.tensor([b[4] for b in batch]),) if self.return_sample_id else out

    _collate_fn = collate_fn


class FeatureToCharDataset(_FeatureText):
    def __init__(self, manifest_filepath, labels: Sequence[str], normalize_transcripts: bool = False, unk_index: int = -1, **kw):
        super().__init__(manifest_filepath, **kw)
        self._map, self.labels, self.norm_text, self.unk_index = {c: i for i, c in enumerate(labels)}, list(labels), normalize_transcripts, unk_index

    def tokenize(self, it):
        text = it["text"].lower() if self.norm_text else it["text"]
        return [self._map.get(c, self.unk_index) for c in text if c in self._map or self.unk_index >= 0]


class FeatureToBPEDataset(_FeatureText):
    def __init__(self, manifest_filepath, tokenizer, use_start_end_token: bool = False, **kw):
        super().__init__(manifest_filepath, **kw)
        self.tokenizer, self.use_start_end_token = tokenizer, use_start_end_token

    def tokenize(self, it):
        return AudioToBPEDataset.tokenize(self, it)


def get_feature_char_dataset(config, augmentor=None) -> FeatureToCharDataset:
    c = _plain(config)
    return FeatureToCharDataset(c["manifest_filepath"], labels=c["labels"], normalize_transcripts=c.get("normalize_transcripts", False),
                                **{k: c[k] for k in ("normalize", "normalize_type", "use_rttm", "rttm_mode", "feat_min_len", "feat_mask_val", "frame_unit_time_secs",
                                                     "min_duration", "max_duration", "max_utts", "return_sample_id") if k in c}, augmentor=augmentor)


def get_feature_bpe_dataset(config, tokenizer, augmentor=None) -> FeatureToBPEDataset:
    c = _plain(config)
    return FeatureToBPEDataset(c["manifest_filepath"], tokenizer, use_start_end_token=c.get("use_start_end_token", True),
                               **{k: c[k] for k in ("normalize", "normalize_type", "use_rttm", "rttm_mode", "feat_min_len", "feat_mask_val", "frame_unit_time_secs",
                                                    "min_duration", "max_duration", "max_utts", "return_sample_id") if k in c}, augmentor=augmentor)


# -------------------------------------------------------------------------------------------------- record (HF-style) data
def get_nested_dict_value(d: dict, key: str):
    """``'audio.array'`` → ``d['audio']['array']``."""
    for k in key.split("."):
        d = d[k]
    return d


class HFTextProcessor:
    """Text clean-up of record datasets: optional lower-casing and symbol removal / replacement before tokenising."""

    def __init__(self, parser: Callable[[str], List[int]], bos_id=None, eos_id=None, pad_id: int = 0, normalize_text: bool = False,
                 symbols_to_keep: Optional[Union[str, Sequence[str]]] = None):
        self.parser, self.bos_id, self.eos_id, self.pad_id, self.normalize_text = parser, bos_id, eos_id, pad_id, normalize_text
        self.symbols_to_keep = list(symbols_to_keep) if symbols_to_keep else []

    def process_text(self, text: str, lang: Optional[str] = None) -> List[int]:
        if self.normalize_text:
            keep = set(self.symbols_to_keep)
            text = "".join(ch if (ch.isalnum() or ch.isspace() or ch in keep or ch == "'") else " " for ch in text.lower())
            text = " ".join(text.split())
        ids = list(self.parser(text, lang) if lang is not None else self.parser(text))
        if self.bos_id is not None:
            ids = [self.bos_id] + ids
        if self.eos_id is not None:
            ids = ids + [self.eos_id]
        return ids


def _load_hf(path, data_kwargs):
    try:
        import datasets as hf_datasets
    except ImportError as e:
        raise ImportError("loading a dataset by name needs the 'datasets' package; pass the records themselves instead") from e
    return hf_datasets.load_dataset(path, **dict(data_kwargs or {}))


def _resample(x: np.ndarray, sr: int, target: int) -> np.ndarray:
    if sr == target:
        return x
    from scipy.signal import resample_poly
    from math import gcd

    g = gcd(int(sr), int(target))
    return resample_poly(x, target // g, sr // g).astype(np.float32)


class _RecordAudioText:
    def _setup(self, audio_key, text_key, sample_rate_key, sample_rate, processor, channel_selector, id_key, augmentor, return_sample_id):
        self.audio_key, self.text_key, self.sample_rate_key, self.sample_rate = audio_key, text_key, sample_rate_key, sample_rate
        self.processor, self.channel_selector, self.id_key, self.augmentor, self.return_sample_id = processor, channel_selector, id_key, augmentor, return_sample_id

    def _build(self, rec, idx):
        x = np.asarray(get_nested_dict_value(rec, self.audio_key), dtype=np.float32)
        if x.ndim == 2:
            sel = self.channel_selector
            x = x.mean(0) if sel in (None, "average") else x[int(sel)]
        x = _resample(x, int(get_nested_dict_value(rec, self.sample_rate_key)), self.sample_rate)
        if self.augmentor is not None:
            x = self.augmentor(x, self.sample_rate)
        ids = self.processor.process_text(get_nested_dict_value(rec, self.text_key))
        out = (torch.from_numpy(np.ascontiguousarray(x)), len(x), torch.tensor(ids, dtype=torch.long), len(ids))
        if self.return_sample_id:
            out = out + (get_nested_dict_value(rec, self.id_key) if self.id_key else idx,)
        return out

    def collate_fn(self, batch):
        return speech_collate(batch, self.processor.pad_id)

    _collate_fn = collate_fn


class HFAudioToCharDataset(_RecordAudioText, Dataset):
    """Map-style dataset over records (a list of dicts, a Hugging Face dataset object, or the name of one to load) with nested
    keys for audio samples, sample rate and text."""

    def __init__(self, labels: Sequence[str], audio_key: str = "audio.array", text_key: str = "text", sample_rate_key: str = "audio.sampling_rate",
                 sample_rate: int = 16000, hf_data_cfg=None, records=None, normalize_text: bool = False, symbols_to_keep=None, channel_selector=None,
                 id_key: Optional[str] = None, augmentor=None, return_sample_id: bool = False, unk_index: int = -1, bos_id=None, eos_id=None, pad_id: int = 0, **_):
        m = {c: i for i, c in enumerate(labels)}
        parser = lambda t: [m.get(c, unk_index) for c in t if c in m or unk_index >= 0]  # noqa: E731
        self._setup(audio_key, text_key, sample_rate_key, sample_rate, HFTextProcessor(parser, bos_id, eos_id, pad_id, normalize_text, symbols_to_keep),
                    channel_selector, id_key, augmentor, return_sample_id)
        self.records = records if records is not None else _load_hf(**_plain(hf_data_cfg))

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self._build(self.records[i], i)


class HFAudioToBPEDataset(HFAudioToCharDataset):
    def __init__(self, tokenizer, use_start_end_token: bool = False, **kw):
        kw.pop("labels", None)
        bos = getattr(tokenizer, "bos_id", None) if use_start_end_token else None
        eos = getattr(tokenizer, "eos_id", None) if use_start_end_token else None
        super().__init__(labels=[], **kw)
        self.tokenizer = tokenizer
        self.processor = HFTextProcessor(tokenizer.text_to_ids, bos if bos is not None and bos >= 0 else None, eos if eos is not None and eos >= 0 else None,
                                         kw.get("pad_id", 0), kw.get("normalize_text", False), kw.get("symbols_to_keep"))


class HFIterableAudioToCharDataset(_RecordAudioText, IterableDataset):
    """Streaming variant: records come from an iterable, are split over ranks and loader workers by index, and pass through a shuffle
    buffer of ``shuffle_n`` records."""

    def __init__(self, labels: Sequence[str], records: Iterable = None, hf_data_cfg=None, shuffle_n: int = 0, shuffle_seed: int = 0, global_rank: int = 0,
                 world_size: int = 1, **kw):
        helper = HFAudioToCharDataset(labels=labels, records=records if records is not None else _load_hf(**_plain(hf_data_cfg)), **kw)
        self.__dict__.update(helper.__dict__)
        self.shuffle_n, self.shuffle_seed, self.global_rank, self.world_size = shuffle_n, shuffle_seed, global_rank, world_size

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        nw, wid = (info.num_workers, info.id) if info is not None else (1, 0)
        stride, mine = self.world_size * nw, self.global_rank * nw + wid
        rng, buf = random.Random(self.shuffle_seed + mine), []
        for i, rec in enumerate(self.records):
            if i % stride != mine:
                continue
            s = self._build(rec, i)
            if self.shuffle_n > 1:
                if len(buf) < self.shuffle_n:
                    buf.append(s)
                    continue
                j = rng.randrange(len(buf))
                buf[j], s = s, buf[j]
            yield s
        rng.shuffle(buf)
        yield from buf


class HFIterableAudioToBPEDataset(HFIterableAudioToCharDataset):
    def __init__(self, tokenizer, use_start_end_token: bool = False, **kw):
        kw.pop("labels", None)
        super().__init__(labels=[], **kw)
        bos = getattr(tokenizer, "bos_id", None) if use_start_end_token else None
        eos = getattr(tokenizer, "eos_id", None) if use_start_end_token else None
        self.tokenizer = tokenizer
        self.processor = HFTextProcessor(tokenizer.text_to_ids, bos if bos is not None and bos >= 0 else None, eos if eos is not None and eos >= 0 else None,
                                         kw.get("pad_id", 0), kw.get("normalize_text", False), kw.get("symbols_to_keep"))


def get_hf_audio_to_text_char_dataset(config, global_rank: int = 0, world_size: int = 1, records=None):
    c = _plain(config)
    keys = {k: c[k] for k in ("audio_key", "text_key", "sample_rate_key", "sample_rate", "normalize_text", "symbols_to_keep", "channel_selector", "id_key",
                              "return_sample_id", "unk_index") if k in c}
    if c.get("streaming", False):
        return HFIterableAudioToCharDataset(labels=c["labels"], records=records, hf_data_cfg=c.get("hf_data_cfg"), shuffle_n=c.get("shuffle_n", 0),
                                            shuffle_seed=c.get("shuffle_seed", 0), global_rank=global_rank, world_size=world_size, **keys)
    return HFAudioToCharDataset(labels=c["labels"], records=records, hf_data_cfg=c.get("hf_data_cfg"), **keys)


def get_hf_audio_to_text_bpe_dataset(config, tokenizer, global_rank: int = 0, world_size: int = 1, records=None):
    c = _plain(config)
    keys = {k: c[k] for k in ("audio_key", "text_key", "sample_rate_key", "sample_rate", "normalize_text", "symbols_to_keep", "channel_selector", "id_key",
                              "return_sample_id") if k in c}
    if c.get("streaming", False):
        return HFIterableAudioToBPEDataset(tokenizer, use_start_end_token=c.get("use_start_end_token", False), records=records, hf_data_cfg=c.get("hf_data_cfg"),
                                           shuffle_n=c.get("shuffle_n", 0), shuffle_seed=c.get("shuffle_seed", 0), global_rank=global_rank, world_size=world_size, **keys)
    return HFAudioToBPEDataset(tokenizer, use_start_end_token=c.get("use_start_end_token", False), records=records, hf_data_cfg=c.get("hf_data_cfg"), **keys)

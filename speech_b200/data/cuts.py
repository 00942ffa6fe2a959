"""Cut-based data pipeline configured with the reference's Lhotse dataloader schema.

``get_dataloader_from_cuts_config(config, ...)`` understands the keys of ``LhotseDataLoadingConfig``
(``common/data/lhotse/dataloader.py:71-256``): inputs (``manifest_filepath``, ``tarred_audio_filepaths``, ``cuts_path``,
``shar_path``, ``input_cfg`` trees with ``type`` / ``weight`` / ``tags`` and nested ``group``; the source types are listed
in :mod:`speech_b200.data.sources`), sampling (``batch_size``,
``batch_duration``, ``quadratic_duration``, ``num_buckets``, ``bucket_duration_bins`` 1-D or 2-D,
``bucket_batch_size``, ``batch_tokens`` + ``token_equivalent_duration``, ``max_open_streams`` ignored), filters
(``min_duration`` / ``max_duration``, ``min_tps`` / ``max_tps``, ``min_tokens`` / ``max_tokens``, ``min_tpt`` / ``max_tpt``,
``max_cer``, ``keep_validation_status``, ``min_context_speaker_similarity``), multimodal sampling
(``use_multimodal_sampling`` + ``batch_tokens`` + ``quadratic_factor`` + ``measure_total_length``), ordering
(``shuffle``, ``seed``, ``shard_seed`` "trng" / "randomized" / int), augmentation (``noise_path`` + ``noise_snr`` +
``noise_mix_prob``, ``perturb_speed``, ``rir_enabled`` + ``rir_path`` + ``rir_prob``, ``truncate_duration``,
``cut_into_windows_duration``), and ``multi_config`` (several sub-configs fused round-robin / zipped / by weight).

A *cut* is a lightweight record (audio source, offset, duration, supervision text / language / custom fields); cut sets
are lazy and composable (filter, map, mux).  Sampling reuses ``DynamicBucketingSampler``; 2-D buckets add the number of
tokens as the second bucketing dimension (``sampling.py`` ``FixedBucketBatchSizeConstraint2D``).
"""
from __future__ import annotations

import bisect
import io
import json
import os
import tarfile
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
from torch.utils.data import Dataset

from ..core.config import DictConfig, to_container
from .audio_to_text import BatchedLoader, DynamicBucketingSampler, expand_sharded_filepaths, load_audio, speech_collate


@dataclass
class Cut:
    id: str
    audio: Any                         # path, (tar_path, member_name) or an in-memory float array
    duration: float
    offset: float = 0.0
    text: str = ""
    lang: Optional[str] = None
    sampling_rate: int = 16000
    custom: Dict[str, Any] = field(default_factory=dict)
    speed: float = 1.0                 # speed-perturbation factor applied at load time

    def load_audio(self, target_sr: int = 16000) -> np.ndarray:
        if isinstance(self.audio, (np.ndarray, torch.Tensor)):
            x = np.asarray(self.audio, dtype=np.float32)
        elif isinstance(self.audio, tuple):
            tar_path, member = self.audio
            with tarfile.open(tar_path) as tf:
                data = tf.extractfile(member).read()
            x = np.asarray(load_audio(io.BytesIO(data), target_sr=target_sr), dtype=np.float32)
        else:
            x = np.asarray(load_audio(self.audio, target_sr=target_sr, offset=self.offset,
                                      duration=self.duration * self.speed if self.duration else None), dtype=np.float32)
        if self.speed != 1.0:
            x = speed_perturb(x, self.speed)
        return x

    def with_speed(self, factor: float) -> "Cut":
        return Cut(f"{self.id}_sp{factor}", self.audio, self.duration / factor, self.offset, self.text, self.lang,
                   self.sampling_rate, dict(self.custom), self.speed * factor)


def speed_perturb(x: np.ndarray, factor: float) -> np.ndarray:
    """Resample by linear interpolation so that the signal plays ``factor`` times faster (pitch shifts with it)."""
    n = max(1, int(round(len(x) / factor)))
    pos = np.linspace(0, len(x) - 1, n)
    return np.interp(pos, np.arange(len(x)), x).astype(np.float32)


class CutSet:
    def __init__(self, source: Union[Sequence[Cut], Callable[[], Iterator[Cut]]]):
        self._source = source

    def __iter__(self) -> Iterator[Cut]:
        return iter(self._source() if callable(self._source) else self._source)

    def to_eager(self) -> "CutSet":
        return CutSet(list(self))

    def __len__(self):
        if callable(self._source):
            self._source = list(self._source())
        return len(self._source)

    def filter(self, pred: Callable[[Cut], bool]) -> "CutSet":
        return CutSet(lambda: (c for c in self if pred(c)))

    def map(self, fn: Callable[[Cut], Cut]) -> "CutSet":
        return CutSet(lambda: (fn(c) for c in self))

    def cut_into_windows(self, duration: float) -> "CutSet":
        def gen():
            for c in self:
                n = max(1, int(np.ceil(c.duration / duration)))
                for k in range(n):
                    d = min(duration, c.duration - k * duration)
                    if d > 0:
                        yield Cut(f"{c.id}-{k}", c.audio, d, c.offset + k * duration, c.text if n == 1 else "", c.lang,
                                  c.sampling_rate, dict(c.custom))
        return CutSet(gen)

    def truncate(self, max_duration: float, rng: Optional[np.random.Generator] = None) -> "CutSet":
        def fn(c: Cut) -> Cut:
            if c.duration <= max_duration:
                return c
            off = float(rng.uniform(0, c.duration - max_duration)) if rng is not None else 0.0
            return Cut(c.id, c.audio, max_duration, c.offset + off, c.text, c.lang, c.sampling_rate, dict(c.custom))
        return self.map(fn)

    @staticmethod
    def mux(sets: Sequence["CutSet"], weights: Optional[Sequence[float]] = None, seed: int = 0, stop_early: bool = False) -> "CutSet":
        """Randomly interleave several cut sets, drawing from set ``i`` with probability ``weights[i]``."""
        def gen():
            rng = np.random.default_rng(seed)
            its = [iter(s) for s in sets]
            w = np.asarray(weights if weights is not None else [1.0] * len(sets), dtype=np.float64)
            alive = [True] * len(sets)
            while any(alive):
                p = w * np.asarray(alive)
                p = p / p.sum()
                i = int(rng.choice(len(sets), p=p))
                try:
                    yield next(its[i])
                except StopIteration:
                    alive[i] = False
                    if stop_early:
                        return
        return CutSet(gen)


# ---------------------------------------------------------------------------------------------- readers
def read_nemo_manifest(paths, lang_field: str = "lang", text_field: str = "text", tags: Optional[Dict[str, Any]] = None) -> CutSet:
    def gen():
        for p in expand_sharded_filepaths(paths):
            base = os.path.dirname(os.path.abspath(p))
            with open(p, encoding="utf-8") as f:
                for k, line in enumerate(f):
                    line = line.strip()
                    if not line:
                        continue
                    it = json.loads(line)
                    ap = it.get("audio_filepath", it.get("audio_file"))
                    if ap and not os.path.isabs(ap) and not os.path.exists(ap):
                        ap = os.path.join(base, ap)
                    custom = {k2: v for k2, v in it.items() if k2 not in ("audio_filepath", "duration", "offset", text_field, lang_field)}
                    custom.update(tags or {})
                    yield Cut(it.get("id", f"{os.path.basename(p)}-{k}"), ap, float(it.get("duration", 0.0) or 0.0),
                              float(it.get("offset", 0.0) or 0.0), it.get(text_field, ""), it.get(lang_field), custom=custom)
    return CutSet(gen)


def read_nemo_tarred(manifest_paths, tar_paths, tags: Optional[Dict[str, Any]] = None, shard_rank: int = 0, shard_world: int = 1) -> CutSet:
    """Tarred audio: manifest ``audio_filepath`` entries name members of the tar shards; shards are split over ranks."""
    def gen():
        tars = expand_sharded_filepaths(tar_paths)[shard_rank::shard_world]
        mans = expand_sharded_filepaths(manifest_paths)
        mans = mans[shard_rank::shard_world] if len(mans) > 1 else mans
        index: Dict[str, Dict[str, Any]] = {}
        for m in mans:
            with open(m, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        it = json.loads(line)
                        index[os.path.basename(it["audio_filepath"])] = it
        for t in tars:
            with tarfile.open(t) as tf:
                for member in tf:
                    it = index.get(os.path.basename(member.name))
                    if it is None or not member.isfile():
                        continue
                    data = tf.extractfile(member).read()
                    x = np.asarray(load_audio(io.BytesIO(data)), dtype=np.float32)
                    custom = dict(tags or {})
                    yield Cut(it.get("id", member.name), x, float(it.get("duration", len(x) / 16000.0)), 0.0, it.get("text", ""),
                              it.get("lang"), custom=custom)
    return CutSet(gen)


def read_txt(paths, language: Optional[str] = None, tags: Optional[Dict[str, Any]] = None) -> CutSet:
    from .sources import get_parser

    return get_parser("txt")({"paths": paths, "language": language, "tags": tags}, {})


def parse_input_cfg(input_cfg, seed: int = 0, rank: int = 0, world: int = 1) -> CutSet:
    """``input_cfg``: list of ``{type, weight, tags, ...}`` entries (or the path of a YAML file holding one); ``type: group``
    nests another ``input_cfg``.  Each type is read by the parser registered for it in :mod:`speech_b200.data.sources`;
    entries are interleaved at random in proportion to their ``weight``."""
    from .sources import get_parser

    if isinstance(input_cfg, str):
        import yaml

        with open(input_cfg) as f:
            input_cfg = yaml.safe_load(f)
    sets, weights = [], []
    for i, e in enumerate(input_cfg):
        e = dict(e)
        t = e.get("type", "nemo")
        if t == "group":
            cs = parse_input_cfg(e["input_cfg"], seed + i + 1, rank, world)
            if e.get("tags"):
                tags = dict(e["tags"])
                cs = cs.map(lambda c, tags=tags: _with_tags(c, tags))
        else:
            cs = get_parser(t)(e, {"seed": seed + i, "rank": rank, "world": world})
        sets.append(cs)
        weights.append(float(e.get("weight", 1.0)))
    if len(sets) == 1:
        return sets[0]
    return CutSet.mux(sets, weights, seed=seed)


def _with_tags(c: Cut, tags: Dict[str, Any]) -> Cut:
    for k, v in tags.items():
        c.custom.setdefault(k, v)
    return c


def reweight_by_temperature(weights: Sequence[float], temperature: float) -> List[float]:
    w = np.asarray(weights, dtype=np.float64) ** temperature
    return (w / w.sum()).tolist()


# ---------------------------------------------------------------------------------------------- augmentation
class NoiseMixer:
    def __init__(self, noise_cuts: Sequence[Cut], snr=(10.0, 20.0), prob: float = 0.5, seed: int = 0, sr: int = 16000):
        self.noise, self.snr, self.prob, self.sr = list(noise_cuts), snr, prob, sr
        self.rng = np.random.default_rng(seed)

    def __call__(self, x: np.ndarray) -> np.ndarray:
        if not self.noise or self.rng.random() > self.prob:
            return x
        n = self.noise[int(self.rng.integers(len(self.noise)))].load_audio(self.sr)
        if len(n) < len(x):
            n = np.tile(n, int(np.ceil(len(x) / max(1, len(n)))))
        s = int(self.rng.integers(0, len(n) - len(x) + 1))
        n = n[s:s + len(x)]
        snr = float(self.rng.uniform(*self.snr)) if isinstance(self.snr, (list, tuple)) else float(self.snr)
        g = np.sqrt((x ** 2).mean() / max((n ** 2).mean(), 1e-10)) * 10 ** (-snr / 20.0)
        return (x + g * n).astype(np.float32)


class RIRConvolver:
    def __init__(self, rir_cuts: Optional[Sequence[Cut]] = None, prob: float = 0.5, seed: int = 0, sr: int = 16000):
        self.rirs, self.prob, self.sr = list(rir_cuts or []), prob, sr
        self.rng = np.random.default_rng(seed)

    def _synthetic(self) -> np.ndarray:
        t60 = self.rng.uniform(0.1, 0.5)
        n = int(t60 * self.sr)
        h = self.rng.standard_normal(n) * np.exp(-6.9 * np.arange(n) / n)
        h[0] = 1.0
        return (h / np.abs(h).max()).astype(np.float32)

    def __call__(self, x: np.ndarray) -> np.ndarray:
        if self.rng.random() > self.prob:
            return x
        h = self.rirs[int(self.rng.integers(len(self.rirs)))].load_audio(self.sr) if self.rirs else self._synthetic()
        n = len(x) + len(h) - 1
        y = np.fft.irfft(np.fft.rfft(x, n) * np.fft.rfft(h, n), n)[: len(x)]
        return (y * (np.abs(x).max() / max(np.abs(y).max(), 1e-8))).astype(np.float32)


# ---------------------------------------------------------------------------------------------- dataset + loader
class CutsSpeechToTextDataset(Dataset):
    """Map-style dataset over an eager cut list → ``(audio, audio_len, tokens, token_len)`` (reference
    ``asr/data/audio_to_text_lhotse.py:28-89``).  ``tokenizer`` may be an aggregate tokenizer (language from ``cut.lang``)."""

    def __init__(self, cuts: Sequence[Cut], tokenizer=None, labels: Optional[Sequence[str]] = None, sample_rate: int = 16000,
                 augmentations: Sequence[Callable[[np.ndarray], np.ndarray]] = (), return_cuts: bool = False, pad_id: int = 0):
        self.cuts, self.tok, self.sr, self.aug, self.return_cuts, self.pad_id = list(cuts), tokenizer, sample_rate, list(augmentations), return_cuts, pad_id
        self.label2id = {l: i for i, l in enumerate(labels)} if labels is not None else None

    def durations(self) -> List[float]:
        return [c.duration for c in self.cuts]

    def num_tokens(self, idx: int) -> int:
        return len(self.tokenize(self.cuts[idx]))

    def tokenize(self, c: Cut) -> List[int]:
        if self.tok is not None:
            try:
                return list(self.tok.text_to_ids(c.text, c.lang)) if c.lang is not None and hasattr(self.tok, "langs") \
                    else list(self.tok.text_to_ids(c.text))
            except TypeError:
                return list(self.tok.text_to_ids(c.text))
        return [self.label2id[ch] for ch in c.text if ch in self.label2id]

    def __len__(self):
        return len(self.cuts)

    def __getitem__(self, idx):
        c = self.cuts[idx]
        x = c.load_audio(self.sr)
        for a in self.aug:
            x = a(x)
        t = self.tokenize(c)
        return torch.as_tensor(x), torch.tensor(len(x)), torch.tensor(t, dtype=torch.long), torch.tensor(len(t))

    def collate_fn(self, batch):
        return speech_collate(batch, pad_id=self.pad_id)


class TwoDimBucketingSampler(DynamicBucketingSampler):
    """``bucket_duration_bins`` given as ``[[max_duration, max_tokens], ...]`` with one ``bucket_batch_size`` each: a cut goes
    to the first bin that fits both its duration and its token count."""

    def __init__(self, durations, num_tokens, bins2d, bucket_batch_size, **kw):
        bins2d = sorted([tuple(b) for b in bins2d])
        super().__init__(durations, bucket_duration_bins=[b[0] for b in bins2d][:-1] if len(bins2d) > 1 else None,
                         bucket_batch_size=bucket_batch_size, **kw)
        tok = np.asarray(num_tokens)
        bucket = np.full(len(tok), len(bins2d) - 1)
        for i, (d, t) in enumerate(zip(self.durs, tok)):
            for b, (md, mt) in enumerate(bins2d):
                if d <= md and t <= mt:
                    bucket[i] = b
                    break
        self.bucket_of = bucket
        self.bins = np.asarray([b[0] for b in bins2d][:-1], dtype=np.float64)


def determine_bucket_duration_bins(durations: Sequence[float], num_buckets: int) -> List[float]:
    """Equal-total-duration bin edges (``dataloader.py:830``)."""
    d = np.sort(np.asarray(durations, dtype=np.float64))
    c = np.cumsum(d)
    total = c[-1]
    return [float(d[min(len(d) - 1, bisect.bisect_left(c, total * k / num_buckets))]) for k in range(1, num_buckets)]


def _cfg(config) -> Dict[str, Any]:
    return to_container(config, resolve=True) if isinstance(config, DictConfig) else dict(config)


def build_cutset_from_config(c: Dict[str, Any], rank: int = 0, world: int = 1) -> CutSet:
    seed = c.get("seed", 0) if isinstance(c.get("seed", 0), int) else 0
    if c.get("input_cfg") is not None:
        cuts = parse_input_cfg(c["input_cfg"], seed, rank, world)
    elif c.get("tarred_audio_filepaths") is not None:
        cuts = read_nemo_tarred(c["manifest_filepath"], c["tarred_audio_filepaths"], None, rank, world)
    elif c.get("manifest_filepath") is not None:
        cuts = read_nemo_manifest(c["manifest_filepath"], c.get("lang_field", "lang"), c.get("text_field", "text"))
    elif c.get("shar_path") is not None or c.get("cuts_path") is not None:
        from .sources import get_parser

        cuts = get_parser("lhotse")(c, {"seed": seed, "rank": rank, "world": world})
    else:
        raise ValueError("the data config needs input_cfg, manifest_filepath, tarred_audio_filepaths, cuts_path or shar_path")
    from .sampling import CERFilter, ContextSpeakerSimilarityFilter, ValidationStatusFilter

    if c.get("keep_validation_status") is not None:
        cuts = cuts.filter(ValidationStatusFilter(c["keep_validation_status"]))
    if c.get("max_cer") is not None:
        cuts = cuts.filter(CERFilter(c["max_cer"]))
    if c.get("min_context_speaker_similarity") is not None:
        cuts = cuts.filter(ContextSpeakerSimilarityFilter(c["min_context_speaker_similarity"]))
    if c.get("cut_into_windows_duration"):
        cuts = cuts.cut_into_windows(float(c["cut_into_windows_duration"]))
    if c.get("truncate_duration"):
        rng = np.random.default_rng(seed) if c.get("truncate_offset_type", "start") == "random" else None
        cuts = cuts.truncate(float(c["truncate_duration"]), rng)
    lo, hi = c.get("min_duration"), c.get("max_duration")
    if lo is not None or hi is not None:
        from .sampling import DurationFilter

        cuts = cuts.filter(DurationFilter(lo, hi))
    ps = c.get("perturb_speed")
    if ps:
        factors = [0.9, 1.1] if ps is True else list(ps)
        base = cuts
        cuts = CutSet(lambda: (v for k in base for v in ([k] + [k.with_speed(f) for f in factors])))
    return cuts


def get_dataloader_from_cuts_config(config, global_rank: int = 0, world_size: int = 1, tokenizer=None, labels=None,
                                    dataset_cls=CutsSpeechToTextDataset):
    c = _cfg(config)
    if c.get("multi_config"):
        subs = [get_dataloader_from_cuts_config({**v, "multi_config": False}, global_rank, world_size, tokenizer, labels, dataset_cls)
                for k, v in c.items() if isinstance(v, dict) and k not in ("sampler_fusion",)]
        return FusedLoader(subs, mode=c.get("sampler_fusion", "round_robin"), weights=c.get("sampler_weights"), seed=c.get("seed", 0))
    tarred = c.get("tarred_audio_filepaths") is not None or c.get("shar_path") is not None
    cuts = build_cutset_from_config(c, global_rank if tarred else 0, world_size if tarred else 1).to_eager()
    aug: List[Callable] = []
    sr = c.get("sample_rate", 16000)
    if c.get("noise_path"):
        aug.append(NoiseMixer(list(read_nemo_manifest(c["noise_path"])), c.get("noise_snr", (10.0, 20.0)), c.get("noise_mix_prob", 0.5),
                              seed=global_rank, sr=sr))
    if c.get("rir_enabled"):
        aug.append(RIRConvolver(list(read_nemo_manifest(c["rir_path"])) if c.get("rir_path") else None, c.get("rir_prob", 0.5),
                                seed=global_rank, sr=sr))
    ds = dataset_cls(list(cuts), tokenizer=tokenizer, labels=labels, sample_rate=sr, augmentations=aug)
    min_tps, max_tps = c.get("min_tps"), c.get("max_tps")
    if min_tps is not None or max_tps is not None:
        keep = [i for i, k in enumerate(ds.cuts) if k.duration <= 0 or
                ((min_tps is None or ds.num_tokens(i) / k.duration >= min_tps) and (max_tps is None or ds.num_tokens(i) / k.duration <= max_tps))]
        ds.cuts = [ds.cuts[i] for i in keep]
    if any(c.get(k) is not None for k in ("min_tokens", "max_tokens", "min_tpt", "max_tpt")):
        from .sampling import TokenCountFilter, TokenPerTokenFilter

        ted_f = c.get("token_equivalent_duration")
        f1 = TokenCountFilter(c.get("min_tokens"), c.get("max_tokens"), bool(c.get("measure_total_length", False)), tokenizer, ted_f)
        f2 = TokenPerTokenFilter(c.get("min_tpt"), c.get("max_tpt"), tokenizer)
        ds.cuts = [k for k in ds.cuts if f1(k) and f2(k)]
    durs = ds.durations()
    if c.get("use_multimodal_sampling"):
        # every example is measured in tokens (audio converted with token_equivalent_duration); the bucketing sampler then
        # works on those lengths and "batch_duration" is the token budget of a mini-batch
        from .sampling import MultimodalSamplingConstraint

        msc = MultimodalSamplingConstraint(c.get("token_equivalent_duration"), measure_total_length=bool(c.get("measure_total_length", False)),
                                           tokenizer=tokenizer)
        durs = [msc.measure_length(k) for k in ds.cuts]
        c = {**c, "batch_duration": float(c["batch_tokens"]) if c.get("batch_tokens") else None,
             "quadratic_duration": c.get("quadratic_factor")}
    elif c.get("batch_tokens"):
        ted = float(c.get("token_equivalent_duration", 0.08))
        durs = [d + ds.num_tokens(i) * ted for i, d in enumerate(durs)]        # audio + text measured in seconds
        c = {**c, "batch_duration": float(c["batch_tokens"]) * ted}
    seed = c.get("shard_seed", c.get("seed", 0))
    seed = seed if isinstance(seed, int) else (int.from_bytes(os.urandom(4), "little") if seed == "randomized" else 0)
    sharded = world_size if not tarred else 1
    rank = global_rank if not tarred else 0
    common = dict(shuffle=c.get("shuffle", False), drop_last=c.get("drop_last", False), shard_seed=seed, rank=rank, world_size=sharded)
    bins = c.get("bucket_duration_bins")
    if bins is not None and len(bins) and isinstance(bins[0], (list, tuple)):
        sampler = TwoDimBucketingSampler(durs, [ds.num_tokens(i) for i in range(len(ds))], bins, c["bucket_batch_size"], **common)
    else:
        nb = c.get("num_buckets", 1) or 1
        if bins is None and nb > 1 and c.get("bucket_batch_size") is None:
            bins = determine_bucket_duration_bins(durs, nb)
        sampler = DynamicBucketingSampler(
            durs, batch_duration=c.get("batch_duration"), batch_size=c.get("batch_size") if c.get("batch_duration") is None else None,
            num_buckets=nb, bucket_duration_bins=bins, quadratic_duration=c.get("quadratic_duration"),
            max_batch_size=c.get("max_batch_size"), bucket_batch_size=c.get("bucket_batch_size"), **common)
    return BatchedLoader(ds, sampler, ds.collate_fn, num_workers=c.get("num_workers", 0), pin_memory=c.get("pin_memory", False),
                         prefetch_factor=c.get("prefetch_factor"))


class FusedLoader:
    """``multi_config``: several loaders fused ``round_robin`` (alternate), ``zip`` (tuple of batches) or ``randomized_round_robin``."""

    def __init__(self, loaders, mode: str = "round_robin", weights=None, seed: int = 0):
        self.loaders, self.mode, self.weights, self.seed = loaders, mode, weights, seed

    def __len__(self):
        return min(len(l) for l in self.loaders) if self.mode == "zip" else sum(len(l) for l in self.loaders)

    def __iter__(self):
        its = [iter(l) for l in self.loaders]
        if self.mode == "zip":
            yield from zip(*its)
            return
        rng = np.random.default_rng(self.seed)
        alive = list(range(len(its)))
        k = 0
        while alive:
            if self.mode == "randomized_round_robin":
                w = np.asarray([(self.weights or [1.0] * len(its))[i] for i in alive], dtype=np.float64)
                i = alive[int(rng.choice(len(alive), p=w / w.sum()))]
            else:
                i = alive[k % len(alive)]
                k += 1
            try:
                yield next(its[i])
            except StopIteration:
                alive.remove(i)


class BroadcastingDataLoader:
    """Under context / tensor parallelism only the data-parallel *source* rank of each (cp, tp) sub-mesh builds batches and
    broadcasts them (a "continue" flag first) to its peers (``common/data/lhotse/broadcasting.py:60-109``)."""

    def __init__(self, loader_factory: Callable[[], Iterable], group, src_rank: int, is_source: bool):
        self.group, self.src, self.is_source = group, src_rank, is_source
        self.loader = loader_factory() if is_source else None

    def __iter__(self):
        import torch.distributed as dist

        it = iter(self.loader) if self.is_source else None
        while True:
            payload = [None, None]
            if self.is_source:
                try:
                    payload = [True, next(it)]
                except StopIteration:
                    payload = [False, None]
            dist.broadcast_object_list(payload, src=self.src, group=self.group)
            if not payload[0]:
                return
            yield payload[1]

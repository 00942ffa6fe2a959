"""Further datasets: pre-computed features with labels / transcripts, text-only pairs, Hugging Face datasets, the DALI loader
gate and the multi-speaker session simulator.

Reference: ``asr/data/feature_to_label.py`` (``FeatureToSeqSpeakerLabelDataset``, ``FeatureToLabelDataset`` — features stored
as ``.npy`` / ``.pt``, window padding, ``feature_to_text.py`` ``FeatureToCharDataset`` / ``FeatureToBPEDataset``),
``asr/data/text_to_text.py`` (text → tokens pairs for text-only adaptation), ``asr/data/huggingface/hf_audio_to_text.py``
(manifest fields mapped from HF dataset columns, optional streaming), ``asr/data/audio_to_text_dali.py`` (DALI pipeline; an
optional dependency), ``asr/data/data_simulation.py`` (``MultiSpeakerSimulator``: sessions mixed from single-speaker
utterances with turn-taking, overlap / silence statistics, RTTM + JSON manifests).
"""
from __future__ import annotations

import json
import os
import random
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

from .audio_to_text import load_audio


def _load_feature(path: str) -> torch.Tensor:
    if path.endswith(".npy"):
        return torch.from_numpy(np.load(path)).float()
    return torch.load(path, map_location="cpu").float()


def _pad_stack(items: Sequence[torch.Tensor], pad_value: float = 0.0, dim: int = -1) -> Tuple[torch.Tensor, torch.Tensor]:
    lens = torch.tensor([t.shape[dim] for t in items], dtype=torch.long)
    T = int(lens.max()) if len(items) else 0
    out = []
    for t in items:
        pad = [0, 0] * t.dim()
        pad[2 * (t.dim() - 1 - (dim % t.dim())) + 1] = T - t.shape[dim]
        out.append(torch.nn.functional.pad(t, pad, value=pad_value))
    return torch.stack(out), lens


class FeatureToLabelDataset(Dataset):
    """Manifest lines ``{"feature_file": "x.npy", "label": "speech"}``; features ``[D, T]``.  Frame-level labels (a string of
    space-separated integers, ``is_regression_task`` floats) are supported through ``delimiter``."""

    def __init__(self, manifest_filepath: str, labels: Optional[List[str]] = None, augmentor: Optional[Callable] = None, window_length_in_sec: float = 0.63,
                 shift_length_in_sec: float = 0.01, is_regression_task: bool = False, delimiter: Optional[str] = None, zero_spec_db_val: float = -16.635):
        self.items = [json.loads(l) for p in manifest_filepath.split(",") for l in open(p, encoding="utf-8") if l.strip()]
        self.labels = list(labels) if labels else sorted({str(it["label"]) for it in self.items if delimiter is None})
        self.label2id = {l: i for i, l in enumerate(self.labels)}
        self.delimiter, self.is_regression, self.augmentor, self.pad_value = delimiter, is_regression_task, augmentor, zero_spec_db_val

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        f = _load_feature(it["feature_file"])
        if self.augmentor is not None:
            f = self.augmentor(f)
        if self.delimiter is not None:
            lab = torch.tensor([float(x) if self.is_regression else int(x) for x in str(it["label"]).split(self.delimiter if self.delimiter != " " else None)])
        elif self.is_regression:
            lab = torch.tensor([float(it["label"])])
        else:
            lab = torch.tensor([self.label2id[str(it["label"])]])
        return f, torch.tensor(f.shape[-1]), lab, torch.tensor(lab.shape[0])

    def collate_fn(self, batch):
        feats, flen = _pad_stack([b[0] for b in batch], self.pad_value)
        labs, llen = _pad_stack([b[2] for b in batch], 0)
        return feats, flen, labs, llen


class FeatureToTextDataset(Dataset):
    """Features + transcript (``FeatureToCharDataset`` with a character parser, ``FeatureToBPEDataset`` with a tokenizer)."""

    def __init__(self, manifest_filepath: str, tokenizer=None, labels: Optional[List[str]] = None, normalize: bool = False,
                 normalize_type: str = "per_feature", use_rttm: bool = False, rttm_mode: str = "mask", feat_min_len: int = 4,
                 feat_mask_val: Optional[float] = None, frame_unit_time_secs: float = 0.01, max_duration=None, min_duration=None, **_):
        self.items = [json.loads(l) for p in manifest_filepath.split(",") for l in open(p, encoding="utf-8") if l.strip()]
        if max_duration is not None:
            self.items = [it for it in self.items if it.get("duration", 0) <= max_duration]
        if min_duration is not None:
            self.items = [it for it in self.items if it.get("duration", 1e9) >= min_duration]
        self.tokenizer, self.labels = tokenizer, labels
        self.char2id = {c: i for i, c in enumerate(labels)} if labels else None
        self.normalize, self.use_rttm, self.rttm_mode = normalize, use_rttm, rttm_mode
        self.mask_val = feat_mask_val if feat_mask_val is not None else -16.635
        self.frame_secs, self.min_len = frame_unit_time_secs, feat_min_len

    def __len__(self):
        return len(self.items)

    def _tokens(self, text: str) -> List[int]:
        if self.tokenizer is not None:
            return list(self.tokenizer.text_to_ids(text))
        return [self.char2id[c] for c in text if c in self.char2id]

    def _apply_rttm(self, f: torch.Tensor, rttm_file: str) -> torch.Tensor:
        """``mask``: frames outside the RTTM speech segments get the mask value; ``drop``: they are removed."""
        keep = torch.zeros(f.shape[-1], dtype=torch.bool)
        with open(rttm_file) as fh:
            for line in fh:
                p = line.split()
                if len(p) >= 5 and p[0] == "SPEAKER":
                    a, d = float(p[3]), float(p[4])
                    keep[int(a / self.frame_secs): int((a + d) / self.frame_secs) + 1] = True
        if self.rttm_mode == "drop":
            f = f[..., keep]
            return f if f.shape[-1] >= self.min_len else torch.nn.functional.pad(f, (0, self.min_len - f.shape[-1]), value=self.mask_val)
        return torch.where(keep, f, torch.full_like(f, self.mask_val))

    def __getitem__(self, i):
        it = self.items[i]
        f = _load_feature(it["feature_file"])
        if self.use_rttm and it.get("rttm_file"):
            f = self._apply_rttm(f, it["rttm_file"])
        if self.normalize:
            f = (f - f.mean(-1, keepdim=True)) / (f.std(-1, keepdim=True) + 1e-5)
        t = torch.tensor(self._tokens(it.get("text", "")), dtype=torch.long)
        return f, torch.tensor(f.shape[-1]), t, torch.tensor(t.shape[0])

    def collate_fn(self, batch):
        feats, flen = _pad_stack([b[0] for b in batch], self.mask_val)
        toks, tlen = _pad_stack([b[2] for b in batch], 0)
        return feats, flen, toks, tlen


FeatureToCharDataset = FeatureToBPEDataset = FeatureToTextDataset


class TextToTextDataset(Dataset):
    """Text-only examples for adapting the decoder / language side: ``(source tokens, target tokens)`` from a manifest with
    ``text`` (and optional ``source_text``) or from a plain text file; a TTS front end may be attached through ``text_to_audio``."""

    def __init__(self, manifest_filepath: str, tokenizer, source_tokenizer=None, text_to_audio: Optional[Callable[[str], torch.Tensor]] = None,
                 max_length: Optional[int] = None):
        self.items = []
        for p in manifest_filepath.split(","):
            with open(p, encoding="utf-8") as f:
                for line in f:
                    line = line.strip()
                    if not line:
                        continue
                    it = json.loads(line) if line.startswith("{") else {"text": line}
                    self.items.append(it)
        self.tok, self.src_tok, self.tta, self.max_length = tokenizer, source_tokenizer or tokenizer, text_to_audio, max_length

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        tgt = torch.tensor(list(self.tok.text_to_ids(it["text"]))[: self.max_length], dtype=torch.long)
        src_text = it.get("source_text", it["text"])
        src = self.tta(src_text) if self.tta is not None else torch.tensor(list(self.src_tok.text_to_ids(src_text))[: self.max_length], dtype=torch.long)
        return src, torch.tensor(src.shape[-1]), tgt, torch.tensor(tgt.shape[0])

    def collate_fn(self, batch):
        src, sl = _pad_stack([b[0] for b in batch], 0)
        tgt, tl = _pad_stack([b[2] for b in batch], 0)
        return src, sl, tgt, tl


class HFAudioToTextDataset(Dataset):
    """Rows of a Hugging Face ``datasets`` dataset (or any sequence of dicts) mapped to (audio, length, tokens, length).
    ``audio_key`` / ``text_key`` may be dotted paths (``"audio.array"``); ``sample_rate_key`` likewise."""

    def __init__(self, data=None, path: Optional[str] = None, name: Optional[str] = None, split: str = "train", audio_key: str = "audio.array",
                 text_key: str = "text", sample_rate_key: str = "audio.sampling_rate", tokenizer=None, labels: Optional[List[str]] = None,
                 sample_rate: int = 16000, normalize_text: bool = False, streaming: bool = False, **load_kwargs):
        if data is None:
            try:
                import datasets
            except ImportError as e:  # pragma: no cover - optional dependency
                raise ImportError("HFAudioToTextDataset needs the `datasets` package when no in-memory `data` is given") from e
            data = datasets.load_dataset(path, name, split=split, streaming=streaming, **load_kwargs)
        self.data, self.audio_key, self.text_key, self.sr_key = data, audio_key, text_key, sample_rate_key
        self.tokenizer, self.sample_rate, self.normalize_text = tokenizer, sample_rate, normalize_text
        self.char2id = {c: i for i, c in enumerate(labels)} if labels else None

    @staticmethod
    def _get(row, dotted: str):
        for k in dotted.split("."):
            row = row[k]
        return row

    def __len__(self):
        return len(self.data)

    def __getitem__(self, i):
        from .perturb import resample

        row = self.data[i]
        x = np.asarray(self._get(row, self.audio_key), dtype=np.float32)
        try:
            sr = int(self._get(row, self.sr_key))
        except (KeyError, TypeError):
            sr = self.sample_rate
        x = torch.from_numpy(resample(x, sr, self.sample_rate))
        text = str(self._get(row, self.text_key))
        if self.normalize_text:
            text = "".join(c for c in text.lower() if c.isalnum() or c in " '")
        ids = list(self.tokenizer.text_to_ids(text)) if self.tokenizer is not None else [self.char2id[c] for c in text if c in self.char2id]
        t = torch.tensor(ids, dtype=torch.long)
        return x, torch.tensor(x.shape[0]), t, torch.tensor(t.shape[0])

    def collate_fn(self, batch):
        a, al = _pad_stack([b[0] for b in batch], 0.0)
        t, tl = _pad_stack([b[2] for b in batch], 0)
        return a, al, t, tl


def dali_available() -> bool:
    try:
        import nvidia.dali  # noqa: F401

        return True
    except ImportError:
        return False


class AudioToCharDALIDataset:
    """Placeholder for the DALI loading pipeline: DALI is an optional package that this environment does not ship; the regular
    loaders (``AudioToCharDataset`` + the fused log-mel kernel) cover the same data and run the feature extraction on the GPU."""

    def __init__(self, *a, **kw):
        raise ImportError("NVIDIA DALI is not installed; use speech_b200.data.audio_to_text datasets (features are computed on the GPU "
                          "by the fused log-mel kernel) or the cuts loader")


# ---------------------------------------------------------------------------------------------- multi-speaker simulator
class MultiSpeakerSimulator:
    """Builds synthetic multi-speaker sessions from single-speaker utterances.

    Speakers take turns; after every utterance the next one starts either overlapping the tail of the session (probability
    derived from ``overlap_prob``, overlap length exponential with mean ``mean_overlap``) or after a silence (exponential with
    mean ``mean_silence``).  ``turn_prob`` is the probability that the speaker changes.  Output per session: mixed waveform,
    RTTM lines, a JSON manifest entry and word-level CTM-like timings when the source items carry ``words`` / ``alignments``."""

    def __init__(self, items: Sequence[Dict[str, Any]], sample_rate: int = 16000, num_speakers: int = 2, session_length: float = 60.0,
                 turn_prob: float = 0.875, overlap_prob: float = 0.1, mean_overlap: float = 0.6, mean_silence: float = 0.4,
                 min_volume: float = 0.7, max_volume: float = 1.0, seed: int = 0, loader: Optional[Callable[[Dict[str, Any]], np.ndarray]] = None):
        self.by_spk: Dict[str, List[Dict[str, Any]]] = {}
        for it in items:
            self.by_spk.setdefault(str(it.get("speaker_id", it.get("speaker", "spk"))), []).append(it)
        if len(self.by_spk) < num_speakers:
            raise ValueError(f"need utterances of at least {num_speakers} speakers, found {len(self.by_spk)}")
        self.sr, self.n_spk, self.length = sample_rate, num_speakers, session_length
        self.turn_prob, self.overlap_prob, self.mean_overlap, self.mean_silence = turn_prob, overlap_prob, mean_overlap, mean_silence
        self.vol = (min_volume, max_volume)
        self.rng = random.Random(seed)
        self.loader = loader or (lambda it: np.asarray(it["samples"], np.float32) if "samples" in it else
                                 load_audio(it["audio_filepath"], self.sr, it.get("offset", 0.0) or 0.0, it.get("duration")))

    def generate_session(self, session_id: str = "session_0") -> Dict[str, Any]:
        speakers = self.rng.sample(sorted(self.by_spk), self.n_spk)
        vols = {s: self.rng.uniform(*self.vol) for s in speakers}
        n_total = int(self.length * self.sr)
        mix = np.zeros(n_total, np.float32)
        rttm, segs = [], []
        cursor, spk = 0, self.rng.choice(speakers)
        while cursor < n_total:
            it = self.rng.choice(self.by_spk[spk])
            x = self.loader(it)
            n = min(x.shape[0], n_total - cursor)
            if n <= 0:
                break
            mix[cursor:cursor + n] += x[:n] * vols[spk]
            a, d = cursor / self.sr, n / self.sr
            rttm.append(f"SPEAKER {session_id} 1 {a:.3f} {d:.3f} <NA> <NA> {spk} <NA> <NA>")
            segs.append({"speaker": spk, "start": a, "end": a + d, "text": it.get("text", "")})
            end = cursor + n
            prev = spk
            if self.rng.random() < self.turn_prob:
                spk = self.rng.choice([s for s in speakers if s != prev])
            if spk != prev and self.rng.random() < self.overlap_prob:
                cursor = max(cursor + 1, end - int(self.rng.expovariate(1.0 / self.mean_overlap) * self.sr))
            else:
                cursor = end + int(self.rng.expovariate(1.0 / self.mean_silence) * self.sr)
        peak = float(np.abs(mix).max())
        if peak > 1.0:
            mix /= peak
        return {"session_id": session_id, "audio": mix, "sample_rate": self.sr, "rttm": rttm, "segments": segs, "speakers": speakers,
                "text": " ".join(s["text"] for s in segs if s["text"])}

    def generate_sessions(self, num_sessions: int, output_dir: Optional[str] = None) -> List[Dict[str, Any]]:
        out = []
        for k in range(num_sessions):
            s = self.generate_session(f"multispeaker_session_{k}")
            if output_dir is not None:
                from scipy.io import wavfile

                os.makedirs(output_dir, exist_ok=True)
                wav, rt = os.path.join(output_dir, s["session_id"] + ".wav"), os.path.join(output_dir, s["session_id"] + ".rttm")
                wavfile.write(wav, self.sr, (np.clip(s["audio"], -1, 1) * 32767).astype(np.int16))
                with open(rt, "w") as f:
                    f.write("\n".join(s["rttm"]) + "\n")
                with open(os.path.join(output_dir, "manifest.json"), "a") as f:
                    f.write(json.dumps({"audio_filepath": wav, "offset": 0, "duration": self.length, "label": "infer", "text": s["text"],
                                        "num_speakers": self.n_spk, "rttm_filepath": rt}) + "\n")
            out.append(s)
        return out


class SemiSortBatchSampler(torch.utils.data.Sampler):
    """Batches of similar durations with randomness: every epoch the durations are perturbed by uniform noise of
    ``+-randomization_factor * (max - min) / 2``, the utterances sorted by the perturbed value, cut into batches of ``batch_size``
    and the batches shuffled; with ``world_size > 1`` every rank takes every ``world_size``-th batch (the list is padded by
    repeating batches so that all ranks get the same count).  Reference: ``asr/parts/utils/asr_batching.py``
    (``SemiSortBatchSampler``)."""

    def __init__(self, durations, batch_size: int, randomization_factor: float = 0.1, drop_last: bool = False, shuffle: bool = True,
                 global_rank: int = 0, world_size: int = 1, seed: int = 0):
        import numpy as np

        if randomization_factor < 0:
            raise ValueError("randomization_factor must be non-negative")
        self.dur = np.asarray(durations, dtype=np.float64)
        self.bs, self.rf, self.drop_last, self.shuffle = int(batch_size), float(randomization_factor), drop_last, shuffle
        self.rank, self.world, self.seed, self.epoch = global_rank, world_size, seed, 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def _batches(self):
        import numpy as np

        g = np.random.default_rng(self.seed + self.epoch)
        spread = (self.dur.max() - self.dur.min()) * self.rf / 2 if len(self.dur) else 0.0
        keys = self.dur + g.uniform(-spread, spread, size=len(self.dur)) if spread > 0 else self.dur
        order = np.argsort(keys, kind="stable")
        batches = [order[i:i + self.bs].tolist() for i in range(0, len(order), self.bs)]
        if self.drop_last and batches and len(batches[-1]) < self.bs:
            batches.pop()
        if self.shuffle:
            perm = g.permutation(len(batches))
            batches = [batches[i] for i in perm]
        if self.world > 1 and batches:
            pad = (-len(batches)) % self.world
            batches = batches + batches[:pad]
            batches = batches[self.rank::self.world]
        return batches

    def __iter__(self):
        return iter(self._batches())

    def __len__(self):
        n = len(self.dur) // self.bs if self.drop_last else -(-len(self.dur) // self.bs)
        return -(-n // self.world)

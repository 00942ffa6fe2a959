"""Manifest collections: lists of named tuples parsed from JSON-lines manifests, filtered by duration / count and optionally
sorted, which the datasets index into.  One collection per manifest flavour — audio + text, audio + class label, feature files +
labels or text, diarization sessions with RTTM files, multi-signal audio, and audio + context / answer pairs of speech-LLM data.
Reference: ``common/parts/preprocessing/collections.py`` and ``common/parts/preprocessing/manifest.py``.
"""
from __future__ import annotations

import collections
import json
import os
from itertools import combinations
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Union

from ..utils.logging import logging


# ---------------------------------------------------------------------------------------------------------------- manifest
def get_full_path(audio_file: Union[str, List[str]], manifest_file: Optional[str] = None, data_dir: Optional[str] = None,
                  audio_file_len_limit: int = 255) -> Union[str, List[str]]:
    """A relative path that does not exist from the working directory is taken relative to ``data_dir`` or to the manifest's
    folder (if it exists there); absolute paths, overlong strings and paths that exist as given are returned unchanged."""
    if isinstance(audio_file, (list, tuple)):
        return [get_full_path(a, manifest_file, data_dir, audio_file_len_limit) for a in audio_file]
    if not isinstance(audio_file, str) or len(audio_file) >= audio_file_len_limit or os.path.isabs(audio_file) or os.path.isfile(audio_file):
        return audio_file
    base = data_dir if data_dir is not None else (os.path.dirname(manifest_file) if manifest_file else None)
    if base is None:
        return audio_file
    cand = os.path.join(base, audio_file)
    return os.path.abspath(cand) if os.path.isfile(cand) else audio_file


def parse_item(line: str, manifest_file: str) -> Dict[str, Any]:
    """One manifest line with its keys normalised: ``audio_file`` (from ``audio_filename`` / ``audio_filepath``), ``duration`` (from
    ``context_duration`` when absent), ``text`` (inline, from ``text_filepath`` or ``normalized_text``), ``rttm_file``,
    ``feature_file``, plus ``offset``, ``speaker``, ``orig_sr``, ``token_labels``, ``lang``."""
    item = json.loads(line)
    for k in ("audio_filename", "audio_filepath"):
        if k in item:
            item["audio_file"] = item.pop(k)
            break
    else:
        if "context" in item and "audio_file" not in item:                       # text-only speech-LLM entry
            item["audio_file"] = None
            item.setdefault("duration", item.get("context_duration", 0.0))
    if "audio_file" not in item:
        raise ValueError(f"manifest {manifest_file}: an entry has no audio file key: {line.strip()[:120]}")
    if item["audio_file"] is not None:
        item["audio_file"] = get_full_path(item["audio_file"], manifest_file)
    if "duration" not in item:
        if "context_duration" in item:
            item["duration"] = item["context_duration"]
        else:
            raise ValueError(f"manifest {manifest_file}: an entry has no duration: {line.strip()[:120]}")
    if "text" not in item:
        if "text_filepath" in item:
            with open(get_full_path(item.pop("text_filepath"), manifest_file), encoding="utf-8") as f:
                item["text"] = f.read().replace("\n", "")
        else:
            item["text"] = item.get("normalized_text", "")
    for dst, keys in (("rttm_file", ("rttm_file", "rttm_filename", "rttm_filepath")), ("feature_file", ("feature_file", "feature_filename", "feature_filepath"))):
        for k in keys:
            if k in item:
                item[dst] = get_full_path(item.pop(k) if k != dst else item[k], manifest_file)
                break
        else:
            item[dst] = None
    return dict(item, offset=item.get("offset"), speaker=item.get("speaker"), orig_sr=item.get("orig_sample_rate", item.get("orig_sr")),
                token_labels=item.get("token_labels"), lang=item.get("lang"))


def item_iter(manifests_files: Union[str, Sequence[str]], parse_func: Optional[Callable[[str, str], Dict[str, Any]]] = None) -> Iterator[Dict[str, Any]]:
    """Entries of one or several manifests (comma-separated string or list), each with a running ``id``."""
    if isinstance(manifests_files, str):
        manifests_files = manifests_files.split(",")
    parse_func = parse_func or parse_item
    k = -1
    for m in manifests_files:
        m = os.path.expanduser(str(m).strip())
        with open(m, encoding="utf-8") as f:
            for line in f:
                if not line.strip():
                    continue
                k += 1
                item = parse_func(line, m)
                item["id"] = k
                yield item


class _Collection(collections.UserList):
    """A list of ``OUTPUT_TYPE`` tuples."""

    OUTPUT_TYPE = None


def _filter_report(kind: str, kept: int, kept_h: float, dropped: int, dropped_h: float) -> None:
    logging.info("%s: %d entries (%.2f h) kept, %d entries (%.2f h) filtered out", kind, kept, kept_h, dropped, dropped_h)


# --------------------------------------------------------------------------------------------------------------------- text
class Text(_Collection):
    OUTPUT_TYPE = collections.namedtuple("TextEntity", "tokens")

    def __init__(self, texts: List[str], parser: Callable[[str], Optional[List[int]]]):
        data = []
        for t in texts:
            tokens = parser(t)
            if tokens is None:
                logging.warning("unparsable text skipped: %r", t[:60])
                continue
            data.append(self.OUTPUT_TYPE(tokens))
        super().__init__(data)


class FromFileText(Text):
    """Texts from a ``.txt`` (one per line), ``.csv`` (column ``transcript``) or ``.json`` manifest (key ``text``)."""

    def __init__(self, file: str, parser):
        super().__init__(self._read(file), parser)

    @staticmethod
    def _read(file: str) -> List[str]:
        ext = os.path.splitext(file)[1].lower()
        if ext == ".csv":
            import csv

            with open(file, newline="", encoding="utf-8") as f:
                return [row["transcript"] for row in csv.DictReader(f)]
        if ext == ".json":
            return [it["text"] for it in item_iter(file)]
        with open(file, encoding="utf-8") as f:
            return [l.rstrip("\n") for l in f]


# --------------------------------------------------------------------------------------------------------------- audio+text
class AudioText(_Collection):
    OUTPUT_TYPE = collections.namedtuple("AudioTextEntity", "id audio_file duration text_tokens offset text_raw speaker orig_sr lang")

    def __init__(self, ids, audio_files, durations, texts, offsets, speakers, orig_sampling_rates, token_labels, langs, parser,
                 min_duration: Optional[float] = None, max_duration: Optional[float] = None, max_number: Optional[int] = None,
                 do_sort_by_duration: bool = False, index_by_file_id: bool = False):
        self.mapping: Dict[str, int] = {}
        data, dropped, dropped_h, kept_h = [], 0, 0.0, 0.0
        for id_, af, dur, text, off, spk, sr, tl, lang in zip(ids, audio_files, durations, texts, offsets, speakers, orig_sampling_rates, token_labels, langs):
            if (min_duration is not None and dur < min_duration) or (max_duration is not None and dur > max_duration):
                dropped, dropped_h = dropped + 1, dropped_h + dur
                continue
            if tl is not None:
                tokens = tl
            elif text != "":
                try:
                    tokens = parser(text, lang) if lang is not None and getattr(parser, "is_aggregate", False) else parser(text)
                except TypeError:
                    tokens = parser(text)
            else:
                tokens = []
            if tokens is None:
                dropped, dropped_h = dropped + 1, dropped_h + dur
                continue
            data.append(self.OUTPUT_TYPE(id_, af, dur, tokens, off, text, spk, sr, lang))
            kept_h += dur
            if index_by_file_id and af is not None:
                key = os.path.splitext(os.path.basename(af if isinstance(af, str) else af[0]))[0]
                if key not in self.mapping:
                    self.mapping[key] = []
                self.mapping[key].append(len(data) - 1)
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration:
            if index_by_file_id:
                logging.warning("sorting by duration is skipped because the collection is indexed by file id")
            else:
                data.sort(key=lambda e: e.duration)
        _filter_report(type(self).__name__, len(data), kept_h / 3600, dropped, dropped_h / 3600)
        super().__init__(data)


class ASRAudioText(AudioText):
    def __init__(self, manifests_files: Union[str, List[str]], parse_func: Optional[Callable] = None, *args, **kwargs):
        cols = [[] for _ in range(9)]
        for it in item_iter(manifests_files, parse_func=parse_func):
            for c, k in zip(cols, ("id", "audio_file", "duration", "text", "offset", "speaker", "orig_sr", "token_labels", "lang")):
                c.append(it.get(k))
        super().__init__(*cols, *args, **kwargs)


# --------------------------------------------------------------------------------------------------------------- speech LLM
class SpeechLLMAudioTextEntity:
    def __init__(self, sid, audio_file, duration, context, answer, offset, speaker, orig_sr, lang):
        self.id, self.audio_file, self.duration, self.context, self.answer = sid, audio_file, duration, context, answer
        self.offset, self.speaker, self.orig_sr, self.lang = offset, speaker, orig_sr, lang

    def __repr__(self):
        return f"SpeechLLMAudioTextEntity(id={self.id}, audio_file={self.audio_file!r}, duration={self.duration}, context={self.context!r}, answer={self.answer!r})"


class SpeechLLMAudioText:
    """Audio with a text context (question / instruction) and an answer, both kept as raw strings (the model's prompt formatter
    tokenises them).  ``max_num_samples`` draws that many entries at random with a seed."""

    def __init__(self, ids, audio_files, durations, context_list, answers, offsets, speakers=None, orig_sampling_rates=None, langs=None,
                 min_duration: Optional[float] = None, max_duration: Optional[float] = None, max_number: Optional[int] = None,
                 do_sort_by_duration: bool = False, index_by_file_id: bool = False, max_num_samples: Optional[int] = None, seed: int = 0):
        n = len(ids)
        speakers, orig_sampling_rates, langs = speakers or [None] * n, orig_sampling_rates or [None] * n, langs or [None] * n
        self.mapping: Dict[str, List[int]] = {}
        data = []
        for k in range(n):
            dur = durations[k]
            if (min_duration is not None and dur < min_duration) or (max_duration is not None and dur > max_duration):
                continue
            data.append(SpeechLLMAudioTextEntity(ids[k], audio_files[k], dur, context_list[k], answers[k], offsets[k], speakers[k], orig_sampling_rates[k], langs[k]))
            if index_by_file_id and audio_files[k] is not None:
                self.mapping.setdefault(os.path.splitext(os.path.basename(audio_files[k]))[0], []).append(len(data) - 1)
            if max_number is not None and len(data) == max_number:
                break
        if max_num_samples is not None and not index_by_file_id and 0 < max_num_samples < len(data):
            import random

            data = random.Random(seed).sample(data, max_num_samples)
        if do_sort_by_duration and not index_by_file_id:
            data.sort(key=lambda e: e.duration)
        self.data = data

    def __getitem__(self, i):
        if not 0 <= i < len(self.data):
            raise IndexError(i)
        return self.data[i]

    def __len__(self):
        return len(self.data)


class SpeechLLMAudioTextCollection(SpeechLLMAudioText):
    """From manifests: the context comes from ``context_key`` (a file path when ``context_file`` is given draws a random line of it, and a
    missing context falls back to ``default_context``), the answer from ``answer_key`` (``answer`` / ``text`` by default)."""

    def __init__(self, manifests_files: Union[str, List[str]], context_file: Optional[str] = None, context_key: str = "context", answer_key: str = "answer",
                 default_context: str = "what does this audio mean", seed: int = 0, *args, **kwargs):
        import random

        self._rng = random.Random(seed)
        self._contexts = None
        if context_file:
            with open(context_file, encoding="utf-8") as f:
                self._contexts = [l.strip() for l in f if l.strip()]
        ids, afs, durs, ctxs, answers, offs, spks, srs, langs = [], [], [], [], [], [], [], [], []
        for it in item_iter(manifests_files):
            raw = it
            if self._contexts:
                ctx = self._rng.choice(self._contexts)
            else:
                ctx = raw.get(context_key) or raw.get("question") or default_context
            ans = raw.get(answer_key)
            if ans is None:
                ans = raw.get("answer", raw.get("text", ""))
            for lst, v in zip((ids, afs, durs, ctxs, answers, offs, spks, srs, langs),
                              (it["id"], it["audio_file"], it["duration"], ctx, ans, it["offset"], it["speaker"], it["orig_sr"], it["lang"])):
                lst.append(v)
        super().__init__(ids, afs, durs, ctxs, answers, offs, spks, srs, langs, *args, seed=seed, **kwargs)


# -------------------------------------------------------------------------------------------------------------- class labels
class SpeechLabel(_Collection):
    OUTPUT_TYPE = collections.namedtuple("SpeechLabelEntity", "audio_file duration label offset")

    def __init__(self, audio_files, durations, labels, offsets, min_duration=None, max_duration=None, max_number=None,
                 do_sort_by_duration: bool = False, index_by_file_id: bool = False):
        self.mapping: Dict[str, int] = {}
        data, self.uniq_labels = [], set()
        dropped = 0
        for af, dur, lab, off in zip(audio_files, durations, labels, offsets):
            if (min_duration is not None and dur < min_duration) or (max_duration is not None and dur > max_duration):
                dropped += 1
                continue
            data.append(self.OUTPUT_TYPE(af, dur, lab, off))
            self.uniq_labels.add(lab)
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(af))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration and not index_by_file_id:
            data.sort(key=lambda e: e.duration)
        self.uniq_labels = sorted(self.uniq_labels, key=str)
        _filter_report(type(self).__name__, len(data), sum(e.duration or 0 for e in data) / 3600, dropped, 0.0)
        super().__init__(data)


class ASRSpeechLabel(SpeechLabel):
    """Manifest entries carry ``label`` (or ``command`` / ``target``); with ``is_regression_task`` the label is a float, with
    ``cal_labels_occurrence`` the per-label counts are kept in ``labels_occurrence``."""

    def __init__(self, manifests_files, is_regression_task: bool = False, cal_labels_occurrence: bool = False, delimiter: Optional[str] = None, *args, **kwargs):
        afs, durs, labs, offs = [], [], [], []
        occ: Dict[Any, int] = collections.Counter()
        for it in item_iter(manifests_files, parse_func=lambda l, m: self._parse(l, m, is_regression_task)):
            afs.append(it["audio_file"]); durs.append(it["duration"]); labs.append(it["label"]); offs.append(it["offset"])
            if cal_labels_occurrence and not is_regression_task:
                for l in (str(it["label"]).split(delimiter) if delimiter else [it["label"]]):
                    occ[l] += 1
        self.labels_occurrence = dict(occ) if cal_labels_occurrence else None
        super().__init__(afs, durs, labs, offs, *args, **kwargs)

    @staticmethod
    def _parse(line: str, manifest_file: str, regression: bool) -> Dict[str, Any]:
        item = json.loads(line)
        af = item.get("audio_filename", item.get("audio_filepath"))
        if af is None:
            raise ValueError(f"manifest {manifest_file}: an entry has no audio file key")
        for k in ("label", "command", "target"):
            if k in item:
                label = item[k]
                break
        else:
            raise ValueError(f"manifest {manifest_file}: an entry has no label (keys tried: label, command, target)")
        return dict(audio_file=get_full_path(af, manifest_file), duration=item.get("duration"), label=float(label) if regression else label, offset=item.get("offset"))


# ------------------------------------------------------------------------------------------------------------------ features
class FeatureSequenceLabel(_Collection):
    OUTPUT_TYPE = collections.namedtuple("FeatureSequenceLabelEntity", "feature_file seq_label")

    def __init__(self, feature_files, seq_labels, max_number=None, index_by_file_id: bool = False):
        self.mapping, self.uniq_labels = {}, set()
        data = []
        for ff, seq in zip(feature_files, seq_labels):
            labs = self.relative_speaker_parser(seq)
            data.append(self.OUTPUT_TYPE(ff, labs))
            self.uniq_labels |= set(labs)
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(ff))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        super().__init__(data)

    @staticmethod
    def relative_speaker_parser(seq_label: str) -> List[int]:
        """Speaker names in order of first appearance become 0, 1, 2, ... (``'c a c b'`` → ``[0, 1, 0, 2]``)."""
        seen: Dict[str, int] = {}
        return [seen.setdefault(s, len(seen)) for s in seq_label.split()]


class ASRFeatureSequenceLabel(FeatureSequenceLabel):
    def __init__(self, manifests_files, max_number=None, index_by_file_id: bool = False):
        ffs, seqs = [], []
        for it in item_iter(manifests_files, parse_func=self._parse):
            ffs.append(it["feature_file"]); seqs.append(it["seq_label"])
        super().__init__(ffs, seqs, max_number, index_by_file_id)

    @staticmethod
    def _parse(line, manifest_file):
        item = json.loads(line)
        ff = item.get("feature_filename", item.get("feature_filepath", item.get("feature_file")))
        if ff is None or "seq_label" not in item:
            raise ValueError(f"manifest {manifest_file}: an entry needs a feature file and 'seq_label'")
        return dict(feature_file=get_full_path(ff, manifest_file), seq_label=item["seq_label"])


class FeatureLabel(_Collection):
    OUTPUT_TYPE = collections.namedtuple("FeatureLabelEntity", "feature_file label duration")

    def __init__(self, feature_files, labels, durations, min_duration=None, max_duration=None, max_number=None, index_by_file_id: bool = False):
        self.mapping, self.uniq_labels = {}, set()
        data = []
        for ff, lab, dur in zip(feature_files, labels, durations):
            if (min_duration is not None and dur is not None and dur < min_duration) or (max_duration is not None and dur is not None and dur > max_duration):
                continue
            data.append(self.OUTPUT_TYPE(ff, lab, dur))
            self.uniq_labels.add(lab)
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(ff))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        self.uniq_labels = sorted(self.uniq_labels, key=str)
        super().__init__(data)


class ASRFeatureLabel(FeatureLabel):
    """``is_regression_task`` → float label; ``delimiter`` with ``cal_labels_occurrence`` counts the labels of multi-label entries."""

    def __init__(self, manifests_files, is_regression_task: bool = False, cal_labels_occurrence: bool = False, delimiter: Optional[str] = None, *args, **kwargs):
        ffs, labs, durs = [], [], []
        occ = collections.Counter()
        for it in item_iter(manifests_files, parse_func=lambda l, m: self._parse(l, m, is_regression_task)):
            ffs.append(it["feature_file"]); labs.append(it["label"]); durs.append(it["duration"])
            if cal_labels_occurrence and not is_regression_task:
                for l in (str(it["label"]).split(delimiter) if delimiter else [it["label"]]):
                    occ[l] += 1
        self.labels_occurrence = dict(occ) if cal_labels_occurrence else None
        super().__init__(ffs, labs, durs, *args, **kwargs)

    @staticmethod
    def _parse(line, manifest_file, regression):
        item = json.loads(line)
        ff = item.get("feature_filename", item.get("feature_filepath", item.get("feature_file")))
        if ff is None or "label" not in item:
            raise ValueError(f"manifest {manifest_file}: an entry needs a feature file and 'label'")
        return dict(feature_file=get_full_path(ff, manifest_file), label=float(item["label"]) if regression else item["label"], duration=item.get("duration"))


class FeatureText(_Collection):
    OUTPUT_TYPE = collections.namedtuple("FeatureTextEntity", "id feature_file rttm_file duration text_tokens offset text_raw speaker orig_sr lang")

    def __init__(self, ids, feature_files, rttm_files, durations, texts, offsets, speakers, orig_sampling_rates, token_labels, langs, parser,
                 min_duration=None, max_duration=None, max_number=None, do_sort_by_duration: bool = False, index_by_file_id: bool = False):
        self.mapping = {}
        data = []
        for id_, ff, rf, dur, text, off, spk, sr, tl, lang in zip(ids, feature_files, rttm_files, durations, texts, offsets, speakers, orig_sampling_rates, token_labels, langs):
            if (min_duration is not None and dur < min_duration) or (max_duration is not None and dur > max_duration):
                continue
            tokens = tl if tl is not None else (parser(text) if text != "" else [])
            if tokens is None:
                continue
            data.append(self.OUTPUT_TYPE(id_, ff, rf, dur, tokens, off, text, spk, sr, lang))
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(ff))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration and not index_by_file_id:
            data.sort(key=lambda e: e.duration)
        super().__init__(data)


class ASRFeatureText(FeatureText):
    def __init__(self, manifests_files, *args, **kwargs):
        cols = [[] for _ in range(10)]
        for it in item_iter(manifests_files, parse_func=self._parse):
            for c, k in zip(cols, ("id", "feature_file", "rttm_file", "duration", "text", "offset", "speaker", "orig_sr", "token_labels", "lang")):
                c.append(it.get(k))
        super().__init__(*cols, *args, **kwargs)

    @staticmethod
    def _parse(line, manifest_file):
        item = json.loads(line)
        if not any(k in item for k in ("audio_filename", "audio_filepath", "audio_file")):
            item["audio_filepath"] = item.get("feature_file", item.get("feature_filepath", item.get("feature_filename", "")))
        return parse_item(json.dumps(item), manifest_file)


# --------------------------------------------------------------------------------------------------------------- diarization
def _rttm_speakers(rttm_file: str) -> List[str]:
    spk = []
    with open(rttm_file) as f:
        for line in f:
            p = line.split()
            if len(p) >= 8 and p[0] == "SPEAKER" and p[7] not in spk:
                spk.append(p[7])
    return spk


class DiarizationLabel(_Collection):
    OUTPUT_TYPE = collections.namedtuple("DiarizationLabelEntity", "audio_file duration rttm_file offset target_spks sess_spk_dict clus_spk_digits rttm_spk_digits")

    def __init__(self, audio_files, durations, rttm_files, offsets, target_spks_list, sess_spk_dicts, clus_spk_list, rttm_spk_list,
                 max_number=None, do_sort_by_duration: bool = False, index_by_file_id: bool = False):
        self.mapping = {}
        data = []
        for vals in zip(audio_files, durations, rttm_files, offsets, target_spks_list, sess_spk_dicts, clus_spk_list, rttm_spk_list):
            data.append(self.OUTPUT_TYPE(*vals))
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(vals[0]))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration and not index_by_file_id:
            data.sort(key=lambda e: e.duration)
        super().__init__(data)


class DiarizationSpeechLabel(DiarizationLabel):
    """Sessions for the pairwise multi-scale diarization decoder.  For training every session is one entry whose target speakers are
    the first two speakers of its RTTM; for inference (``pairwise_infer``) a session with n estimated speakers (from ``clus_label_dict``:
    session id → cluster labels ``'start end speaker_k'``) gives one entry per speaker pair (a single-speaker session pairs it with a
    dummy second speaker)."""

    def __init__(self, manifests_files, emb_dict=None, clus_label_dict=None, round_digit: int = 2, seq_eval_mode: bool = False, pairwise_infer: bool = False, *args, **kwargs):
        self.round_digit, self.emb_dict, self.clus_label_dict = round_digit, emb_dict, clus_label_dict
        self.seq_eval_mode, self.pairwise_infer = seq_eval_mode, pairwise_infer
        cols = [[] for _ in range(8)]
        for it in item_iter(manifests_files, parse_func=_parse_diar_item):
            uniq = os.path.splitext(os.path.basename(it["audio_file"]))[0]
            rttm_spk = _rttm_speakers(it["rttm_file"]) if it["rttm_file"] and os.path.isfile(it["rttm_file"]) else []
            if pairwise_infer:
                clus = sorted({int(l.split()[-1].split("_")[-1]) for l in (clus_label_dict or {}).get(uniq, [])})
                sess = {k: s for k, s in enumerate(rttm_spk)}
                pairs = list(combinations(clus, 2)) if len(clus) > 1 else [(clus[0] if clus else 0, (clus[0] if clus else 0) + 1)]
                clus_digits, rttm_digits = clus, list(range(len(rttm_spk)))
            else:
                sess = {k: s for k, s in enumerate(rttm_spk)}
                pairs = [tuple(range(min(2, max(len(rttm_spk), 2))))]
                clus_digits, rttm_digits = None, list(range(len(rttm_spk)))
            for pair in pairs:
                for c, v in zip(cols, (it["audio_file"], it["duration"], it["rttm_file"], it["offset"], pair, sess, clus_digits, rttm_digits)):
                    c.append(v)
        super().__init__(*cols, *args, **kwargs)


def _parse_diar_item(line: str, manifest_file: str) -> Dict[str, Any]:
    item = json.loads(line)
    af = item.get("audio_filename", item.get("audio_filepath"))
    if af is None:
        raise ValueError(f"manifest {manifest_file}: an entry has no audio file key")
    rf = item.get("rttm_filename", item.get("rttm_filepath", item.get("rttm_file")))
    return dict(audio_file=get_full_path(af, manifest_file), rttm_file=get_full_path(rf, manifest_file) if rf else None, duration=item.get("duration"),
                offset=item.get("offset"), uniq_id=item.get("uniq_id"), num_speakers=item.get("num_speakers"))


class EndtoEndDiarizationLabel(_Collection):
    OUTPUT_TYPE = collections.namedtuple("DiarizationLabelEntity", "audio_file uniq_id duration rttm_file offset")

    def __init__(self, audio_files, uniq_ids, durations, rttm_files, offsets, max_number=None, do_sort_by_duration: bool = False, index_by_file_id: bool = False):
        self.mapping = {}
        data = []
        for vals in zip(audio_files, uniq_ids, durations, rttm_files, offsets):
            data.append(self.OUTPUT_TYPE(*vals))
            if index_by_file_id:
                self.mapping[os.path.splitext(os.path.basename(vals[0]))[0]] = len(data) - 1
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration and not index_by_file_id:
            data.sort(key=lambda e: e.duration)
        super().__init__(data)


class EndtoEndDiarizationSpeechLabel(EndtoEndDiarizationLabel):
    """Sessions for end-to-end diarization; the unique id is the manifest's ``uniq_id`` or the audio file stem (with the offset and
    duration appended in milliseconds when a session is a segment of a longer file)."""

    def __init__(self, manifests_files, round_digits: int = 2, *args, **kwargs):
        cols = [[] for _ in range(5)]
        for it in item_iter(manifests_files, parse_func=_parse_diar_item):
            uid = it["uniq_id"] or os.path.splitext(os.path.basename(it["audio_file"]))[0]
            if not it["uniq_id"] and it["offset"]:
                uid = f"{uid}_{int(round(it['offset'], round_digits) * 1000)}_{int(round(it['duration'] or 0, round_digits) * 1000)}"
            for c, v in zip(cols, (it["audio_file"], uid, it["duration"], it["rttm_file"], it["offset"])):
                c.append(v)
        super().__init__(*cols, *args, **kwargs)


# ------------------------------------------------------------------------------------------------------- multi-signal audio
class Audio(_Collection):
    OUTPUT_TYPE = collections.namedtuple("Audio", "audio_files duration offset text")

    def __init__(self, audio_files_list: List[Dict[str, Any]], duration_list, offset_list, text_list, min_duration=None, max_duration=None,
                 max_number=None, do_sort_by_duration: bool = False):
        data = []
        for af, dur, off, text in zip(audio_files_list, duration_list, offset_list, text_list):
            if (min_duration is not None and dur < min_duration) or (max_duration is not None and dur > max_duration):
                continue
            data.append(self.OUTPUT_TYPE(af, dur, off, text))
            if max_number is not None and len(data) == max_number:
                break
        if do_sort_by_duration:
            data.sort(key=lambda e: e.duration)
        super().__init__(data)


class AudioCollection(Audio):
    """Entries with several named audio signals: ``audio_to_manifest_key`` maps a signal name to the manifest key (or a comma-separated
    list of keys, or a list) that holds its file(s), e.g. ``{'input_signal': 'noisy_filepath', 'target_signal': 'clean_filepath'}``."""

    def __init__(self, manifest_files, audio_to_manifest_key: Dict[str, Union[str, List[str]]], *args, **kwargs):
        keys = {a: (k.split(",") if isinstance(k, str) and "," in k else k) for a, k in audio_to_manifest_key.items()}
        afs, durs, offs, texts = [], [], [], []
        if isinstance(manifest_files, str):
            manifest_files = manifest_files.split(",")
        for m in manifest_files:
            with open(m, encoding="utf-8") as f:
                for line in f:
                    if not line.strip():
                        continue
                    item = json.loads(line)
                    files = {}
                    for name, key in keys.items():
                        if isinstance(key, (list, tuple)):
                            vals = [item[k] for k in key]
                            files[name] = get_full_path([v for x in vals for v in (x if isinstance(x, list) else [x])], m)
                        else:
                            if key not in item:
                                raise KeyError(f"manifest {m}: key '{key}' for signal '{name}' is missing")
                            files[name] = get_full_path(item[key], m)
                    afs.append(files); durs.append(item["duration"]); offs.append(item.get("offset", 0.0)); texts.append(item.get("text", ""))
        super().__init__(afs, durs, offs, texts, *args, **kwargs)

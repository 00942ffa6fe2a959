"""Diarization joined with recognition, offline: words with timestamps from an ASR model are given to speakers from diarization
output, optionally re-assigned around speaker changes with a language-model score, grouped into sentences, written in several
formats and scored (DER, cpWER, word-level diarization error rate).  Plus the interval / RTTM / label helpers the speaker tools share.

References: ``asr/parts/utils/diarization_utils.py`` (``OfflineDiarWithASR``, session dictionaries, CTM / text / Audacity writers,
SegLST reading and chunking), ``asr/parts/utils/speaker_utils.py`` (label / RTTM conversion, interval merging, ``audio_rttm_map``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from ..utils.diar_metrics import cp_wer, diarization_error_rate, read_rttm
from ..utils.metrics import edit_distance

__all__ = ["OfflineDiarWithASR", "audio_rttm_map", "chunk_seglst", "get_overlap_range", "get_sub_range_list", "get_uniqname_from_filepath", "is_overlap",
           "labels_to_rttmfile", "merge_float_intervals", "read_seglst", "rttm_to_labels", "word_diarization_error_rate"]


# ------------------------------------------------------------------------------------------------ labels, RTTM, intervals
def get_uniqname_from_filepath(filepath: str) -> str:
    return os.path.splitext(os.path.basename(filepath))[0]


def rttm_to_labels(rttm_filename: str) -> List[str]:
    """``"start end speaker"`` strings, the form the diarizers exchange."""
    return [f"{a:.3f} {b:.3f} {s}" for a, b, s in read_rttm(rttm_filename)]


def labels_to_rttmfile(labels: Sequence[str], uniq_id: str, out_rttm_dir: str) -> str:
    os.makedirs(out_rttm_dir, exist_ok=True)
    path = os.path.join(out_rttm_dir, uniq_id + ".rttm")
    with open(path, "w", encoding="utf-8") as f:
        for l in labels:
            a, b, s = l.split()
            f.write(f"SPEAKER {uniq_id} 1 {float(a):.3f} {float(b) - float(a):.3f} <NA> <NA> {s} <NA> <NA>\n")
    return path


def audio_rttm_map(manifest: str, attach_dur: bool = False) -> Dict[str, dict]:
    """``{unique id: manifest entry}``; ids are the audio file stems (with offset and duration appended when ``attach_dur`` so that
    several windows of one file stay distinct).  Duplicate ids are an error."""
    out: Dict[str, dict] = {}
    for line in open(manifest, encoding="utf-8"):
        if not line.strip():
            continue
        e = json.loads(line)
        uid = get_uniqname_from_filepath(e["audio_filepath"])
        if attach_dur and e.get("duration") is not None:
            uid = f"{uid}_{int(round(float(e.get('offset', 0) or 0) * 1000))}_{int(round(float(e['duration']) * 1000))}"
        if uid in out:
            raise KeyError(f"file {e['audio_filepath']} is listed twice in {manifest}")
        out[uid] = e
    return out


def is_overlap(a: Sequence[float], b: Sequence[float]) -> bool:
    return a[1] > b[0] and b[1] > a[0]


def get_overlap_range(a: Sequence[float], b: Sequence[float]) -> List[float]:
    if not is_overlap(a, b):
        raise ValueError("the ranges do not overlap")
    return [max(a[0], b[0]), min(a[1], b[1])]


def merge_float_intervals(ranges: Sequence[Sequence[float]], decimals: int = 5, margin: int = 2) -> List[List[float]]:
    """Union of intervals; intervals closer than ``margin`` units of the last kept decimal are joined (rounding noise)."""
    if not ranges:
        return []
    tol = margin * 10 ** (-decimals)
    rs = sorted([round(float(a), decimals), round(float(b), decimals)] for a, b in ranges)
    out = [rs[0]]
    for a, b in rs[1:]:
        if a <= out[-1][1] + tol:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return out


def get_sub_range_list(target_range: Sequence[float], source_range_list: Sequence[Sequence[float]]) -> List[List[float]]:
    """The parts of the source ranges that lie inside ``target_range``."""
    return [get_overlap_range(target_range, r) for r in source_range_list if is_overlap(target_range, r)]


def read_seglst(path: str, round_digits: int = 3, sort_by_start_time: bool = True) -> List[Dict[str, Any]]:
    rows = json.load(open(path, encoding="utf-8"))
    for r in rows:
        r["start_time"], r["end_time"] = round(float(r["start_time"]), round_digits), round(float(r["end_time"]), round_digits)
    return sorted(rows, key=lambda r: r["start_time"]) if sort_by_start_time else rows


def chunk_seglst(seglst: Sequence[Dict[str, Any]], chunk_size: float = 10.0) -> List[List[Dict[str, Any]]]:
    """Segments grouped into consecutive windows of ``chunk_size`` seconds by their start time; a segment that crosses a window
    boundary is split there and its words are divided in proportion to time."""
    if not seglst:
        return []
    end = max(s["end_time"] for s in seglst)
    n = int(end // chunk_size) + 1
    out: List[List[Dict[str, Any]]] = [[] for _ in range(n)]
    for s in seglst:
        words = s["words"].split()
        a, b = s["start_time"], s["end_time"]
        k0, k1 = int(a // chunk_size), int(min(b, end - 1e-9) // chunk_size)
        if k0 == k1 or not words:
            out[k0].append(dict(s))
            continue
        used = 0
        for k in range(k0, k1 + 1):
            lo, hi = max(a, k * chunk_size), min(b, (k + 1) * chunk_size)
            share = (hi - lo) / max(b - a, 1e-9)
            cnt = len(words) - used if k == k1 else int(round(share * len(words)))
            part = words[used: used + cnt]
            used += cnt
            if part:
                out[k].append(dict(s, start_time=round(lo, 3), end_time=round(hi, 3), words=" ".join(part)))
    return out


# ------------------------------------------------------------------------------------------------ word-level diarization error
def word_diarization_error_rate(hyp_words: Sequence[Tuple[str, str]], ref_words: Sequence[Tuple[str, str]], mapping: Optional[Dict[str, str]] = None) -> float:
    """``(word, speaker)`` sequences in time order.  Words are aligned by edit distance; among aligned word pairs (correct or
    substituted) the share whose speaker differs after mapping hypothesis speakers to reference speakers (majority vote when
    ``mapping`` is not given)."""
    h, r = [w for w, _ in hyp_words], [w for w, _ in ref_words]
    n, m = len(h), len(r)
    d = [[0] * (m + 1) for _ in range(n + 1)]
    for i in range(n + 1):
        d[i][0] = i
    for j in range(m + 1):
        d[0][j] = j
    for i in range(1, n + 1):
        for j in range(1, m + 1):
            d[i][j] = min(d[i - 1][j] + 1, d[i][j - 1] + 1, d[i - 1][j - 1] + (h[i - 1] != r[j - 1]))
    pairs, i, j = [], n, m
    while i > 0 and j > 0:
        if d[i][j] == d[i - 1][j - 1] + (h[i - 1] != r[j - 1]):
            pairs.append((i - 1, j - 1))
            i, j = i - 1, j - 1
        elif d[i][j] == d[i - 1][j] + 1:
            i -= 1
        else:
            j -= 1
    if not pairs:
        return 0.0
    if mapping is None:
        votes: Dict[str, Dict[str, int]] = {}
        for a, b in pairs:
            votes.setdefault(hyp_words[a][1], {}).setdefault(ref_words[b][1], 0)
            votes[hyp_words[a][1]][ref_words[b][1]] += 1
        mapping = {hs: max(v, key=v.get) for hs, v in votes.items()}
    wrong = sum(mapping.get(hyp_words[a][1], hyp_words[a][1]) != ref_words[b][1] for a, b in pairs)
    return wrong / len(pairs)


# ------------------------------------------------------------------------------------------------ the pipeline
class OfflineDiarWithASR:
    """``word_ts``: ``{uid: [{"word", "start_time", "end_time"}, ...]}``; ``diar_labels``: ``{uid: ["start end speaker", ...]}``.

    ``word_anchor``: which point of a word decides its speaker ("start", "mid", "end").  ``realigning_lm(words) -> log-probability``
    enables re-assignment around speaker changes: for every change point the boundary may move up to ``max_shift`` words either
    way, and the position where the two sides' LM scores sum highest wins (a speaker change inside a fluent phrase is unlikely)."""

    def __init__(self, word_anchor: str = "mid", max_gap_in_sentence: float = 1.5, realigning_lm: Optional[Callable[[List[str]], float]] = None,
                 max_shift: int = 3, min_number_of_words: int = 3):
        if word_anchor not in ("start", "mid", "end"):
            raise ValueError("word_anchor must be 'start', 'mid' or 'end'")
        self.anchor, self.max_gap, self.lm, self.max_shift, self.min_words = word_anchor, max_gap_in_sentence, realigning_lm, max_shift, min_number_of_words

    # .............................................................. speaker assignment
    def _anchor(self, w) -> float:
        return {"start": w["start_time"], "end": w["end_time"], "mid": 0.5 * (w["start_time"] + w["end_time"])}[self.anchor]

    def assign_speakers(self, words: Sequence[Dict[str, Any]], labels: Sequence[str]) -> List[Dict[str, Any]]:
        segs = [(float(a), float(b), s) for a, b, s in (l.split() for l in labels)]
        out = []
        for w in words:
            t = self._anchor(w)
            inside = [s for s in segs if s[0] <= t < s[1]]
            if inside:
                spk = max(inside, key=lambda s: min(s[1], w["end_time"]) - max(s[0], w["start_time"]))[2]
            elif segs:
                spk = min(segs, key=lambda s: min(abs(t - s[0]), abs(t - s[1])))[2]
            else:
                spk = "speaker_0"
            out.append(dict(w, speaker=spk))
        return self.realign(out) if self.lm is not None else out

    def realign(self, words: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        if len(words) < self.min_words:
            return words
        words = [dict(w) for w in words]
        i = 1
        while i < len(words):
            if words[i]["speaker"] == words[i - 1]["speaker"]:
                i += 1
                continue
            left_spk, right_spk = words[i - 1]["speaker"], words[i]["speaker"]
            lo = i
            while lo > 0 and words[lo - 1]["speaker"] == left_spk:
                lo -= 1
            hi = i
            while hi < len(words) and words[hi]["speaker"] == right_spk:
                hi += 1
            best, best_score = i, None
            for c in range(max(lo + 1, i - self.max_shift), min(hi - 1, i + self.max_shift) + 1):
                score = self.lm([w["word"] for w in words[lo:c]]) + self.lm([w["word"] for w in words[c:hi]])
                if best_score is None or score > best_score + 1e-9:
                    best, best_score = c, score
            for k in range(lo, hi):
                words[k]["speaker"] = left_spk if k < best else right_spk
            i = hi
        return words

    # .............................................................. sentences and outputs
    def sentences(self, words: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
        out: List[Dict[str, Any]] = []
        for w in words:
            if out and out[-1]["speaker"] == w["speaker"] and w["start_time"] - out[-1]["end_time"] <= self.max_gap:
                out[-1]["text"] += " " + w["word"]
                out[-1]["end_time"] = w["end_time"]
            else:
                out.append({"speaker": w["speaker"], "start_time": w["start_time"], "end_time": w["end_time"], "text": w["word"]})
        return out

    def get_transcript_with_speaker_labels(self, diar_labels: Dict[str, Sequence[str]], word_ts: Dict[str, Sequence[Dict[str, Any]]]) -> Dict[str, Dict[str, Any]]:
        res = {}
        for uid, words in word_ts.items():
            tagged = self.assign_speakers(words, diar_labels.get(uid, []))
            sents = self.sentences(tagged)
            res[uid] = {"status": "success", "session_id": uid, "transcription": " ".join(w["word"] for w in tagged),
                        "speaker_count": len({w["speaker"] for w in tagged}), "words": tagged, "sentences": sents}
        return res

    @staticmethod
    def write_outputs(result: Dict[str, Dict[str, Any]], out_dir: str) -> None:
        """Per session: ``.json`` (everything), ``.txt`` (``[mm:ss.xx - mm:ss.xx] speaker: text``), ``.ctm`` (words with speakers) and
        ``.w.label`` (Audacity label track)."""
        os.makedirs(out_dir, exist_ok=True)
        fmt = lambda t: f"{int(t // 60):02d}:{t % 60:05.2f}"  # noqa: E731
        for uid, r in result.items():
            with open(os.path.join(out_dir, uid + ".json"), "w", encoding="utf-8") as f:
                json.dump(r, f, indent=2, ensure_ascii=False)
            with open(os.path.join(out_dir, uid + ".txt"), "w", encoding="utf-8") as f:
                for s in r["sentences"]:
                    f.write(f"[{fmt(s['start_time'])} - {fmt(s['end_time'])}] {s['speaker']}: {s['text']}\n")
            with open(os.path.join(out_dir, uid + ".ctm"), "w", encoding="utf-8") as f:
                for w in r["words"]:
                    f.write(f"{uid} 1 {w['start_time']:.3f} {w['end_time'] - w['start_time']:.3f} {w['word']} NA lex {w['speaker']}\n")
            with open(os.path.join(out_dir, uid + ".w.label"), "w", encoding="utf-8") as f:
                for w in r["words"]:
                    f.write(f"{w['start_time']:.3f}\t{w['end_time']:.3f}\t[{w['speaker']}] {w['word']}\n")

    # .............................................................. evaluation
    @staticmethod
    def evaluate(result: Dict[str, Dict[str, Any]], ref_rttm: Optional[Dict[str, str]] = None, ref_words: Optional[Dict[str, Sequence[Tuple[str, str]]]] = None,
                 diar_labels: Optional[Dict[str, Sequence[str]]] = None, collar: float = 0.25, ignore_overlap: bool = True) -> Dict[str, Dict[str, float]]:
        """Per session: DER of the diarization labels against reference RTTM, cpWER and word-level diarization error against
        reference ``(word, speaker)`` sequences, and plain WER of the word sequence."""
        out: Dict[str, Dict[str, float]] = {}
        for uid, r in result.items():
            m: Dict[str, float] = {}
            mapping = None
            if ref_rttm and uid in ref_rttm and diar_labels and uid in diar_labels:
                hyp = [(float(a), float(b), s) for a, b, s in (l.split() for l in diar_labels[uid])]
                d = diarization_error_rate(read_rttm(ref_rttm[uid]), hyp, collar=collar, ignore_overlap=ignore_overlap)
                m.update(DER=d["DER"], miss=d["miss"], FA=d["false_alarm"], CER=d["confusion"])
                mapping = d["mapping"]
            if ref_words and uid in ref_words:
                ref = list(ref_words[uid])
                hyp_w = [(w["word"], w["speaker"]) for w in r["words"]]
                by_h: Dict[str, List[str]] = {}
                for w, s in hyp_w:
                    by_h.setdefault(s, []).append(w)
                by_r: Dict[str, List[str]] = {}
                for w, s in ref:
                    by_r.setdefault(s, []).append(w)
                m["cpWER"] = cp_wer([" ".join(v) for v in by_h.values()], [" ".join(v) for v in by_r.values()])[0]
                m["WDER"] = word_diarization_error_rate(hyp_w, ref, mapping if mapping and all(s in mapping for _, s in hyp_w) else None)
                m["WER"] = edit_distance([w for w, _ in hyp_w], [w for w, _ in ref]) / max(1, len(ref))
            out[uid] = m
        return out

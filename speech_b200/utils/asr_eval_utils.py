"""Evaluation and bookkeeping helpers around transcription: reference / hypothesis text cleaning, corpus WER written back into a
manifest, punctuation error rate, latency of simultaneous output (LAAL), merging the hypotheses of consecutive chunks of one
recording, timestamps in seconds, CTM lines and sub-segment manifests.

References: ``asr/parts/utils/eval_utils.py`` (``clean_label``, ``cal_write_wer``, ``compute_laal``; ``PunctuationErrorRate`` in
``asr/metrics``-adjacent utilities), ``asr/parts/utils/chunking_utils.py`` (``merge_parallel_chunks``, ``merge_hypotheses_of_same_audio``),
``asr/parts/utils/manifest_utils.py`` (``get_ctm_line``, ``create_segment_manifest``, ``get_subsegment_dict``), ``asr/parts/utils/timestamp_utils.py``
(``process_timestamp_outputs``).
"""
from __future__ import annotations

import copy
import json
import os
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .metrics import edit_operations, word_error_rate

__all__ = ["PunctuationErrorRate", "cal_write_wer", "clean_label", "compute_laal", "convert_num_to_words", "create_segment_manifest", "get_ctm_line",
           "get_subsegment_dict", "merge_hypotheses_of_same_audio", "merge_parallel_chunks", "process_timestamp_outputs", "remove_punctuations",
           "strip_spaces_before_punctuations"]

_ONES = "zero one two three four five six seven eight nine ten eleven twelve thirteen fourteen fifteen sixteen seventeen eighteen nineteen".split()
_TENS = "twenty thirty forty fifty sixty seventy eighty ninety".split()


def _int_to_words(n: int) -> str:
    if n < 20:
        return _ONES[n]
    if n < 100:
        return _TENS[n // 10 - 2] + ("" if n % 10 == 0 else " " + _ONES[n % 10])
    if n < 1000:
        return _ONES[n // 100] + " hundred" + ("" if n % 100 == 0 else " " + _int_to_words(n % 100))
    for scale, name in ((10 ** 9, "billion"), (10 ** 6, "million"), (1000, "thousand")):
        if n >= scale:
            return _int_to_words(n // scale) + " " + name + ("" if n % scale == 0 else " " + _int_to_words(n % scale))
    return str(n)


def convert_num_to_words(text: str, langid: str = "en") -> str:
    """Spells out integers (English only; other languages are returned unchanged)."""
    if langid != "en":
        return text
    return re.sub(r"\d+", lambda m: _int_to_words(int(m.group(0))) if len(m.group(0)) <= 12 else m.group(0), text)


def strip_spaces_before_punctuations(text: str) -> str:
    return re.sub(r"\s+([.,!?;:])", r"\1", text)


def remove_punctuations(text: str, punctuations: Optional[Sequence[str]] = None) -> str:
    p = "".join(punctuations) if punctuations is not None else "!,.?"
    return re.sub(r"\s+", " ", re.sub(f"[{re.escape(p)}]", " ", text)).strip()


def clean_label(text: str, num_to_words: bool = True, langid: str = "en") -> str:
    """Lower case, bracketed remarks and punctuation other than apostrophes removed, numbers spelled out."""
    t = text.strip().lower()
    t = re.sub(r"[\[\(\{<].*?[\]\)\}>]", " ", t)
    t = re.sub(r"[^\w\s']", " ", t, flags=re.UNICODE)
    if num_to_words:
        t = convert_num_to_words(t, langid)
    return re.sub(r"\s+", " ", t).strip()


def cal_write_wer(pred_manifest: str, gt_text_attr_name: str = "text", pred_text_attr_name: str = "pred_text", clean_groundtruth_text: bool = False,
                  langid: str = "en", use_cer: bool = False, output_filename: Optional[str] = None, ignore_capitalization: bool = False,
                  ignore_punctuation: bool = False, punctuations: Optional[Sequence[str]] = None) -> Tuple[str, float, float, int, Dict[str, float]]:
    """Reads a manifest with references and predictions, adds per-sample ``wer`` / ``tokens`` / ``ins_rate`` / ``del_rate`` /
    ``sub_rate`` and writes it next to the input (``_wer`` / ``_cer`` suffix).  Returns ``(output path, total WER, total tokens,
    number of samples, {"ins","del","sub"} rates)``."""
    rows = [json.loads(l) for l in open(pred_manifest, encoding="utf-8") if l.strip()]
    tot = {"i": 0, "d": 0, "s": 0, "n": 0}
    for r in rows:
        if pred_text_attr_name not in r:
            raise ValueError(f"{pred_manifest} has lines without {pred_text_attr_name!r}")
        ref, hyp = r[gt_text_attr_name], r[pred_text_attr_name]
        if clean_groundtruth_text:
            ref = clean_label(ref, langid=langid)
        if ignore_punctuation:
            ref, hyp = remove_punctuations(ref, punctuations), remove_punctuations(hyp, punctuations)
        if ignore_capitalization:
            ref, hyp = ref.lower(), hyp.lower()
        a, b = (list(hyp), list(ref)) if use_cer else (hyp.split(), ref.split())
        ins, dele, sub = edit_operations(a, b)
        n = max(1, len(b))
        r.update({"cer" if use_cer else "wer": (ins + dele + sub) / n, "tokens": len(b), "ins_rate": ins / n, "del_rate": dele / n, "sub_rate": sub / n})
        tot["i"], tot["d"], tot["s"], tot["n"] = tot["i"] + ins, tot["d"] + dele, tot["s"] + sub, tot["n"] + len(b)
    out = output_filename or (os.path.splitext(pred_manifest)[0] + ("_cer" if use_cer else "_wer") + ".json")
    with open(out, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    n = max(1, tot["n"])
    return out, (tot["i"] + tot["d"] + tot["s"]) / n, tot["n"], len(rows), {"ins": tot["i"] / n, "del": tot["d"] / n, "sub": tot["s"] / n}


class PunctuationErrorRate:
    """Compares the punctuation marks that follow aligned words of reference and hypothesis: a mark is correct when the same mark
    follows the matching word; otherwise it counts as substituted, deleted (missing in the hypothesis) or inserted.  Words are
    aligned by edit distance on the punctuation-free text, so recognition errors do not shift the comparison."""

    def __init__(self, punctuation_marks: Sequence[str] = (".", ",", "?")):
        self.marks = list(punctuation_marks)
        self.reset()

    def reset(self):
        self.c = {m: {"correct": 0, "sub": 0, "del": 0, "ins": 0} for m in self.marks}

    def _split(self, text: str) -> List[Tuple[str, str]]:
        out = []
        for w in text.split():
            mark = ""
            while w and w[-1] in self.marks:
                mark, w = w[-1], w[:-1]
            if w:
                out.append((w.lower(), mark))
            elif out and mark:
                out[-1] = (out[-1][0], mark)
        return out

    @staticmethod
    def _align(a: List[str], b: List[str]) -> List[Tuple[Optional[int], Optional[int]]]:
        n, m = len(a), len(b)
        d = [[0] * (m + 1) for _ in range(n + 1)]
        for i in range(n + 1):
            d[i][0] = i
        for j in range(m + 1):
            d[0][j] = j
        for i in range(1, n + 1):
            for j in range(1, m + 1):
                d[i][j] = min(d[i - 1][j] + 1, d[i][j - 1] + 1, d[i - 1][j - 1] + (a[i - 1] != b[j - 1]))
        pairs, i, j = [], n, m
        while i > 0 or j > 0:
            if i > 0 and j > 0 and d[i][j] == d[i - 1][j - 1] + (a[i - 1] != b[j - 1]):
                pairs.append((i - 1, j - 1))
                i, j = i - 1, j - 1
            elif i > 0 and d[i][j] == d[i - 1][j] + 1:
                pairs.append((i - 1, None))
                i -= 1
            else:
                pairs.append((None, j - 1))
                j -= 1
        return pairs[::-1]

    def update(self, hypotheses: Sequence[str], references: Sequence[str]):
        for hyp, ref in zip(hypotheses, references):
            h, r = self._split(hyp), self._split(ref)
            for hi, ri in self._align([w for w, _ in h], [w for w, _ in r]):
                hm = h[hi][1] if hi is not None else ""
                rm = r[ri][1] if ri is not None else ""
                if rm and hm == rm:
                    self.c[rm]["correct"] += 1
                elif rm and hm:
                    self.c[rm]["sub"] += 1
                elif rm:
                    self.c[rm]["del"] += 1
                elif hm:
                    self.c[hm]["ins"] += 1

    def compute(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        tc = ts = td = ti = 0
        for m, c in self.c.items():
            denom = max(1, c["correct"] + c["sub"] + c["del"] + c["ins"])
            out[m] = {"correct_rate": c["correct"] / denom, "sub_rate": c["sub"] / denom, "del_rate": c["del"] / denom, "ins_rate": c["ins"] / denom,
                      "per": (c["sub"] + c["del"] + c["ins"]) / denom}
            tc, ts, td, ti = tc + c["correct"], ts + c["sub"], td + c["del"], ti + c["ins"]
        out["punct_er"] = (ts + td + ti) / max(1, tc + ts + td + ti)
        return out


def compute_laal(delays: Sequence[float], source_length: float, target_length: int) -> float:
    """Length-adaptive average lagging (seconds or frames, as ``delays``): ``delays[i]`` is how much source had been read when
    target token i was emitted.  Lagging is averaged up to the first token emitted after the whole source was read, against an
    ideal translator that emits at the rate ``max(len(delays), target_length) / source_length``."""
    if not len(delays) or (delays[0] > source_length):
        return float(delays[0]) if len(delays) else 0.0
    gamma = max(len(delays), target_length) / source_length
    lag, tau = 0.0, 0
    for t, d in enumerate(delays):
        lag += d - t / gamma
        tau = t + 1
        if d >= source_length:
            break
    return lag / tau


# ------------------------------------------------------------------------------------------------ chunk merging
def merge_parallel_chunks(hypotheses: Sequence, encoded_len: Sequence[int], decode_tokens_to_str=None) -> Any:
    """Hypotheses of consecutive, non-overlapping chunks of ONE recording -> one hypothesis: token sequences are concatenated,
    per-token frame indices are shifted by the number of encoder frames of the chunks before, confidences are joined."""
    if not hypotheses:
        return None
    merged = copy.copy(hypotheses[0])
    ys, ts, fc, tc, wc = [], [], [], [], []
    offset = 0
    score = 0.0
    for h, n in zip(hypotheses, encoded_len):
        y = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
        t = h.timestamp if not isinstance(h.timestamp, dict) else h.timestamp.get("timestep", [])
        t = t.tolist() if torch.is_tensor(t) else list(t or [])
        ys += y
        ts += [int(v) + offset for v in t]
        for acc, v in ((fc, h.frame_confidence), (tc, h.token_confidence), (wc, h.word_confidence)):
            if v is not None:
                acc += list(v)
        score += float(h.score or 0.0)
        offset += int(n)
    merged.y_sequence, merged.timestamp, merged.score, merged.length = torch.tensor(ys, dtype=torch.long), ts, score, offset
    merged.frame_confidence, merged.token_confidence, merged.word_confidence = (fc or None), (tc or None), (wc or None)
    if decode_tokens_to_str is not None:
        merged.text = decode_tokens_to_str(ys)
    else:
        merged.text = " ".join((h.text or "").strip() for h in hypotheses if (h.text or "").strip())
    return merged


def merge_hypotheses_of_same_audio(items: Sequence[Tuple[str, Any, int]], decode_tokens_to_str=None) -> Dict[str, Any]:
    """``items``: ``(chunk id, hypothesis, encoder frames)`` where chunk ids look like ``<recording>-<chunk index>`` (or
    ``<recording>_cut<index>``); chunks are grouped per recording, ordered by index and merged."""
    groups: Dict[str, List[Tuple[int, Any, int]]] = {}
    for cid, h, n in items:
        m = re.match(r"^(.*?)(?:[-_](?:cut|chunk)?(\d+))$", cid)
        rec, k = (m.group(1), int(m.group(2))) if m else (cid, 0)
        groups.setdefault(rec, []).append((k, h, n))
    return {rec: merge_parallel_chunks([h for _, h, _ in sorted(g, key=lambda x: x[0])], [n for _, _, n in sorted(g, key=lambda x: x[0])], decode_tokens_to_str)
            for rec, g in groups.items()}


def process_timestamp_outputs(hypotheses: Sequence, subsampling_factor: int = 1, window_stride: float = 0.01) -> Sequence:
    """Adds ``start`` / ``end`` in seconds beside the frame offsets of the word / segment / char timestamp dictionaries."""
    unit = subsampling_factor * window_stride
    for h in hypotheses:
        ts = getattr(h, "timestamp", None)
        if not isinstance(ts, dict):
            continue
        for level in ("char", "word", "segment"):
            for e in ts.get(level, []) or []:
                if "start_offset" in e:
                    e["start"], e["end"] = round(e["start_offset"] * unit, 4), round(e["end_offset"] * unit, 4)
    return hypotheses


# ------------------------------------------------------------------------------------------------ CTM / segments
def get_ctm_line(source: str, channel: int, start_time: float, duration: float, token: str, conf: Optional[float] = None, type_of_token: str = "lex",
                 speaker: Optional[str] = None, output_precision: int = 3) -> str:
    """``<source> <channel> <start> <duration> <token> <conf> <type> <speaker>`` with ``NA`` for missing fields."""
    if duration < 0 or start_time < 0:
        raise ValueError("start_time and duration must be non-negative")
    if conf is not None and not 0.0 <= conf <= 1.0:
        raise ValueError(f"confidence must be in [0, 1], got {conf}")
    f = lambda v: f"{v:.{output_precision}f}"  # noqa: E731
    return f"{source} {channel} {f(start_time)} {f(duration)} {token} {'NA' if conf is None else f(conf)} {type_of_token} {speaker or 'NA'}\n"


def create_segment_manifest(input_manifest: str, output_manifest: str, window: float, shift: float, step_count: int = 1, min_duration: float = 0.1) -> int:
    """Recordings with RTTM references -> one manifest line per sliding-window sub-segment of every speech region, labelled with
    the speaker (for speaker-embedding training on diarization corpora)."""
    from .diar_metrics import read_rttm

    n = 0
    with open(output_manifest, "w", encoding="utf-8") as f:
        for line in open(input_manifest, encoding="utf-8"):
            if not line.strip():
                continue
            e = json.loads(line)
            for a, b, spk in read_rttm(e["rttm_filepath"]):
                k = 0
                for s, d in get_subsegments(a, b - a, window, shift):
                    if d < min_duration or (k % step_count):
                        k += 1
                        continue
                    f.write(json.dumps({"audio_filepath": e["audio_filepath"], "offset": round(s, 3), "duration": round(d, 3), "label": spk,
                                        "uniq_id": os.path.splitext(os.path.basename(e["audio_filepath"]))[0]}) + "\n")
                    n += 1
                    k += 1
    return n


def get_subsegments(offset: float, duration: float, window: float, shift: float) -> List[Tuple[float, float]]:
    out, s = [], offset
    end = offset + duration
    while s + window < end:
        out.append((s, window))
        s += shift
    if end - s > 0:
        out.append((s, end - s))
    return out


def get_subsegment_dict(subsegments_manifest_file: str, window: float, shift: float, deci: int = 3) -> Dict[str, dict]:
    """``{recording id: {"ts": [[start, end], ...], "json_dic": [lines]}}`` from a sub-segment manifest."""
    out: Dict[str, dict] = {}
    for line in open(subsegments_manifest_file, encoding="utf-8"):
        if not line.strip():
            continue
        d = json.loads(line)
        uid = d.get("uniq_id") or os.path.splitext(os.path.basename(d["audio_filepath"]))[0]
        e = out.setdefault(uid, {"ts": [], "json_dic": []})
        e["ts"].append([round(d["offset"], deci), round(d["offset"] + d["duration"], deci)])
        e["json_dic"].append(d)
    return out

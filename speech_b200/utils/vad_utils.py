"""Voice-activity post-processing and evaluation: window the audio, smooth overlapping window posteriors into frame posteriors,
binarise with hysteresis and padding, filter short segments / gaps, score against reference segments, tune the thresholds on a
development set, and convert between frame labels, segments and RTTM.

Reference: ``asr/parts/utils/vad_utils.py`` (``prepare_manifest``, ``generate_overlap_vad_seq``, ``binarization``, ``filtering``,
``vad_tune_threshold_on_dev``, ``generate_vad_frame_pred``, frame-VAD label helpers) and the scripts under
``scripts/voice_activity_detection``.  The detection error rate is computed here from interval arithmetic (the reference defers to
an external diarization-metrics package).
"""
from __future__ import annotations

import itertools
import json
import math
import os
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = ["align_labels_to_frames", "binarization", "convert_labels_to_speech_segments", "detection_error_rate", "extract_labels", "filtering",
           "frame_auroc", "generate_overlap_vad_seq", "generate_vad_frame_pred", "generate_vad_segment_table", "get_gap_segments", "merge_overlap_segment",
           "read_rttm_as_segments", "remove_segments", "vad_tune_threshold_on_dev", "write_long_audio_manifest", "write_rttm"]

Segments = torch.Tensor        # [N, 2] start / end seconds


# ------------------------------------------------------------------------------------------------ windows
def write_long_audio_manifest(manifest: str, out_manifest: str, split_duration: float = 400.0, window_length_in_sec: float = 0.63, min_tail: float = 0.0) -> int:
    """Long recordings are cut into pieces of ``split_duration`` seconds (each overlapping the next by one analysis window, so that
    frame posteriors near the cut have their full context); ``offset`` / ``duration`` / ``label`` per piece."""
    n = 0
    with open(out_manifest, "w", encoding="utf-8") as f:
        for line in open(manifest, encoding="utf-8"):
            if not line.strip():
                continue
            e = json.loads(line)
            total, base = float(e["duration"]), float(e.get("offset", 0.0) or 0.0)
            if total <= split_duration:
                f.write(json.dumps(dict(e, offset=base, duration=total, label=e.get("label", "infer"))) + "\n")
                n += 1
                continue
            pos = 0.0
            while pos < total - min_tail:
                last = pos + split_duration >= total
                d = min(split_duration + (0.0 if last else window_length_in_sec), total - pos)
                tag = "single" if (pos == 0.0 and last) else "start" if pos == 0.0 else "end" if last else "next"
                f.write(json.dumps(dict(e, offset=base + pos, duration=d, label=e.get("label", "infer"), stream_status=tag)) + "\n")
                n += 1
                pos += split_duration
    return n


# ------------------------------------------------------------------------------------------------ smoothing
def generate_overlap_vad_seq(window_probs: torch.Tensor, window_length_in_sec: float, shift_length_in_sec: float, frame_unit: float = 0.01,
                             smoothing_method: str = "mean") -> torch.Tensor:
    """``window_probs[k]`` is the speech probability of the window starting at ``k * shift``.  Every ``frame_unit`` frame is
    covered by several windows; its posterior is their mean or median."""
    if smoothing_method not in ("mean", "median"):
        raise ValueError("smoothing_method must be 'mean' or 'median'")
    p = torch.as_tensor(window_probs, dtype=torch.float32)
    win, shift = max(1, int(round(window_length_in_sec / frame_unit))), max(1, int(round(shift_length_in_sec / frame_unit)))
    K = p.numel()
    T = (K - 1) * shift + win
    if smoothing_method == "mean":
        acc, cnt = torch.zeros(T), torch.zeros(T)
        idx = (torch.arange(K)[:, None] * shift + torch.arange(win)[None, :]).reshape(-1)
        acc.index_add_(0, idx, p[:, None].expand(K, win).reshape(-1))
        cnt.index_add_(0, idx, torch.ones(K * win))
        return acc / cnt.clamp(min=1)
    per = -(-win // shift)                                                # windows covering an interior frame
    table = torch.full((T, per), float("nan"))
    fill = torch.zeros(T, dtype=torch.long)
    for k in range(K):
        sl = slice(k * shift, k * shift + win)
        table[torch.arange(sl.start, sl.stop), fill[sl].clamp(max=per - 1)] = p[k]
        fill[sl] += 1
    return torch.nanmedian(table, dim=1).values


# ------------------------------------------------------------------------------------------------ segments
def binarization(sequence: torch.Tensor, per_args: Dict[str, float]) -> Segments:
    """Hysteresis thresholding: speech starts where the posterior rises above ``onset`` and ends where it falls below ``offset``;
    every segment is then widened by ``pad_onset`` / ``pad_offset`` seconds, and overlapping results are merged."""
    onset, offset = per_args.get("onset", 0.5), per_args.get("offset", 0.5)
    pad_on, pad_off, unit = per_args.get("pad_onset", 0.0), per_args.get("pad_offset", 0.0), per_args.get("frame_length_in_sec", 0.01)
    x = torch.as_tensor(sequence, dtype=torch.float32)
    above_on, below_off = (x > onset).tolist(), (x < offset).tolist()
    segs, speech, start = [], False, 0
    for i in range(len(above_on)):
        if not speech and above_on[i]:
            speech, start = True, i
        elif speech and below_off[i]:
            segs.append((max(0.0, start * unit - pad_on), i * unit + pad_off))
            speech = False
    if speech:
        segs.append((max(0.0, start * unit - pad_on), len(above_on) * unit + pad_off))
    return merge_overlap_segment(torch.tensor(segs, dtype=torch.float32).reshape(-1, 2))


def merge_overlap_segment(segments: Segments) -> Segments:
    if segments.numel() == 0:
        return segments.reshape(0, 2)
    s = segments[segments[:, 0].argsort()]
    out = [s[0].tolist()]
    for a, b in s[1:].tolist():
        if a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return torch.tensor(out, dtype=torch.float32)


def remove_segments(segments: Segments, to_remove: Segments) -> Segments:
    """Rows of ``segments`` that appear (exactly) in ``to_remove`` are dropped."""
    if segments.numel() == 0 or to_remove.numel() == 0:
        return segments
    keep = ~(segments[:, None, :] == to_remove[None, :, :]).all(-1).any(-1)
    return segments[keep]


def get_gap_segments(segments: Segments) -> Segments:
    s = segments[segments[:, 0].argsort()]
    return torch.stack([s[:-1, 1], s[1:, 0]], dim=1) if s.shape[0] > 1 else torch.zeros(0, 2)


def filtering(speech_segments: Segments, per_args: Dict[str, float]) -> Segments:
    """Drops speech shorter than ``min_duration_on`` and fills silences shorter than ``min_duration_off``; ``filter_speech_first``
    chooses which of the two happens first (the order matters when a short burst sits between two short gaps)."""
    if speech_segments.numel() == 0:
        return speech_segments.reshape(0, 2)
    min_on, min_off = per_args.get("min_duration_on", 0.0), per_args.get("min_duration_off", 0.0)
    first = bool(per_args.get("filter_speech_first", 1.0))

    def drop_short(s):
        return s[(s[:, 1] - s[:, 0]) >= min_on] if min_on > 0 and s.numel() else s

    def fill_gaps(s):
        if min_off <= 0 or s.shape[0] < 2:
            return s
        gaps = get_gap_segments(s)
        short = gaps[(gaps[:, 1] - gaps[:, 0]) < min_off]
        return merge_overlap_segment(torch.cat([s, short], dim=0)) if short.numel() else s

    s = speech_segments
    s = fill_gaps(drop_short(s)) if first else drop_short(fill_gaps(s))
    return s.reshape(-1, 2)


def generate_vad_segment_table(frame_probs: torch.Tensor, postprocessing_params: Dict[str, float], frame_length_in_sec: float = 0.01) -> Segments:
    p = dict(postprocessing_params, frame_length_in_sec=frame_length_in_sec)
    return filtering(binarization(frame_probs, p), p)


# ------------------------------------------------------------------------------------------------ scoring
def _total(s: Segments) -> float:
    return float((s[:, 1] - s[:, 0]).clamp(min=0).sum()) if s.numel() else 0.0


def _intersection(a: Segments, b: Segments) -> float:
    if a.numel() == 0 or b.numel() == 0:
        return 0.0
    lo = torch.maximum(a[:, None, 0], b[None, :, 0])
    hi = torch.minimum(a[:, None, 1], b[None, :, 1])
    return float((hi - lo).clamp(min=0).sum())


def detection_error_rate(reference: Segments, hypothesis: Segments) -> Dict[str, float]:
    """Detection error rate = (missed speech + false alarm) / reference speech, with its two parts, from merged segment lists."""
    r, h = merge_overlap_segment(reference.reshape(-1, 2)), merge_overlap_segment(hypothesis.reshape(-1, 2))
    inter = _intersection(r, h)
    ref, hyp = _total(r), _total(h)
    miss, fa = ref - inter, hyp - inter
    return {"DetER": 100.0 * (miss + fa) / max(ref, 1e-9), "miss": 100.0 * miss / max(ref, 1e-9), "FA": 100.0 * fa / max(ref, 1e-9), "total": ref}


def vad_tune_threshold_on_dev(params: Dict[str, Sequence[float]], frame_probs: Dict[str, torch.Tensor], references: Dict[str, Segments],
                              frame_length_in_sec: float = 0.01, focus_metric: str = "DetER") -> Tuple[Dict[str, float], Dict[str, float], List[Tuple[Dict[str, float], Dict[str, float]]]]:
    """Grid search: every combination of the listed values is applied to all recordings, errors are pooled by duration, and the
    combination with the lowest ``focus_metric`` wins.  Returns ``(best parameters, its scores, all trials)``."""
    keys = list(params)
    for k in keys:
        if k not in ("onset", "offset", "pad_onset", "pad_offset", "min_duration_on", "min_duration_off", "filter_speech_first"):
            raise ValueError(f"unknown post-processing parameter {k!r}")
    trials = []
    for combo in itertools.product(*[list(params[k]) for k in keys]):
        p = dict(zip(keys, [float(c) for c in combo]))
        if "offset" not in p and "onset" in p:
            p["offset"] = p["onset"]
        miss = fa = tot = 0.0
        for name, probs in frame_probs.items():
            seg = generate_vad_segment_table(probs, p, frame_length_in_sec)
            sc = detection_error_rate(references[name], seg)
            miss, fa, tot = miss + sc["miss"] * sc["total"], fa + sc["FA"] * sc["total"], tot + sc["total"]
        score = {"DetER": (miss + fa) / max(tot, 1e-9), "miss": miss / max(tot, 1e-9), "FA": fa / max(tot, 1e-9)}
        trials.append((p, score))
    best = min(trials, key=lambda t: t[1][focus_metric])
    return best[0], best[1], trials


def frame_auroc(probs: torch.Tensor, labels: torch.Tensor) -> float:
    """Area under the ROC curve of frame posteriors against 0 / 1 labels (rank statistic; ties get their average rank)."""
    p, y = torch.as_tensor(probs, dtype=torch.float64).reshape(-1), torch.as_tensor(labels).reshape(-1).bool()
    n1, n0 = int(y.sum()), int((~y).sum())
    if n1 == 0 or n0 == 0:
        return float("nan")
    order = p.argsort()
    ranks = torch.empty_like(p)
    ranks[order] = torch.arange(1, p.numel() + 1, dtype=torch.float64)
    _, inv, cnt = torch.unique(p, return_inverse=True, return_counts=True)
    sums = torch.zeros(cnt.numel(), dtype=torch.float64).index_add_(0, inv, ranks)
    ranks = (sums / cnt)[inv]
    return float((ranks[y].sum() - n1 * (n1 + 1) / 2) / (n1 * n0))


# ------------------------------------------------------------------------------------------------ labels, RTTM
def extract_labels(path_or_text: str, time: Sequence[float]) -> List[int]:
    """0 / 1 label at each time stamp from an RTTM file (speech inside any segment) or from a string of space-separated labels."""
    if os.path.exists(path_or_text):
        seg = read_rttm_as_segments(path_or_text)
        t = torch.as_tensor(list(time), dtype=torch.float32)
        return ((t[:, None] >= seg[None, :, 0]) & (t[:, None] < seg[None, :, 1])).any(-1).long().tolist() if seg.numel() else [0] * len(t)
    return [int(x) for x in path_or_text.split()]


def align_labels_to_frames(probs: Sequence[float], labels: Sequence[int], threshold: float = 0.2) -> List[int]:
    """Stretches or shrinks a label sequence by an integer ratio to the length of ``probs`` (labels and posteriors often come at
    different frame rates), then pads with the last label / trims; raises when the lengths disagree by more than ``threshold``."""
    n, m = len(probs), len(labels)
    if m == 0 or n == 0:
        return [0] * n
    labels = list(labels)
    if m < n:
        r = int(round(n / m))
        out = [l for l in labels for _ in range(r)]
    else:
        r = int(round(m / n))
        out = [int(round(sum(labels[i:i + r]) / max(1, len(labels[i:i + r])) + 1e-9)) for i in range(0, m, r)] if r > 1 else labels
    if abs(len(out) - n) / n > threshold:
        raise ValueError(f"label length {m} cannot be aligned to {n} frames")
    return (out + [out[-1]] * (n - len(out)))[:n]


def convert_labels_to_speech_segments(labels: Sequence[int], frame_length_in_sec: float = 0.01) -> List[Tuple[float, float]]:
    segs, start = [], None
    for i, l in enumerate(list(labels) + [0]):
        if l and start is None:
            start = i
        elif not l and start is not None:
            segs.append((start * frame_length_in_sec, i * frame_length_in_sec))
            start = None
    return segs


def read_rttm_as_segments(path: str) -> Segments:
    rows = []
    for line in open(path, encoding="utf-8"):
        f = line.split()
        if len(f) >= 5 and f[0] == "SPEAKER":
            rows.append((float(f[3]), float(f[3]) + float(f[4])))
    return merge_overlap_segment(torch.tensor(rows, dtype=torch.float32).reshape(-1, 2))


def write_rttm(path: str, segments: Segments, file_id: str, speaker: str = "speech"):
    with open(path, "w", encoding="utf-8") as f:
        for a, b in segments.tolist():
            f.write(f"SPEAKER {file_id} 1 {a:.3f} {b - a:.3f} <NA> <NA> {speaker} <NA> <NA>\n")


# ------------------------------------------------------------------------------------------------ inference
@torch.no_grad()
def generate_vad_frame_pred(vad_model, audio: torch.Tensor, sample_rate: int = 16000, window_length_in_sec: float = 0.63, shift_length_in_sec: float = 0.08,
                            batch_size: int = 256, speech_class: int = 1, smoothing_method: str = "mean", frame_unit: float = 0.01) -> torch.Tensor:
    """Window-classification VAD over one recording: the model scores windows of ``window_length_in_sec`` every
    ``shift_length_in_sec`` (``vad_model(input_signal, input_signal_length) -> logits [B, C]``, or ``[B, T, C]`` for frame
    models, which are averaged over the window); the window scores are smoothed into frame posteriors."""
    x = audio.reshape(-1).float()
    win, shift = int(round(window_length_in_sec * sample_rate)), int(round(shift_length_in_sec * sample_rate))
    x = torch.nn.functional.pad(x, (win // 2, win // 2))
    frames = x.unfold(0, win, shift)
    dev = next(vad_model.parameters()).device if hasattr(vad_model, "parameters") else torch.device("cpu")
    out = []
    for s in range(0, frames.shape[0], batch_size):
        b = frames[s:s + batch_size].to(dev)
        logits = vad_model(input_signal=b, input_signal_length=torch.full((b.shape[0],), win, device=dev))
        logits = logits[0] if isinstance(logits, (tuple, list)) else logits
        if logits.dim() == 3:
            logits = logits.mean(dim=1)
        out.append(torch.softmax(logits.float(), dim=-1)[:, speech_class].cpu())
    return generate_overlap_vad_seq(torch.cat(out), window_length_in_sec, shift_length_in_sec, frame_unit, smoothing_method)

"""Diarization and multi-speaker ASR metrics, computed here from interval arithmetic and assignment problems (the reference defers
DER to an external metrics package and to the NIST ``md-eval`` script).

* ``diarization_error_rate`` — DER with a forgiveness collar around reference boundaries, with or without overlapped speech,
  under the speaker mapping that maximises the matched time (Hungarian assignment); returns miss / false alarm / confusion and
  the mapping.  ``score_labels`` pools it over recordings.
* ``cp_wer`` — concatenated minimum-permutation word error rate: the hypothesis speakers are permuted (assignment on the
  per-pair edit distances, extra speakers count in full) so that the total number of word errors is smallest.
* ``MultiBinaryAccuracy`` — frame-level accuracy / precision / recall / F1 of multi-label speaker activity.
* ``long_form_clustering`` — clustering of very long recordings in windows with a merge of the window clusters.
* ``sot_speaker_alignment`` — splits a serialised-output transcript (speaker-change tokens) into per-speaker texts and aligns
  them to reference speakers.

References: ``asr/metrics/der.py``, ``asr/metrics/cpwer.py``, ``asr/metrics/multi_binary_acc.py``, ``asr/parts/utils/longform_clustering.py``,
``asr/parts/utils/sot_speaker_alignment.py``.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
from scipy.optimize import linear_sum_assignment

from .metrics import edit_distance

__all__ = ["MultiBinaryAccuracy", "cp_wer", "diarization_error_rate", "long_form_clustering", "read_rttm", "score_labels", "sot_speaker_alignment"]

Turn = Tuple[float, float, str]


def read_rttm(path: str) -> List[Turn]:
    out = []
    for line in open(path, encoding="utf-8"):
        f = line.split()
        if len(f) >= 8 and f[0] == "SPEAKER":
            out.append((float(f[3]), float(f[3]) + float(f[4]), f[7]))
    return out


def _activity(turns: Sequence[Turn], speakers: Sequence[str], edges: np.ndarray) -> np.ndarray:
    """[speakers, segments] bool: whether a speaker talks during each elementary segment between consecutive ``edges``."""
    mid = 0.5 * (edges[:-1] + edges[1:])
    act = np.zeros((len(speakers), len(mid)), dtype=bool)
    idx = {s: i for i, s in enumerate(speakers)}
    for a, b, s in turns:
        act[idx[s]] |= (mid >= a) & (mid < b)
    return act


def diarization_error_rate(reference: Sequence[Turn], hypothesis: Sequence[Turn], collar: float = 0.25, ignore_overlap: bool = False,
                           uem: Optional[Sequence[Tuple[float, float]]] = None) -> Dict[str, object]:
    """``collar``: seconds on each side of every reference boundary that are not scored (0.25 is the customary value).
    ``ignore_overlap``: regions where more than one reference speaker talks are not scored.  ``uem``: scored regions (all time
    when ``None``).  The timeline is cut at every boundary into elementary segments on which all activities are constant; in a
    segment with ``r`` reference and ``h`` hypothesis speakers of which ``c`` are correctly matched, miss = max(0, r - h),
    false alarm = max(0, h - r), confusion = min(r, h) - c, and the denominator is r (all times the segment's duration)."""
    ref = [(float(a), float(b), str(s)) for a, b, s in reference if b > a]
    hyp = [(float(a), float(b), str(s)) for a, b, s in hypothesis if b > a]
    cuts = {0.0}
    for a, b, _ in ref + hyp:
        cuts.update((a, b))
    for a, b, _ in ref:
        cuts.update((max(0.0, a - collar), a + collar, max(0.0, b - collar), b + collar))
    for a, b in uem or ():
        cuts.update((a, b))
    edges = np.array(sorted(cuts))
    if len(edges) < 2:
        return {"DER": 0.0, "miss": 0.0, "false_alarm": 0.0, "confusion": 0.0, "total": 0.0, "mapping": {}}
    dur = np.diff(edges)
    mid = 0.5 * (edges[:-1] + edges[1:])
    rs, hs = sorted({s for _, _, s in ref}), sorted({s for _, _, s in hyp})
    R, H = _activity(ref, rs, edges), _activity(hyp, hs, edges)
    scored = np.ones(len(mid), dtype=bool)
    if uem:
        scored &= np.any([(mid >= a) & (mid < b) for a, b in uem], axis=0)
    if collar > 0:
        for a, b, _ in ref:
            scored &= ~((mid >= a - collar) & (mid < a + collar)) & ~((mid >= b - collar) & (mid < b + collar))
    if ignore_overlap:
        scored &= R.sum(0) <= 1
    w = dur * scored
    # speaker mapping: maximise the time on which a reference and a hypothesis speaker are both active
    mapping: Dict[str, str] = {}
    matched = np.zeros(len(mid))
    if len(rs) and len(hs):
        overlap = (R[:, None, :] & H[None, :, :]).astype(float) @ w            # [R, H]
        ri, hi = linear_sum_assignment(-overlap)
        for i, j in zip(ri, hi):
            if overlap[i, j] > 0:
                mapping[hs[j]] = rs[i]
                matched += R[i] & H[j]
    nr, nh = R.sum(0), H.sum(0)
    miss = float((np.maximum(0, nr - nh) * w).sum())
    fa = float((np.maximum(0, nh - nr) * w).sum())
    conf = float(((np.minimum(nr, nh) - matched) * w).sum())
    total = float((nr * w).sum())
    d = max(total, 1e-9)
    return {"DER": (miss + fa + conf) / d, "miss": miss / d, "false_alarm": fa / d, "confusion": conf / d, "total": total, "mapping": mapping,
            "miss_time": miss, "false_alarm_time": fa, "confusion_time": conf}


def score_labels(references: Dict[str, Sequence[Turn]], hypotheses: Dict[str, Sequence[Turn]], collar: float = 0.25, ignore_overlap: bool = True,
                 uems: Optional[Dict[str, Sequence[Tuple[float, float]]]] = None) -> Dict[str, object]:
    """Pooled over recordings (errors and reference time are summed before the division); per-recording results under ``"items"``."""
    tot = {"miss_time": 0.0, "false_alarm_time": 0.0, "confusion_time": 0.0, "total": 0.0}
    items, mappings = {}, {}
    for uid, ref in references.items():
        r = diarization_error_rate(ref, hypotheses.get(uid, []), collar, ignore_overlap, (uems or {}).get(uid))
        items[uid] = r["DER"]
        mappings[uid] = r["mapping"]
        for k in tot:
            tot[k] += r[k]
    d = max(tot["total"], 1e-9)
    return {"DER": (tot["miss_time"] + tot["false_alarm_time"] + tot["confusion_time"]) / d, "miss": tot["miss_time"] / d, "false_alarm": tot["false_alarm_time"] / d,
            "confusion": tot["confusion_time"] / d, "items": items, "mapping": mappings}


# ------------------------------------------------------------------------------------------------ cpWER
def cp_wer(hyp_by_speaker: Sequence[str], ref_by_speaker: Sequence[str]) -> Tuple[float, List[str], List[str]]:
    """``hyp_by_speaker[i]``: everything hypothesis speaker i said, concatenated; same for the references.  Returns
    ``(cpWER, hypothesis texts in the order matched to the references, reference texts)``; unmatched speakers on either side are
    paired with the empty string, so all their words count as errors."""
    hyp, ref = [h.split() for h in hyp_by_speaker], [r.split() for r in ref_by_speaker]
    n = max(len(hyp), len(ref))
    hyp += [[]] * (n - len(hyp))
    ref += [[]] * (n - len(ref))
    cost = np.array([[edit_distance(h, r) for r in ref] for h in hyp], dtype=float)
    hi, ri = linear_sum_assignment(cost)
    errors = float(cost[hi, ri].sum())
    words = sum(len(r) for r in ref)
    order = [None] * n
    for h, r in zip(hi, ri):
        order[r] = h
    return errors / max(1, words), [" ".join(hyp[h]) for h in order], [" ".join(r) for r in ref]


# ------------------------------------------------------------------------------------------------ multi-label frame accuracy
class MultiBinaryAccuracy:
    """``update(preds [B, T, S] probabilities, targets [B, T, S] 0/1, lengths [B])`` accumulates confusion counts over the valid
    frames; ``compute()`` -> ``(f1, precision, recall)``; ``accuracy()`` is the share of correct frame-speaker decisions."""

    def __init__(self, threshold: float = 0.5):
        self.thr = threshold
        self.reset()

    def reset(self):
        self.tp = self.fp = self.fn = self.tn = 0.0

    def update(self, preds: torch.Tensor, targets: torch.Tensor, signal_lengths: Optional[torch.Tensor] = None):
        p, t = preds.detach() > self.thr, targets.detach() > 0.5
        if signal_lengths is not None:
            m = (torch.arange(p.shape[1], device=p.device)[None, :] < signal_lengths[:, None].to(p.device)).unsqueeze(-1).expand_as(p)
        else:
            m = torch.ones_like(p)
        self.tp += float((p & t & m).sum())
        self.fp += float((p & ~t & m).sum())
        self.fn += float((~p & t & m).sum())
        self.tn += float((~p & ~t & m).sum())

    def sync(self):
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            v = torch.tensor([self.tp, self.fp, self.fn, self.tn], dtype=torch.float64)
            if torch.distributed.get_backend() == "nccl":
                v = v.cuda()
            torch.distributed.all_reduce(v)
            self.tp, self.fp, self.fn, self.tn = [float(x) for x in v.cpu()]

    def compute(self) -> Tuple[float, float, float]:
        prec = self.tp / max(1e-9, self.tp + self.fp)
        rec = self.tp / max(1e-9, self.tp + self.fn)
        return 2 * prec * rec / max(1e-9, prec + rec), prec, rec

    def accuracy(self) -> float:
        return (self.tp + self.tn) / max(1e-9, self.tp + self.tn + self.fp + self.fn)


# ------------------------------------------------------------------------------------------------ long recordings
def long_form_clustering(embeddings: np.ndarray, cluster_fn, window: int = 2000, keep_per_cluster: int = 50, max_num_speakers: int = 8,
                         oracle_num_speakers: Optional[int] = None) -> np.ndarray:
    """Clustering cost grows with the square (affinity) or cube (eigen-decomposition) of the number of segments.  Here the
    sequence is clustered window by window (``cluster_fn(affinity, max_num_speakers, oracle) -> labels``), every window cluster
    is reduced to its ``keep_per_cluster`` embeddings closest to the cluster mean, the kept embeddings of all windows are
    clustered together, and every original segment takes the final label of its window cluster."""
    from ..models.diarizers import cosine_affinity

    n = len(embeddings)
    if n <= window:
        return np.asarray(cluster_fn(cosine_affinity(embeddings), max_num_speakers, oracle_num_speakers))
    kept, owner, win_labels = [], [], np.zeros(n, dtype=np.int64)
    next_id = 0
    for s in range(0, n, window):
        e = embeddings[s:s + window]
        lab = np.asarray(cluster_fn(cosine_affinity(e), max_num_speakers, None))
        for c in np.unique(lab):
            idx = np.nonzero(lab == c)[0]
            mean = e[idx].mean(0, keepdims=True)
            sim = (e[idx] @ mean.T)[:, 0] / (np.linalg.norm(e[idx], axis=1) * np.linalg.norm(mean) + 1e-9)
            top = idx[np.argsort(-sim)[:keep_per_cluster]]
            kept.append(e[top])
            owner += [next_id] * len(top)
            win_labels[s + idx] = next_id
            next_id += 1
    kept_e, owner = np.concatenate(kept), np.asarray(owner)
    final = np.asarray(cluster_fn(cosine_affinity(kept_e), max_num_speakers, oracle_num_speakers))
    vote = np.zeros(next_id, dtype=np.int64)
    for c in range(next_id):
        vals, counts = np.unique(final[owner == c], return_counts=True)
        vote[c] = vals[counts.argmax()]
    return vote[win_labels]


# ------------------------------------------------------------------------------------------------ serialised output training
def sot_speaker_alignment(hyp_text: str, ref_by_speaker: Sequence[str], change_token: str = "<sc>") -> Tuple[float, List[str]]:
    """A serialised-output-training transcript lists the speakers' utterances in order of start time separated by
    ``change_token``; in the two-speaker convention consecutive pieces alternate speakers, in general piece ``k`` may belong to any
    speaker.  Pieces are assigned greedily to the reference speaker whose remaining text they match best (edit distance to the
    prefix of equal length), then cpWER is computed on the per-speaker concatenations."""
    pieces = [p.strip() for p in hyp_text.split(change_token) if p.strip()]
    refs = [r.split() for r in ref_by_speaker]
    pos = [0] * len(refs)
    by = [[] for _ in refs]
    for p in pieces:
        w = p.split()
        best, best_cost = 0, None
        for k, r in enumerate(refs):
            seg = r[pos[k]: pos[k] + len(w)]
            cost = edit_distance(w, seg) + (0 if seg else len(w))
            if best_cost is None or cost < best_cost:
                best, best_cost = k, cost
        by[best] += w
        pos[best] += len(w)
    hyp_by = [" ".join(x) for x in by]
    score, _, _ = cp_wer(hyp_by, list(ref_by_speaker))
    return score, hyp_by

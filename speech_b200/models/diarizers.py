"""Clustering-based speaker diarization: VAD → multi-scale segmentation → speaker embeddings → NME-SC spectral clustering
→ RTTM; and the online variant that re-clusters a bounded history while keeping speaker labels stable.

Reference: ``models/clustering_diarizer.py``, ``models/online_diarizer.py``, ``parts/utils/offline_clustering.py``
(NME-SC: normalised maximum eigengap spectral clustering), ``parts/utils/online_clustering.py``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..core.config import DictConfig, OmegaConf, cfg_get
from ..data.audio_to_text import load_audio
from ..data.diarization import write_rttm


def energy_vad(x: np.ndarray, sr: int, frame: float = 0.02, threshold_db: float = -35.0, min_speech: float = 0.2,
               min_silence: float = 0.2) -> List[Tuple[float, float]]:
    n = max(1, int(frame * sr))
    T = len(x) // n
    if T == 0:
        return []
    e = 10 * np.log10((x[: T * n].reshape(T, n) ** 2).mean(1) + 1e-12)
    active = e > max(threshold_db, e.max() - 40.0)
    segs, on, st = [], False, 0
    for t in range(T):
        if active[t] and not on:
            on, st = True, t
        elif not active[t] and on:
            on = False
            segs.append((st * frame, t * frame))
    if on:
        segs.append((st * frame, T * frame))
    merged: List[Tuple[float, float]] = []
    for s, e2 in segs:
        if merged and s - merged[-1][1] < min_silence:
            merged[-1] = (merged[-1][0], e2)
        else:
            merged.append((s, e2))
    return [(s, e2) for s, e2 in merged if e2 - s >= min_speech]


def get_subsegments(start: float, end: float, window: float, shift: float) -> List[Tuple[float, float]]:
    out, t = [], start
    while t + window <= end + 1e-9:
        out.append((t, t + window))
        t += shift
    if not out or out[-1][1] < end - 0.1 * window:
        out.append((max(start, end - window), end))
    return out


def cosine_affinity(emb: np.ndarray) -> np.ndarray:
    e = emb / np.maximum(np.linalg.norm(emb, axis=1, keepdims=True), 1e-8)
    a = e @ e.T
    return (a - a.min()) / max(a.max() - a.min(), 1e-8)


def nme_spectral_clustering(affinity: np.ndarray, max_num_speakers: int = 8, oracle_num_speakers: Optional[int] = None,
                            max_rp_threshold: float = 0.25, sparse_search_volume: int = 10, seed: int = 0) -> np.ndarray:
    """Binarise the affinity by keeping the ``p`` strongest neighbours per row, choose ``p`` minimising
    ``(p / N) / max eigengap`` of the graph Laplacian, estimate the speaker count from the eigengap and run k-means on the
    spectral embedding."""
    N = affinity.shape[0]
    if N <= 2:
        return np.zeros(N, dtype=np.int64)
    max_p = max(2, int(N * max_rp_threshold))
    cand = sorted(set(np.linspace(2, max_p, num=min(sparse_search_volume, max_p - 1), dtype=int).tolist()))
    if N < 40:
        # too few segments for the eigengap search to be stable: one well-connected graph instead
        cand = [max(3, int(0.4 * N))]
    best = None
    for p in cand:
        idx = np.argsort(-affinity, axis=1)[:, :p]
        B = np.zeros_like(affinity)
        np.put_along_axis(B, idx, 1.0, axis=1)
        B = 0.5 * (B + B.T)
        L = np.diag(B.sum(1)) - B
        w = np.linalg.eigvalsh(L)
        k_max = min(max_num_speakers, N - 1)
        gaps = np.diff(w[: k_max + 1])
        g = gaps.max() / max(w[: k_max + 1].max(), 1e-8)
        ratio = (p / N) / max(g, 1e-8)
        if best is None or ratio < best[0]:
            best = (ratio, p, B, int(np.argmax(gaps)) + 1)
    _, p, B, k_est = best
    k = oracle_num_speakers or max(1, min(k_est, max_num_speakers))
    L = np.diag(B.sum(1)) - B
    w, v = np.linalg.eigh(L)
    spec = v[:, :k]
    from sklearn.cluster import KMeans

    return KMeans(n_clusters=k, n_init=10, random_state=seed).fit_predict(spec).astype(np.int64)


class ClusteringDiarizer:
    """``diarize(paths)`` writes ``<out_dir>/pred_rttms/<name>.rttm`` and returns ``{name: [(start, end, speaker)]}``."""

    def __init__(self, cfg=None, speaker_model=None, vad_model=None):
        cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg or {})
        self.cfg = cfg
        d = cfg.get("diarizer", cfg)
        self.out_dir = cfg_get(d, "out_dir", None)
        se = cfg_get(d, "speaker_embeddings", {}) or {}
        p = cfg_get(se, "parameters", {}) or {}
        self.windows = list(_as_list(cfg_get(p, "window_length_in_sec", [1.5, 1.0, 0.5])))
        self.shifts = list(_as_list(cfg_get(p, "shift_length_in_sec", [0.75, 0.5, 0.25])))
        self.scale_weights = list(_as_list(cfg_get(p, "multiscale_weights", [1.0] * len(self.windows))))
        cl = cfg_get(cfg_get(d, "clustering", {}) or {}, "parameters", {}) or {}
        self.oracle_num_speakers = cfg_get(cl, "oracle_num_speakers", False)
        self.max_num_speakers = cfg_get(cl, "max_num_speakers", 8)
        self.max_rp_threshold = cfg_get(cl, "max_rp_threshold", 0.25)
        self.sparse_search_volume = cfg_get(cl, "sparse_search_volume", 10)
        self.sample_rate = cfg_get(cfg, "sample_rate", 16000)
        self.speaker_model = speaker_model
        self.vad_model = vad_model
        if speaker_model is None and cfg_get(se, "model_path", None):
            from .classification_models import EncDecSpeakerLabelModel

            self.speaker_model = EncDecSpeakerLabelModel.restore_from(se["model_path"])

    def _vad(self, x: np.ndarray) -> List[Tuple[float, float]]:
        if self.vad_model is not None and hasattr(self.vad_model, "speech_segments"):
            return self.vad_model.speech_segments(x, self.sample_rate)
        return energy_vad(x, self.sample_rate)

    @torch.no_grad()
    def _embed(self, x: np.ndarray, segs: Sequence[Tuple[float, float]]) -> np.ndarray:
        chunks = [x[int(s * self.sample_rate): int(e * self.sample_rate)] for s, e in segs]
        embs, _ = self.speaker_model.batch_inference(chunks, batch_size=64)
        return embs.numpy()

    def diarize_array(self, x: np.ndarray, num_speakers: Optional[int] = None) -> List[Tuple[float, float, str]]:
        speech = self._vad(x)
        if not speech:
            return []
        base_scale = len(self.windows) - 1
        scale_segs = [[ss for s, e in speech for ss in get_subsegments(s, e, w, sh)] for w, sh in zip(self.windows, self.shifts)]
        embs = [self._embed(x, segs) for segs in scale_segs]
        base = scale_segs[base_scale]
        centers = np.array([(s + e) / 2 for s, e in base])
        aff = np.zeros((len(base), len(base)))
        for segs, e, wt in zip(scale_segs, embs, self.scale_weights):
            c = np.array([(s + t) / 2 for s, t in segs])
            nearest = np.abs(centers[:, None] - c[None, :]).argmin(1)     # map every base segment to this scale
            aff += wt * cosine_affinity(e[nearest])
        aff /= max(sum(self.scale_weights), 1e-8)
        labels = nme_spectral_clustering(aff, self.max_num_speakers, num_speakers, self.max_rp_threshold, self.sparse_search_volume)
        out: List[Tuple[float, float, str]] = []
        for (s, e), l in zip(base, labels):
            spk = f"speaker_{int(l)}"
            if out and out[-1][2] == spk and s <= out[-1][1] + 1e-6:
                out[-1] = (out[-1][0], max(e, out[-1][1]), spk)
            else:
                if out and s < out[-1][1]:                           # overlapping windows of different speakers: split in the middle
                    mid = (s + out[-1][1]) / 2
                    out[-1] = (out[-1][0], mid, out[-1][2])
                    s = mid
                out.append((s, e, spk))
        return out

    def diarize(self, paths_or_arrays: Sequence, num_speakers: Optional[Sequence[Optional[int]]] = None, batch_size: int = 0):
        results = {}
        for i, a in enumerate(paths_or_arrays):
            name = os.path.splitext(os.path.basename(a))[0] if isinstance(a, str) else f"session_{i}"
            x = np.asarray(load_audio(a, target_sr=self.sample_rate) if isinstance(a, str) else a, dtype=np.float32)
            k = num_speakers[i] if num_speakers is not None else None
            segs = self.diarize_array(x, k)
            results[name] = segs
            if self.out_dir:
                os.makedirs(os.path.join(self.out_dir, "pred_rttms"), exist_ok=True)
                write_rttm(os.path.join(self.out_dir, "pred_rttms", name + ".rttm"), segs, uniq_id=name)
        return results


class OnlineDiarizer(ClusteringDiarizer):
    """Streaming variant: call ``diarize_step(chunk)`` repeatedly.  A bounded history of embeddings is re-clustered at every
    step and the new clusters are matched to the previous speakers by centroid similarity so that labels stay stable."""

    def __init__(self, cfg=None, speaker_model=None, vad_model=None, history_sec: float = 120.0):
        super().__init__(cfg, speaker_model, vad_model)
        self.history_sec = history_sec
        self.reset()

    def reset(self):
        self.audio = np.zeros(0, dtype=np.float32)
        self.offset = 0.0
        self.centroids: Dict[str, np.ndarray] = {}
        self.total = 0.0

    def diarize_step(self, chunk: np.ndarray) -> List[Tuple[float, float, str]]:
        chunk = np.asarray(chunk, dtype=np.float32)
        self.total += len(chunk) / self.sample_rate
        self.audio = np.concatenate([self.audio, chunk])
        keep = int(self.history_sec * self.sample_rate)
        if len(self.audio) > keep:
            self.offset += (len(self.audio) - keep) / self.sample_rate
            self.audio = self.audio[-keep:]
        segs = self.diarize_array(self.audio)
        if not segs:
            return []
        w = self.windows[-1]
        names = sorted({s[2] for s in segs})
        cents = {}
        for n in names:
            sub = [(s, e) for s, e, k in segs if k == n and e - s >= 0.2]
            if sub:
                cents[n] = self._embed(self.audio, sub).mean(0)
        mapping: Dict[str, str] = {}
        used = set()
        for n, c in cents.items():
            best, bs = None, 0.5
            for old, oc in self.centroids.items():
                if old in used:
                    continue
                sim = float(c @ oc / max(np.linalg.norm(c) * np.linalg.norm(oc), 1e-8))
                if sim > bs:
                    best, bs = old, sim
            if best is None:
                best = f"speaker_{len(self.centroids) + len([m for m in mapping.values() if m not in self.centroids])}"
            mapping[n] = best
            used.add(best)
        for n, c in cents.items():
            old = self.centroids.get(mapping[n])
            self.centroids[mapping[n]] = c if old is None else 0.9 * old + 0.1 * c
        return [(s + self.offset, e + self.offset, mapping.get(k, k)) for s, e, k in segs]


def _as_list(v):
    if isinstance(v, (int, float)):
        return [v]
    return list(v)

"""Room impulse responses by the image-source method, and a corpus generator for augmentation manifests.

A shoebox room with frequency-independent wall absorption: the response from a source to a microphone is the sum over image
sources ``(±x + 2 n_x L_x, ...)`` of ``beta^(number of reflections) / (4 pi d) * delta(t - d / c)``, each impulse rendered with a
windowed-sinc fractional delay.  The reflection coefficient follows from the requested reverberation time through Sabine's
formula.  ``RIRCorpusGenerator`` draws rooms, reverberation times and positions from configured ranges, writes the responses as
audio files plus a manifest that ``ImpulsePerturbation`` / ``RirAndNoisePerturbation`` read, and records the measured RT60.

Reference: ``tools/rir_corpus_generator`` and ``collections/audio/data/data_simulation.py`` (room / position sampling, manifest
fields ``room_dim``, ``rt60``, ``source_position``, ``mic_positions``); the reference calls pyroomacoustics for the simulation.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

SPEED_OF_SOUND = 343.0


def sabine_reflection(room_dim: Sequence[float], rt60: float) -> float:
    """Uniform wall reflection coefficient beta = sqrt(1 - alpha) for a target RT60 (Sabine: RT60 = 0.161 V / (alpha S))."""
    lx, ly, lz = room_dim
    vol, surf = lx * ly * lz, 2 * (lx * ly + ly * lz + lx * lz)
    alpha = min(0.999, max(1e-3, 0.161 * vol / (surf * max(rt60, 1e-3))))
    return math.sqrt(1.0 - alpha)


def image_source_rir(room_dim: Sequence[float], source: Sequence[float], mic: Sequence[float], rt60: float, sample_rate: int = 16000,
                     max_order: int = 12, length_s: Optional[float] = None, frac_taps: int = 41) -> np.ndarray:
    room, src, m = np.asarray(room_dim, float), np.asarray(source, float), np.asarray(mic, float)
    if np.any(src <= 0) or np.any(src >= room) or np.any(m <= 0) or np.any(m >= room):
        raise ValueError("source and microphone must lie inside the room")
    beta = sabine_reflection(room_dim, rt60)
    n = int((length_s or max(0.1, 1.2 * rt60)) * sample_rate)
    h = np.zeros(n + frac_taps, dtype=np.float64)
    rng = np.arange(-max_order, max_order + 1)
    half = frac_taps // 2
    win = np.hanning(frac_taps)
    taps = np.arange(frac_taps) - half
    # per axis: image coordinate and its reflection count for (n, parity)
    axes = []
    for a in range(3):
        pos, cnt = [], []
        for k in rng:
            for par in (0, 1):
                pos.append((1 - 2 * par) * src[a] + 2 * k * room[a])
                cnt.append(abs(2 * k - par))
        axes.append((np.asarray(pos), np.asarray(cnt)))
    (px, cx), (py, cy), (pz, cz) = axes
    dx, dy, dz = px - m[0], py - m[1], pz - m[2]
    for ix in range(len(px)):
        for iy in range(len(py)):
            d = np.sqrt(dx[ix] ** 2 + dy[iy] ** 2 + dz ** 2)
            refl = cx[ix] + cy[iy] + cz
            keep = refl <= max_order
            delay = d[keep] / SPEED_OF_SOUND * sample_rate
            amp = beta ** refl[keep] / (4 * math.pi * np.maximum(d[keep], 1e-2))
            ok = delay < n - 1
            for dl, am in zip(delay[ok], amp[ok]):
                i0 = int(math.floor(dl))
                frac = dl - i0
                lo = i0 - half
                kern = np.sinc(taps - frac) * win * am
                s = max(0, -lo)
                h[lo + s: lo + frac_taps] += kern[s:]
    return h[:n].astype(np.float32)


def measure_rt60(h: np.ndarray, sample_rate: int, decay_db: float = 30.0) -> float:
    """Schroeder backward integration; RT60 extrapolated from the -5 .. -(5 + decay_db) dB slope."""
    e = np.cumsum((h.astype(np.float64) ** 2)[::-1])[::-1]
    e = 10 * np.log10(np.maximum(e / max(e[0], 1e-30), 1e-30))
    try:
        i0 = int(np.argmax(e <= -5.0))
        i1 = int(np.argmax(e <= -5.0 - decay_db))
    except ValueError:
        return float("nan")
    if i1 <= i0:
        return float("nan")
    return 60.0 / decay_db * (i1 - i0) / sample_rate


class RIRCorpusGenerator:
    def __init__(self, room_dim_range=((3, 8), (3, 8), (2.4, 4)), rt60_range=(0.15, 0.8), num_mics: int = 1, mic_spacing: float = 0.05,
                 min_wall_distance: float = 0.3, sample_rate: int = 16000, max_order: int = 10, seed: int = 0):
        self.room_dim_range, self.rt60_range = room_dim_range, rt60_range
        self.num_mics, self.mic_spacing, self.min_wall = num_mics, mic_spacing, min_wall_distance
        self.sample_rate, self.max_order = sample_rate, max_order
        self.rng = np.random.default_rng(seed)

    def _inside(self, room) -> np.ndarray:
        return np.array([self.rng.uniform(self.min_wall, r - self.min_wall) for r in room])

    def sample(self) -> Dict:
        room = [float(self.rng.uniform(*r)) for r in self.room_dim_range]
        rt60 = float(self.rng.uniform(*self.rt60_range))
        src = self._inside(room)
        centre = self._inside(room)
        mics = [np.clip(centre + np.array([(k - (self.num_mics - 1) / 2) * self.mic_spacing, 0, 0]), 0.05, np.array(room) - 0.05)
                for k in range(self.num_mics)]
        rirs = np.stack([image_source_rir(room, src, m, rt60, self.sample_rate, self.max_order) for m in mics])
        return {"room_dim": room, "rt60": rt60, "source_position": src.tolist(), "mic_positions": [m.tolist() for m in mics],
                "rir": rirs, "rt60_measured": measure_rt60(rirs[0], self.sample_rate)}

    def generate(self, out_dir: str, num_rooms: int) -> str:
        from .audio_to_text import save_wav

        os.makedirs(out_dir, exist_ok=True)
        manifest = os.path.join(out_dir, "rir_manifest.json")
        with open(manifest, "w") as f:
            for i in range(num_rooms):
                s = self.sample()
                path = os.path.join(out_dir, f"rir_{i:05d}.wav")
                gain = 0.9 / max(float(np.abs(s["rir"]).max()), 1e-9)             # 16-bit files: use the full range, keep the gain
                save_wav(path, (s["rir"].T if self.num_mics > 1 else s["rir"][0]) * gain, self.sample_rate)
                rec = {k: v for k, v in s.items() if k != "rir"}
                rec.update(audio_filepath=path, duration=s["rir"].shape[1] / self.sample_rate, gain=gain)
                f.write(json.dumps(rec) + "\n")
        return manifest

"""Simulation of multichannel recordings: microphone array geometry with orientation, room impulse responses for sources placed
relative to the array, and mixtures of a target speaker with interfering speakers, directional noise and diffuse background noise at
chosen level ratios.

Reference: ``audio/data/data_simulation.py`` (``ArrayGeometry``, ``RIRCorpusGenerator``, ``RIRMixGenerator`` and helpers).  Room
responses come from this package's image-source model (``data/rir_generator.py``) instead of an external room simulator.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..data.rir_generator import image_source_rir, measure_rt60
from .utils import db2mag, generate_approximate_noise_field, rms

__all__ = ["ArrayGeometry", "RIRMixGenerator", "calculate_drr", "convolve_rir", "normalize_max", "scaled_disturbance", "simulate_array_rirs",
           "simultaneously_active_rms", "wrap_to_180"]


def wrap_to_180(angle: float) -> float:
    return float((angle + 180.0) % 360.0 - 180.0)


class ArrayGeometry:
    """Microphone positions ``[mics, 3]`` in metres.  The array can be moved (``translate``) and turned (``rotate`` by yaw, pitch,
    roll in degrees about its centre); ``spherical_relative_to_array(point)`` gives range, azimuth and elevation of a point as the
    array sees it, and ``new_point`` places a point at a wanted range / azimuth / elevation."""

    def __init__(self, mic_positions, center: Optional[Sequence[float]] = None, internal_cs=None):
        self.positions = np.asarray(mic_positions, dtype=np.float64).reshape(-1, 3)
        self.centroid = self.positions.mean(0) if center is None else np.asarray(center, dtype=np.float64)
        self.internal_cs = np.eye(3) if internal_cs is None else np.asarray(internal_cs, dtype=np.float64)     # columns: the array's x, y, z axes

    @property
    def num_mics(self) -> int:
        return self.positions.shape[0]

    @property
    def radius(self) -> float:
        return float(np.linalg.norm(self.positions - self.centroid, axis=1).max())

    @staticmethod
    def _rotation(yaw: float, pitch: float, roll: float) -> np.ndarray:
        y, p, r = np.deg2rad([yaw, pitch, roll])
        Rz = np.array([[np.cos(y), -np.sin(y), 0], [np.sin(y), np.cos(y), 0], [0, 0, 1]])
        Ry = np.array([[np.cos(p), 0, np.sin(p)], [0, 1, 0], [-np.sin(p), 0, np.cos(p)]])
        Rx = np.array([[1, 0, 0], [0, np.cos(r), -np.sin(r)], [0, np.sin(r), np.cos(r)]])
        return Rz @ Ry @ Rx

    def translate(self, to: Sequence[float]) -> "ArrayGeometry":
        to = np.asarray(to, dtype=np.float64)
        return ArrayGeometry(self.positions - self.centroid + to, to, self.internal_cs)

    def rotate(self, yaw: float = 0.0, pitch: float = 0.0, roll: float = 0.0) -> "ArrayGeometry":
        R = self._rotation(yaw, pitch, roll)
        return ArrayGeometry((self.positions - self.centroid) @ R.T + self.centroid, self.centroid, R @ self.internal_cs)

    def spherical_relative_to_array(self, point: Sequence[float]) -> Tuple[float, float, float]:
        v = self.internal_cs.T @ (np.asarray(point, dtype=np.float64) - self.centroid)
        rng = float(np.linalg.norm(v))
        return rng, float(np.rad2deg(np.arctan2(v[1], v[0]))), float(np.rad2deg(np.arcsin(v[2] / rng))) if rng > 0 else 0.0

    def new_point(self, rng: float, azimuth: float, elevation: float) -> np.ndarray:
        a, e = np.deg2rad([azimuth, elevation])
        v = rng * np.array([np.cos(e) * np.cos(a), np.cos(e) * np.sin(a), np.sin(e)])
        return self.centroid + self.internal_cs @ v


def simulate_array_rirs(room_dim: Sequence[float], array: ArrayGeometry, sources: Sequence[Sequence[float]], rt60: float, sample_rate: int = 16000,
                        max_order: int = 10) -> List[np.ndarray]:
    """One ``[mics, taps]`` response per source (all padded to the longest)."""
    out = []
    for s in sources:
        h = [image_source_rir(room_dim, s, m, rt60, sample_rate, max_order) for m in array.positions]
        L = max(len(x) for x in h)
        out.append(np.stack([np.pad(x, (0, L - len(x))) for x in h]))
    return out


def convolve_rir(signal: np.ndarray, rir: np.ndarray) -> np.ndarray:
    """``signal`` [samples], ``rir`` [mics, taps] -> [samples, mics] (the tail beyond the input length is cut)."""
    n = len(signal)
    nf = 1 << (n + rir.shape[1] - 2).bit_length()
    S = np.fft.rfft(signal, nf)
    return np.stack([np.fft.irfft(S * np.fft.rfft(h, nf), nf)[:n] for h in rir], axis=1)


def calculate_drr(rir: np.ndarray, sample_rate: float, n_0_ms: float = 2.5) -> List[float]:
    """Direct-to-reverberant ratio in dB per microphone: energy within ``n_0_ms`` of the direct-path peak over the energy after."""
    out = []
    w = int(n_0_ms * 1e-3 * sample_rate)
    for h in np.atleast_2d(rir):
        p = int(np.argmax(np.abs(h)))
        direct = np.sum(h[max(0, p - w): p + w + 1] ** 2)
        rest = np.sum(h[p + w + 1:] ** 2)
        out.append(float(10 * np.log10(direct / max(rest, 1e-16))))
    return out


def normalize_max(x: np.ndarray, max_db: float = 0.0, eps: float = 1e-16) -> np.ndarray:
    return x * db2mag(max_db) / (np.abs(x).max() + eps)


def simultaneously_active_rms(x: np.ndarray, y: np.ndarray, sample_rate: float, rms_threshold_db: float = -60.0, window_len_ms: float = 200.0) -> Tuple[float, float]:
    """RMS of ``x`` and ``y`` over the windows in which both are active (level within ``rms_threshold_db`` of their own maximum):
    level ratios between intermittent signals such as speech should be set where both are present."""
    n = int(window_len_ms * 1e-3 * sample_rate)
    k = min(len(x), len(y)) // n
    if k == 0:
        return rms(x), rms(y)
    xw, yw = x[: k * n].reshape(k, n), y[: k * n].reshape(k, n)
    xr, yr = np.sqrt((xw ** 2).mean(1)), np.sqrt((yw ** 2).mean(1))
    act = (20 * np.log10(xr / (xr.max() + 1e-16) + 1e-16) > rms_threshold_db) & (20 * np.log10(yr / (yr.max() + 1e-16) + 1e-16) > rms_threshold_db)
    if not act.any():
        return rms(x), rms(y)
    return float(np.sqrt((xw[act] ** 2).mean())), float(np.sqrt((yw[act] ** 2).mean()))


def scaled_disturbance(signal: np.ndarray, disturbance: np.ndarray, sdr_db: float, sample_rate: Optional[float] = None, ref_channel: int = 0,
                       eps: float = 1e-16) -> np.ndarray:
    """The disturbance scaled so that signal-to-disturbance ratio at the reference channel is ``sdr_db``; with ``sample_rate`` the
    levels are measured where both are active."""
    s = signal[:, ref_channel] if signal.ndim > 1 else signal
    d = disturbance[:, ref_channel] if disturbance.ndim > 1 else disturbance
    rs, rd = simultaneously_active_rms(s, d, sample_rate) if sample_rate else (rms(s), rms(d))
    return disturbance * (rs / (rd + eps)) * db2mag(-sdr_db)


class RIRMixGenerator:
    """Draws a room, an array pose, a target and interferers around the array, convolves dry signals with the responses and mixes
    ``target + interference (at ``rsir`` dB) + directional noise and diffuse noise (at ``rsnr`` dB)``; ``target_reverberant`` is the
    target with the full response, ``target_anechoic`` the direct path only (what dereverberation should recover)."""

    def __init__(self, array: ArrayGeometry, room_dim_range=((3, 8), (3, 8), (2.4, 4.0)), rt60_range=(0.2, 0.8), target_range=(0.5, 2.5),
                 interferer_range=(1.0, 4.0), azimuth_range=(-180.0, 180.0), elevation_range=(-10.0, 30.0), num_interferers=(0, 2), rsnr_range=(5.0, 25.0),
                 rsir_range=(0.0, 15.0), diffuse_field: Optional[str] = "spherical", sample_rate: int = 16000, min_wall_distance: float = 0.3, max_order: int = 8,
                 ref_mic: int = 0, seed: int = 0):
        self.array, self.room_dim_range, self.rt60_range = array, room_dim_range, rt60_range
        self.target_range, self.interferer_range, self.az, self.el = target_range, interferer_range, azimuth_range, elevation_range
        self.num_interferers, self.rsnr, self.rsir, self.diffuse = num_interferers, rsnr_range, rsir_range, diffuse_field
        self.sr, self.wall, self.max_order, self.ref = sample_rate, min_wall_distance, max_order, ref_mic
        self.rng = np.random.default_rng(seed)

    def _place(self, arr: ArrayGeometry, room, rng_range) -> np.ndarray:
        for _ in range(200):
            p = arr.new_point(self.rng.uniform(*rng_range), self.rng.uniform(*self.az), self.rng.uniform(*self.el))
            if np.all(p > self.wall) and np.all(p < np.asarray(room) - self.wall):
                return p
        return np.clip(arr.centroid + np.array([0.5, 0.0, 0.0]), self.wall, np.asarray(room) - self.wall)

    def sample_scene(self) -> Dict[str, Any]:
        room = [float(self.rng.uniform(*r)) for r in self.room_dim_range]
        margin = self.wall + self.array.radius
        centre = np.array([self.rng.uniform(margin, r - margin) for r in room])
        arr = self.array.translate(centre).rotate(yaw=float(self.rng.uniform(-180, 180)))
        n_int = int(self.rng.integers(self.num_interferers[0], self.num_interferers[1] + 1))
        target = self._place(arr, room, self.target_range)
        inter = [self._place(arr, room, self.interferer_range) for _ in range(n_int)]
        return {"room_dim": room, "rt60": float(self.rng.uniform(*self.rt60_range)), "array": arr, "target": target, "interferers": inter,
                "rsnr": float(self.rng.uniform(*self.rsnr)), "rsir": float(self.rng.uniform(*self.rsir))}

    def mix(self, target: np.ndarray, interferers: Sequence[np.ndarray] = (), noise: Optional[np.ndarray] = None, scene: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        sc = scene or self.sample_scene()
        arr: ArrayGeometry = sc["array"]
        srcs = [sc["target"]] + list(sc["interferers"])[: len(interferers)]
        rirs = simulate_array_rirs(sc["room_dim"], arr, srcs, sc["rt60"], self.sr, self.max_order)
        n = len(target)
        tgt_rev = convolve_rir(target, rirs[0])
        direct = np.zeros_like(rirs[0])
        w = int(2.5e-3 * self.sr)
        for m, h in enumerate(rirs[0]):
            p = int(np.argmax(np.abs(h)))
            direct[m, max(0, p - w): p + w + 1] = h[max(0, p - w): p + w + 1]
        tgt_dir = convolve_rir(target, direct)
        mix = tgt_rev.copy()
        out: Dict[str, Any] = {"target_reverberant": tgt_rev, "target_anechoic": tgt_dir}
        if len(srcs) > 1:
            total = np.zeros_like(tgt_rev)
            for sig, h in zip(interferers, rirs[1:]):
                s = np.resize(sig, n) if len(sig) < n else sig[:n]
                total += convolve_rir(s, h)
            total = scaled_disturbance(tgt_rev, total, sc["rsir"], self.sr, self.ref)
            out["interference"] = total
            mix += total
        if noise is not None:
            nz = np.resize(noise, (n,) + noise.shape[1:]) if len(noise) < n else noise[:n]
            if nz.ndim == 1:
                if self.diffuse and arr.num_mics > 1:
                    seeds = np.stack([np.roll(nz, int(self.rng.integers(n // 4, n // 2)) * (m + 1)) for m in range(arr.num_mics)], axis=1)
                    seeds = seeds + 1e-3 * rms(nz) * self.rng.standard_normal(seeds.shape)
                    try:
                        nz = generate_approximate_noise_field(arr.positions, seeds, self.sr, self.diffuse)
                    except RuntimeError:                                  # shifted copies still too alike: fall back to independent noise
                        nz = generate_approximate_noise_field(arr.positions, rms(nz) * self.rng.standard_normal(seeds.shape), self.sr, self.diffuse)
                else:
                    nz = np.repeat(nz[:, None], arr.num_mics, axis=1)
            nz = scaled_disturbance(tgt_rev, nz, sc["rsnr"], None, self.ref)
            out["noise"] = nz
            mix += nz
        peak = np.abs(mix).max()
        gain = 0.99 / peak if peak > 0.99 else 1.0
        out.update({k: v * gain for k, v in out.items()})
        out["mix"] = mix * gain
        rng_, az, el = arr.spherical_relative_to_array(sc["target"])
        out["metadata"] = {"room_dim": sc["room_dim"], "rt60": sc["rt60"], "rt60_measured": measure_rt60(rirs[0][self.ref], self.sr), "rsnr": sc["rsnr"], "rsir": sc["rsir"],
                           "target_range": rng_, "target_azimuth": az, "target_elevation": el, "drr": calculate_drr(rirs[0], self.sr)[self.ref],
                           "num_interferers": len(srcs) - 1, "gain": gain}
        return out

    def generate(self, out_dir: str, targets: Sequence[np.ndarray], interferer_pool: Sequence[np.ndarray] = (), noise_pool: Sequence[np.ndarray] = ()) -> str:
        from ..data.audio_to_text import save_wav

        os.makedirs(out_dir, exist_ok=True)
        manifest = os.path.join(out_dir, "mix_manifest.json")
        with open(manifest, "w") as f:
            for i, t in enumerate(targets):
                sc = self.sample_scene()
                ints = [interferer_pool[int(self.rng.integers(len(interferer_pool)))] for _ in sc["interferers"]] if len(interferer_pool) else []
                nz = noise_pool[int(self.rng.integers(len(noise_pool)))] if len(noise_pool) else None
                r = self.mix(t, ints, nz, sc)
                rec = dict(r["metadata"])
                for key in ("mix", "target_reverberant", "target_anechoic", "interference", "noise"):
                    if key in r:
                        p = os.path.join(out_dir, f"{key}_{i:05d}.wav")
                        save_wav(p, r[key].astype(np.float32), self.sr)
                        rec[f"{key}_filepath"] = p
                rec["duration"] = len(t) / self.sr
                f.write(json.dumps(rec) + "\n")
        return manifest

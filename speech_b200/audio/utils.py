"""Numerical helpers of the audio collection: level conversions, spatial coherence of diffuse noise and synthesis of multichannel
noise with a wanted coherence, convolution matrices for linear prediction, scale- and convolution-invariant targets for SDR,
time alignment of a segment inside a signal, and spatial covariance matrices.

Reference: ``audio/parts/utils/audio.py``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

__all__ = ["calculate_sdr_numpy", "convmtx_mc_numpy", "convmtx_numpy", "convolution_invariant_target_numpy", "covariance_matrix", "db2mag", "estimated_coherence",
           "generate_approximate_noise_field", "get_segment_start", "mag2db", "pow2db", "rms", "scale_invariant_target_numpy", "theoretical_coherence",
           "toeplitz", "transform_to_match_coherence", "wrap_to_pi"]

SOUND_VELOCITY = 343.0


def rms(x: np.ndarray) -> float:
    return float(np.sqrt(np.mean(np.abs(x) ** 2)))


def mag2db(mag, eps: Optional[float] = 1e-16):
    return 20 * np.log10(np.asarray(mag) + (eps or 0.0))


def db2mag(db):
    return 10 ** (np.asarray(db) / 20)


def pow2db(power, eps: Optional[float] = 1e-16):
    return 10 * np.log10(np.asarray(power) + (eps or 0.0))


def wrap_to_pi(x: torch.Tensor) -> torch.Tensor:
    return torch.remainder(x + torch.pi, 2 * torch.pi) - torch.pi


# ------------------------------------------------------------------------------------------------ coherence
def theoretical_coherence(mic_positions: np.ndarray, sample_rate: float, field: str = "spherical", fft_length: int = 512,
                          sound_velocity: float = SOUND_VELOCITY) -> np.ndarray:
    """Coherence ``[bins, mics, mics]`` of an isotropic noise field between all microphone pairs: ``sinc(2 f d / c)`` for a
    spherically and ``J0(2 pi f d / c)`` for a cylindrically isotropic field, ``d`` the microphone distance."""
    pos = np.asarray(mic_positions, dtype=np.float64)
    d = np.linalg.norm(pos[:, None, :] - pos[None, :, :], axis=-1)
    f = np.arange(fft_length // 2 + 1) * sample_rate / fft_length
    arg = 2 * f[:, None, None] * d[None] / sound_velocity
    if field == "spherical":
        return np.sinc(arg)
    if field == "cylindrical":
        from scipy.special import j0

        return j0(np.pi * arg)
    raise ValueError(f"unknown noise field {field!r}")


def estimated_coherence(S: np.ndarray, eps: float = 1e-16) -> np.ndarray:
    """``S`` [bins, frames, mics] -> coherence [bins, mics, mics] estimated over the frames."""
    psd = np.einsum("ftm,ftn->fmn", S, S.conj()) / S.shape[1]
    p = np.real(np.einsum("fmm->fm", psd))
    return psd / (np.sqrt(p[:, :, None] * p[:, None, :]) + eps)


def transform_to_match_coherence(signal: np.ndarray, desired_coherence: np.ndarray, method: str = "cholesky", ref_channel: int = 0,
                                 corrcoef_threshold: float = 0.2, fft_length: int = 512, hop: Optional[int] = None) -> np.ndarray:
    """Mixes mutually uncorrelated channels ``signal`` [samples, mics] per frequency bin so that their coherence becomes
    ``desired_coherence`` [bins, mics, mics]: ``X' = X A`` with ``A^H A = Gamma`` (Cholesky or eigen-decomposition factor)."""
    M = signal.shape[1]
    cc = np.corrcoef(signal.T)
    if M > 1 and np.abs(cc[~np.eye(M, dtype=bool)]).max() > corrcoef_threshold:
        raise RuntimeError("the input channels must be (nearly) uncorrelated")
    hop = hop or fft_length // 4
    w = torch.hann_window(fft_length, dtype=torch.float64)
    X = torch.stft(torch.as_tensor(signal.T, dtype=torch.float64), fft_length, hop, fft_length, w, return_complex=True).numpy()   # [M, F, N]
    X = np.transpose(X, (1, 2, 0))                                                                                               # [F, N, M]
    Y = np.empty_like(X)
    for f in range(X.shape[0]):
        G = desired_coherence[f] + 1e-9 * np.eye(M)
        if method == "cholesky":
            A = np.linalg.cholesky(G).conj().T
        elif method == "evd":
            lam, V = np.linalg.eigh(G)
            A = np.sqrt(np.clip(lam, 0, None))[:, None] * V.conj().T
        else:
            raise ValueError(f"unknown method {method!r}")
        Y[f] = X[f] @ A
    y = torch.istft(torch.as_tensor(np.transpose(Y, (2, 0, 1))), fft_length, hop, fft_length, w, length=signal.shape[0]).numpy()
    return y.T


def generate_approximate_noise_field(mic_positions: np.ndarray, noise_signal: np.ndarray, sample_rate: float, field: str = "spherical", fft_length: int = 512,
                                     method: str = "cholesky", sound_velocity: float = SOUND_VELOCITY) -> np.ndarray:
    """Multichannel noise [samples, mics] whose inter-channel coherence approximates that of an isotropic field, from ``mics``
    uncorrelated noise signals."""
    g = theoretical_coherence(mic_positions, sample_rate, field, fft_length, sound_velocity)
    return transform_to_match_coherence(noise_signal, g, method=method, fft_length=fft_length)


# ------------------------------------------------------------------------------------------------ alignment, targets, SDR
def get_segment_start(signal: np.ndarray, segment: np.ndarray) -> int:
    """Index in ``signal`` at which ``segment`` starts (peak of the cross-correlation)."""
    n = len(signal) + len(segment) - 1
    nf = 1 << (n - 1).bit_length()
    cc = np.fft.irfft(np.fft.rfft(signal, nf) * np.conj(np.fft.rfft(segment, nf)), nf)
    lag = int(np.argmax(cc))
    return lag if lag < len(signal) else lag - nf


def convmtx_numpy(x: np.ndarray, filter_length: int, delay: int = 0, n_steps: Optional[int] = None) -> np.ndarray:
    """``[n_steps, filter_length]``: row ``t`` holds ``x[t - delay], x[t - delay - 1], ...`` (zeros before the start), so that
    ``convmtx @ h`` filters ``x`` with ``h`` after a delay."""
    n = n_steps or len(x)
    xp = np.concatenate([np.zeros(filter_length - 1 + delay, dtype=x.dtype), x])
    idx = (np.arange(n)[:, None] + (filter_length - 1) - np.arange(filter_length)[None, :])
    return xp[idx]


def convmtx_mc_numpy(x: np.ndarray, filter_length: int, delay: int = 0, n_steps: Optional[int] = None) -> np.ndarray:
    """Multichannel: ``x`` [samples, mics] -> [n_steps, mics * filter_length] (channel blocks side by side)."""
    return np.hstack([convmtx_numpy(x[:, m], filter_length, delay, n_steps) for m in range(x.shape[1])])


def scale_invariant_target_numpy(estimate: np.ndarray, target: np.ndarray, eps: float = 1e-8) -> np.ndarray:
    return (np.dot(estimate, target) / (np.dot(target, target) + eps)) * target


def convolution_invariant_target_numpy(estimate: np.ndarray, target: np.ndarray, filter_length: int, diag_reg: float = 1e-6, eps: float = 1e-8) -> np.ndarray:
    """The target passed through the FIR filter of ``filter_length`` taps that brings it closest to the estimate (least squares):
    distortions a short filter can explain (colouring, small delays) are not counted as errors."""
    T = convmtx_numpy(target, filter_length)
    R = T.T @ T
    R += diag_reg * (np.trace(R) / filter_length + eps) * np.eye(filter_length)
    h = np.linalg.solve(R, T.T @ estimate)
    return T @ h


def calculate_sdr_numpy(estimate: np.ndarray, target: np.ndarray, scale_invariant: bool = False, convolution_invariant: bool = False,
                        convolution_filter_length: int = 512, remove_mean: bool = True, sdr_max: Optional[float] = None, eps: float = 1e-8) -> float:
    if scale_invariant and convolution_invariant:
        raise ValueError("choose one of scale_invariant / convolution_invariant")
    e, t = np.asarray(estimate, dtype=np.float64), np.asarray(target, dtype=np.float64)
    if remove_mean:
        e, t = e - e.mean(), t - t.mean()
    if scale_invariant:
        t = scale_invariant_target_numpy(e, t, eps)
    elif convolution_invariant:
        t = convolution_invariant_target_numpy(e, t, convolution_filter_length, eps=eps)
    tp, dp = np.mean(t ** 2), np.mean((e - t) ** 2)
    if sdr_max is not None:
        dp = dp + 10 ** (-sdr_max / 10) * tp
    return float(10 * np.log10(tp / (dp + eps) + eps))


# ------------------------------------------------------------------------------------------------ covariance
def toeplitz(x: torch.Tensor) -> torch.Tensor:
    """``[..., L]`` -> Hermitian Toeplitz matrices ``[..., L, L]`` with first column ``x``."""
    L = x.shape[-1]
    i = torch.arange(L, device=x.device)
    d = i[:, None] - i[None, :]
    low = x[..., d.clamp(min=0)]
    up = x[..., (-d).clamp(min=0)].conj()
    return torch.where(d >= 0, low, up)


def covariance_matrix(x: torch.Tensor, mask: Optional[torch.Tensor] = None, normalize_mask: bool = True, eps: float = 1e-8) -> torch.Tensor:
    """``x`` [B, C, F, N] complex -> spatial covariance [B, F, C, C], frames weighted by ``mask`` [B, F, N] when given."""
    if mask is None:
        return torch.einsum("bcfn,bdfn->bfcd", x, x.conj()) / x.shape[-1]
    m = mask.to(x.real.dtype)
    if normalize_mask:
        m = m / (m.sum(dim=-1, keepdim=True) + eps)
    return torch.einsum("bcfn,bfn,bdfn->bfcd", x, m.to(x.dtype), x.conj())

"""Losses of the audio collection beyond SDR: mean squared and mean absolute error over valid samples / frames with per-channel
weights, and a combined enhancement loss (SI-SDR + spectral magnitude distance + a distance between features of a frozen
recogniser's encoder, which ties the enhancement to what an ASR model hears).

Reference: ``audio/losses/audio.py`` (``MSELoss``, ``MAELoss``, temporal means), ``audio/losses/maxine/losses_combined.py`` (``CombinedLoss``).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from .modules import si_sdr

__all__ = ["CombinedLoss", "MAELoss", "MSELoss", "calculate_mean", "temporal_mean"]


def temporal_mean(x: torch.Tensor, input_length: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None, keepdim: bool = False, eps: float = 1e-10):
    """Mean over the last dimension counting only the first ``input_length`` entries (or the entries where ``mask`` is set)."""
    if input_length is not None and mask is not None:
        raise RuntimeError("give input_length or mask, not both")
    if input_length is None and mask is None:
        return x.mean(dim=-1, keepdim=keepdim)
    if input_length is not None:
        m = torch.arange(x.shape[-1], device=x.device)[None, :] < input_length[:, None]
        m = m.view(x.shape[0], *([1] * (x.dim() - 2)), -1)
    else:
        m = mask
    m = m.to(x.dtype).expand_as(x)
    return (x * m).sum(dim=-1, keepdim=keepdim) / (m.sum(dim=-1, keepdim=keepdim) + eps)


def calculate_mean(x: torch.Tensor, input_length: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None, ndim: int = 3):
    """``ndim = 3``: signals [B, C, T] -> [B, C]; ``ndim = 4``: spectrograms [B, C, F, N] -> [B, C] (mean over F after the masked
    mean over frames)."""
    if x.dim() != ndim:
        raise RuntimeError(f"expected {ndim} dimensions, got {tuple(x.shape)}")
    m = temporal_mean(x, input_length, mask)
    return m.mean(dim=-1) if ndim == 4 else m


class _ErrLoss(nn.Module):
    def __init__(self, weight: Optional[Sequence[float]] = None, reduction: str = "mean", ndim: int = 3):
        super().__init__()
        if reduction != "mean":
            raise ValueError("only reduction='mean' is supported")
        if ndim not in (3, 4):
            raise ValueError("ndim must be 3 (signals) or 4 (spectrograms)")
        self.ndim = ndim
        if weight is not None:
            w = torch.tensor(list(weight), dtype=torch.float32)
            if bool((w <= 0).any()) or abs(float(w.sum()) - 1) > 1e-6:
                raise ValueError(f"channel weights must be positive and sum to one, got {list(weight)}")
            self.register_buffer("weight", w)
        else:
            self.weight = None

    def _err(self, d: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, estimate, target, input_length=None, mask=None):
        d = self._err(estimate - target)
        per = calculate_mean(d, input_length, mask, self.ndim)                # [B, C]
        per = (per * self.weight.to(per)).sum(-1) if self.weight is not None else per.mean(-1)
        return per.mean()


class MSELoss(_ErrLoss):
    def _err(self, d):
        return d.abs().pow(2) if d.is_complex() else d.pow(2)


class MAELoss(_ErrLoss):
    def _err(self, d):
        return d.abs()


class CombinedLoss(nn.Module):
    """``sisnr_weight * (-SI-SDR) + spectral_weight * |log-magnitude difference| + asr_weight * L1(features(est), features(tgt))``.
    ``feature_extractor(audio [B, T], lengths) -> features`` is a frozen model (typically an ASR encoder); its parameters get no
    gradient but the gradient flows through it to the estimate."""

    def __init__(self, sample_rate: int = 16000, fft_length: int = 1920, hop_length: int = 480, num_mels: int = 320, sisnr_loss_weight: float = 1.0,
                 spectral_loss_weight: float = 15.0, asr_loss_weight: float = 1.0, feature_extractor: Optional[Callable] = None, use_mel_spec: bool = True):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        self.n_fft, self.hop = fft_length, hop_length
        self.w = (sisnr_loss_weight, spectral_loss_weight, asr_loss_weight)
        object.__setattr__(self, "_features", feature_extractor)
        fb = torch.as_tensor(mel_filterbank(sample_rate, fft_length, num_mels), dtype=torch.float32) if use_mel_spec else None
        self.register_buffer("fb", fb, persistent=False) if fb is not None else setattr(self, "fb", None)

    def _spec(self, x):
        w = torch.hann_window(self.n_fft, device=x.device)
        s = torch.stft(x.float(), self.n_fft, self.hop, self.n_fft, w, return_complex=True).abs()
        return torch.matmul(self.fb.to(s), s) if self.fb is not None else s

    def forward(self, estimate: torch.Tensor, target: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        """Signals ``[B, 1, T]`` or ``[B, T]``."""
        e = estimate.squeeze(1) if estimate.dim() == 3 else estimate
        t = target.squeeze(1) if target.dim() == 3 else target
        loss = e.new_zeros(())
        if self.w[0]:
            loss = loss - self.w[0] * si_sdr(e.unsqueeze(1), t.unsqueeze(1), input_length).mean() / 100.0     # dB -> a scale comparable to the others
        if self.w[1]:
            loss = loss + self.w[1] * (torch.log1p(self._spec(e)) - torch.log1p(self._spec(t))).abs().mean()
        if self.w[2] and self._features is not None:
            lens = input_length if input_length is not None else torch.full((e.shape[0],), e.shape[1], device=e.device)
            with torch.no_grad():
                ft = self._features(t, lens)
            fe = self._features(e, lens)
            loss = loss + self.w[2] * F.l1_loss(fe, ft)
        return loss

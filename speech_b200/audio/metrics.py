"""Audio quality metrics: a wrapper that selects a channel, trims to the valid length and accumulates over batches and ranks; the
intrusive metrics SDR / SI-SDR / SNR / STOI computed here; and reference-free quality estimation (STOI, PESQ, SI-SDR and MOS
predicted from the signal alone) through a small estimator network or any injected one.

References: ``audio/metrics/audio.py`` (``AudioMetricWrapper``), ``audio/metrics/squim.py`` (``SquimMOSMetric``,
``SquimObjectiveMetric``, which wrap pre-trained estimators of an external package; here the estimator is a module of this package
that is trained with ``QualityEstimator.training_loss`` against the intrusive metrics, or any callable).
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .modules import sdr

__all__ = ["AudioMetricWrapper", "QualityEstimator", "SquimMOSMetric", "SquimObjectiveMetric", "snr", "stoi"]


def snr(estimate: torch.Tensor, target: torch.Tensor, input_length: Optional[torch.Tensor] = None, eps: float = 1e-8) -> torch.Tensor:
    return sdr(estimate, target, input_length, scale_invariant=False, remove_mean=False, eps=eps)


# ------------------------------------------------------------------------------------------------ STOI
def _third_octave_bands(fs: int, n_fft: int, n_bands: int, f_min: float) -> torch.Tensor:
    f = torch.linspace(0, fs, n_fft + 1)[: n_fft // 2 + 1]
    k = torch.arange(n_bands, dtype=torch.float32)
    cf = 2.0 ** (k / 3.0) * f_min
    lo, hi = cf * 2 ** (-1 / 6), cf * 2 ** (1 / 6)
    obm = torch.zeros(n_bands, f.numel())
    for i in range(n_bands):
        a = int((f - lo[i]).pow(2).argmin())
        b = int((f - hi[i]).pow(2).argmin())
        obm[i, a:b] = 1.0
    return obm


def _resample_linear(x: torch.Tensor, fs_in: int, fs_out: int) -> torch.Tensor:
    if fs_in == fs_out:
        return x
    n = int(round(x.shape[-1] * fs_out / fs_in))
    return F.interpolate(x.reshape(-1, 1, x.shape[-1]), size=n, mode="linear", align_corners=False).reshape(*x.shape[:-1], n)


def stoi(estimate: torch.Tensor, target: torch.Tensor, fs: int = 16000, extended: bool = False) -> torch.Tensor:
    """Short-time objective intelligibility of ``estimate`` [T] against the clean ``target`` [T], in [-1, 1] (higher is more
    intelligible): both signals go to 10 kHz, silent frames (40 dB below the loudest clean frame) are removed, 512-point spectra
    are pooled into 15 one-third octave bands from 150 Hz, and within 384 ms segments the degraded envelope is normalised, clipped
    at -15 dB signal-to-distortion and correlated with the clean envelope; the mean correlation is the score.  ``extended`` uses
    row- and column-normalised segments without clipping (ESTOI)."""
    FS, NF, NFFT, NB, FMIN, N, BETA = 10000, 256, 512, 15, 150.0, 30, -15.0
    x, y = _resample_linear(target.float(), fs, FS), _resample_linear(estimate.float(), fs, FS)
    T = min(x.shape[-1], y.shape[-1])
    x, y = x[..., :T], y[..., :T]
    w = torch.hann_window(NF + 2, periodic=False, device=x.device)[1:-1]
    hop = NF // 2
    if T < NF:
        return x.new_tensor(1e-5)
    xf, yf = x.unfold(-1, NF, hop) * w, y.unfold(-1, NF, hop) * w
    # drop frames whose clean energy is more than 40 dB under the loudest one
    e = 20 * torch.log10(xf.norm(dim=-1) + 1e-10)
    keep = e > e.max() - 40.0
    xf, yf = xf[keep], yf[keep]
    if xf.shape[0] < N:
        return x.new_tensor(1e-5)
    X = torch.fft.rfft(xf, NFFT).abs().pow(2)
    Y = torch.fft.rfft(yf, NFFT).abs().pow(2)
    obm = _third_octave_bands(FS, NFFT, NB, FMIN).to(x.device)
    Xb, Yb = (X @ obm.t()).sqrt().t(), (Y @ obm.t()).sqrt().t()          # [bands, frames]
    xs, ys = Xb.unfold(-1, N, 1).permute(1, 0, 2), Yb.unfold(-1, N, 1).permute(1, 0, 2)   # [segments, bands, N]
    if extended:
        def rc(z):
            z = z - z.mean(-1, keepdim=True)
            z = z / (z.norm(dim=-1, keepdim=True) + 1e-10)
            z = z - z.mean(-2, keepdim=True)
            return z / (z.norm(dim=-2, keepdim=True) + 1e-10)
        return (rc(xs) * rc(ys)).sum() / (N * xs.shape[0])
    alpha = xs.norm(dim=-1, keepdim=True) / (ys.norm(dim=-1, keepdim=True) + 1e-10)
    yn = torch.minimum(ys * alpha, xs * (1 + 10 ** (-BETA / 20)))
    xc, yc = xs - xs.mean(-1, keepdim=True), yn - yn.mean(-1, keepdim=True)
    corr = (xc * yc).sum(-1) / (xc.norm(dim=-1) * yc.norm(dim=-1) + 1e-10)
    return corr.mean()


# ------------------------------------------------------------------------------------------------ wrapper
class AudioMetricWrapper:
    """Accumulates ``metric(preds, target) -> value per example`` over batches.

    ``channel``: evaluate only that channel of ``[B, C, T]`` signals (``None``: all, the metric sees ``[B, C, T]``).
    ``metric_using_batch_averaging``: the metric already returns one batch-averaged number; then examples of different length are
    evaluated one by one, since trimming cannot be done inside a batch.  ``compute()`` is the mean over all examples of all ranks
    (sum and count are all-reduced when a process group is initialised)."""

    def __init__(self, metric: Callable[..., torch.Tensor], channel: Optional[int] = None, metric_using_batch_averaging: bool = False,
                 needs_length: bool = False):
        self.metric, self.channel, self.batch_avg, self.needs_length = metric, channel, metric_using_batch_averaging, needs_length
        self.reset()

    def reset(self):
        self._sum, self._n = 0.0, 0

    def _select(self, p, t):
        if self.channel is None:
            return p, t
        if p.dim() != 3 or t.dim() != 3:
            raise RuntimeError(f"a channel can only be selected from [B, C, T] signals, got {tuple(p.shape)} and {tuple(t.shape)}")
        if self.channel >= p.shape[1] or self.channel >= t.shape[1]:
            raise RuntimeError(f"channel {self.channel} is out of range for {tuple(p.shape)} / {tuple(t.shape)}")
        return p[:, self.channel], t[:, self.channel]

    def update(self, preds: torch.Tensor, target: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        p, t = self._select(preds, target)
        if input_length is None or self.needs_length:
            v = self.metric(p, t, input_length) if self.needs_length else self.metric(p, t)
            v = torch.as_tensor(v, dtype=torch.float32)
            if self.batch_avg or v.dim() == 0:
                self._sum += float(v) * p.shape[0]
                self._n += p.shape[0]
            else:
                self._sum += float(v.float().sum())
                self._n += v.numel()
            return
        for b in range(p.shape[0]):                                  # trim every example to its own length
            n = int(input_length[b])
            v = torch.as_tensor(self.metric(p[b:b + 1, ..., :n], t[b:b + 1, ..., :n]), dtype=torch.float32)
            self._sum += float(v.mean())
            self._n += 1

    def compute(self) -> torch.Tensor:
        s = torch.tensor([self._sum, float(self._n)], dtype=torch.float64)
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.distributed.get_backend() == "nccl" else torch.device("cpu")
            s = s.to(dev)
            torch.distributed.all_reduce(s)
            s = s.cpu()
        return (s[0] / s[1].clamp(min=1)).float()

    def __call__(self, preds, target, input_length=None) -> torch.Tensor:
        """Value of this batch alone; the running state is updated too."""
        before = (self._sum, self._n)
        self.update(preds, target, input_length)
        return torch.tensor((self._sum - before[0]) / max(1, self._n - before[1]))


# ------------------------------------------------------------------------------------------------ reference-free estimation
class QualityEstimator(nn.Module):
    """Predicts STOI, PESQ, SI-SDR (and MOS) of a 16 kHz signal without its clean reference: a strided 1-D convolutional encoder,
    a few Transformer layers over frames, attention pooling, and one bounded head per quantity (STOI in [0, 1], PESQ in
    [1, 4.64], SI-SDR unbounded in dB, MOS in [1, 5]).  ``training_loss`` regresses the heads on labels computed with the intrusive
    metrics on simulated degradations."""

    ranges = {"stoi": (0.0, 1.0), "pesq": (1.0, 4.64), "si_sdr": None, "mos": (1.0, 5.0)}

    def __init__(self, d_model: int = 128, n_layers: int = 3, n_heads: int = 4, kernel: int = 400, stride: int = 160):
        super().__init__()
        self.enc = nn.Sequential(nn.Conv1d(1, d_model, kernel, stride=stride, padding=kernel // 2), nn.GELU(), nn.Conv1d(d_model, d_model, 3, padding=1), nn.GELU())
        self.layers = nn.ModuleList([nn.TransformerEncoderLayer(d_model, n_heads, 4 * d_model, 0.0, batch_first=True, norm_first=True) for _ in range(n_layers)])
        self.pool = nn.Linear(d_model, 1)
        self.heads = nn.ModuleDict({k: nn.Sequential(nn.Linear(d_model, d_model), nn.GELU(), nn.Linear(d_model, 1)) for k in self.ranges})

    def forward(self, audio: torch.Tensor) -> Dict[str, torch.Tensor]:
        x = audio.float()
        x = x / (x.abs().amax(dim=-1, keepdim=True) + 1e-8)
        h = self.enc(x.unsqueeze(1)).transpose(1, 2)
        for l in self.layers:
            h = l(h)
        a = torch.softmax(self.pool(h), dim=1)
        z = (a * h).sum(1)
        out = {}
        for k, head in self.heads.items():
            v = head(z).squeeze(-1)
            r = self.ranges[k]
            out[k] = v if r is None else r[0] + (r[1] - r[0]) * torch.sigmoid(v)
        return out

    def training_loss(self, audio: torch.Tensor, labels: Dict[str, torch.Tensor]) -> torch.Tensor:
        pred = self(audio)
        loss = 0.0
        for k, y in labels.items():
            r = self.ranges[k]
            scale = 1.0 if r is not None else 0.1                      # dB targets are an order of magnitude larger
            loss = loss + F.l1_loss(pred[k] * scale / ((r[1] - r[0]) if r else 1.0), y.float() * scale / ((r[1] - r[0]) if r else 1.0))
        return loss


class _EstimatedMetric:
    fs_model = 16000

    def __init__(self, fs: int, estimator: Optional[Callable[[torch.Tensor], Dict[str, torch.Tensor]]] = None):
        self.fs = fs
        self.estimator = estimator if estimator is not None else QualityEstimator().eval()
        self._sum, self._n = 0.0, 0

    def reset(self):
        self._sum, self._n = 0.0, 0

    def _prep(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 2:
            raise ValueError(f"expected [B, T] signals, got {tuple(x.shape)}")
        return _resample_linear(x, self.fs, self.fs_model)

    def compute(self) -> torch.Tensor:
        return torch.tensor(self._sum / max(1, self._n))

    def state_dict(self, *a, **k):
        return {}                                                     # the estimator's weights are not part of a model checkpoint


class SquimObjectiveMetric(_EstimatedMetric):
    """Reference-free estimate of ``metric`` in {"stoi", "pesq", "si_sdr"} averaged over examples; ``target`` is ignored."""

    def __init__(self, fs: int, metric: str, estimator=None):
        if metric not in ("stoi", "pesq", "si_sdr"):
            raise ValueError(f"unknown metric {metric!r}: expected 'stoi', 'pesq' or 'si_sdr'")
        super().__init__(fs, estimator)
        self.metric = metric

    @torch.no_grad()
    def update(self, preds: torch.Tensor, target: Any = None):
        v = self.estimator(self._prep(preds))[self.metric]
        self._sum += float(v.sum())
        self._n += v.numel()


class SquimMOSMetric(_EstimatedMetric):
    """Estimated mean opinion score of ``preds``; estimators that take a non-matching clean reference get ``target`` as second
    argument (``estimator(preds, target)``), the built-in one looks at ``preds`` alone."""

    @torch.no_grad()
    def update(self, preds: torch.Tensor, target: Optional[torch.Tensor] = None):
        p = self._prep(preds)
        try:
            out = self.estimator(p, self._prep(target)) if target is not None and not isinstance(self.estimator, QualityEstimator) else self.estimator(p)
        except TypeError:
            out = self.estimator(p)
        v = out["mos"] if isinstance(out, dict) else out
        self._sum += float(v.sum())
        self._n += v.numel()

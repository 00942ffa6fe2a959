"""Multichannel front-end modules: spatial features, channel-mixing blocks, flexible-channel mask estimator, guided source
separation (cACGMM), parametric multichannel Wiener filter, reference-channel estimator, WPE dereverberation, mixture
consistency, and the masked-patch pretext masker.

Shapes follow the audio collection: complex spectrograms are ``[B, C, F, N]`` (batch, channels, sub-bands, frames); lengths
count frames.  References (behaviour, not code): ``audio/modules/features.py`` (``SpectrogramToMultichannelFeatures``),
``audio/modules/masking.py`` (``MaskEstimatorFlexChannels`` :236, ``MaskEstimatorGSS`` :440, ``MaskBasedDereverbWPE`` :960),
``audio/parts/submodules/multichannel.py`` (``ChannelAugment``, ``TransformAverageConcatenate``, ``TransformAttendConcatenate``,
``ChannelAveragePool``, ``ChannelAttentionPool``, ``ParametricMultichannelWienerFilter``, ``ReferenceChannelEstimatorSNR``,
``WPEFilter``), ``audio/modules/projections.py``, ``audio/modules/ssl_pretrain_masking.py``.
"""
from __future__ import annotations

import math
import random
from typing import List, Optional, Tuple

import torch
from torch import nn

from ..core.module import NeuralModule


def _frame_mask(lens: Optional[torch.Tensor], N: int, device) -> Optional[torch.Tensor]:
    return None if lens is None else torch.arange(N, device=device)[None, :] < lens.to(device)[:, None]


# ---------------------------------------------------------------------------------------------- features
class SpectrogramToMultichannelFeatures(NeuralModule):
    """Magnitude (optionally reduced over channels) and inter-channel phase differences of a multichannel spectrogram.

    ``mag_reduction``: ``None`` keeps one magnitude per channel, ``abs_mean`` / ``mean_abs`` / ``rms`` reduce over channels.
    IPD of channel c is the phase of ``x_c`` relative to the channel mean, wrapped to ``(-pi, pi]``.  Output: real
    ``[B, C', F', N]`` where ``F'`` stacks magnitude and IPD along the feature axis."""

    def __init__(self, num_subbands: int, num_input_channels: Optional[int] = None, mag_reduction: Optional[str] = None,
                 mag_power: Optional[float] = None, use_ipd: bool = False, mag_normalization: Optional[str] = None,
                 ipd_normalization: Optional[str] = None, eps: float = 1e-8):
        super().__init__()
        if mag_reduction not in (None, "abs_mean", "mean_abs", "rms"):
            raise ValueError(f"unknown mag_reduction '{mag_reduction}'")
        for n in (mag_normalization, ipd_normalization):
            if n not in (None, "mean", "mean_var"):
                raise ValueError(f"unknown normalization '{n}'")
        self.F, self.C = num_subbands, num_input_channels
        self.mag_reduction, self.mag_power, self.use_ipd = mag_reduction, mag_power, use_ipd
        self.mag_norm, self.ipd_norm, self.eps = mag_normalization, ipd_normalization, eps

    @property
    def num_features(self) -> int:
        return self.F * (2 if self.use_ipd else 1)

    @property
    def num_channels(self) -> int:
        if self.use_ipd or self.mag_reduction is None:
            return self.C
        return 1

    @staticmethod
    def _normalize(x: torch.Tensor, mask: Optional[torch.Tensor], kind: Optional[str], eps: float) -> torch.Tensor:
        """Statistics over valid frames, per (batch, channel, feature)."""
        if kind is None:
            return x
        if mask is None:
            mean = x.mean(dim=-1, keepdim=True)
            var = x.var(dim=-1, keepdim=True, unbiased=False)
        else:
            m = mask[:, None, None, :].to(x.dtype)
            n = m.sum(dim=-1, keepdim=True).clamp(min=1)
            mean = (x * m).sum(dim=-1, keepdim=True) / n
            var = (((x - mean) * m) ** 2).sum(dim=-1, keepdim=True) / n
        x = x - mean
        if kind == "mean_var":
            x = x / (var.sqrt() + eps)
        return x if mask is None else x * mask[:, None, None, :].to(x.dtype)

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        B, C, F, N = input.shape
        mask = _frame_mask(input_length, N, input.device)
        if self.mag_reduction is None:
            mag = input.abs()
        elif self.mag_reduction == "abs_mean":
            mag = input.mean(dim=1, keepdim=True).abs()
        elif self.mag_reduction == "mean_abs":
            mag = input.abs().mean(dim=1, keepdim=True)
        else:
            mag = input.abs().pow(2).mean(dim=1, keepdim=True).sqrt()
        if self.mag_power is not None:
            mag = mag.pow(self.mag_power)
        mag = self._normalize(mag, mask, self.mag_norm, self.eps)
        feats = mag
        if self.use_ipd:
            mean = input.mean(dim=1, keepdim=True)
            ipd = torch.angle(input) - torch.angle(mean)
            ipd = torch.remainder(ipd + math.pi, 2 * math.pi) - math.pi
            ipd = self._normalize(ipd, mask, self.ipd_norm, self.eps)
            feats = torch.cat([mag.expand(B, C, F, N), ipd], dim=2)
        return feats, input_length


class ChannelAugment(NeuralModule):
    """Training-time augmentation: keep a random subset of ``[num_channels_min, num_channels_max]`` channels, in random order
    when ``permute_channels``."""

    def __init__(self, permute_channels: bool = True, num_channels_min: int = 1, num_channels_max: Optional[int] = None,
                 rng: Optional[random.Random] = None):
        super().__init__()
        self.permute, self.lo, self.hi = permute_channels, num_channels_min, num_channels_max
        self.rng = rng or random.Random()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        C = input.shape[1]
        hi = C if self.hi is None else min(self.hi, C)
        k = self.rng.randint(min(self.lo, hi), hi)
        idx = list(range(C))
        if self.permute:
            self.rng.shuffle(idx)
        return input[:, idx[:k]]


# ---------------------------------------------------------------------------------------------- channel blocks
class TransformAverageConcatenate(NeuralModule):
    """Per-channel transform concatenated with the channel average of a second transform: every channel sees a summary of the
    others, and the block is equivariant to channel permutations.  ``[B, C, D_in, N] -> [B, C, D_out, N]``."""

    def __init__(self, in_features: int, out_features: Optional[int] = None):
        super().__init__()
        out_features = out_features or in_features
        if out_features % 2:
            raise ValueError("out_features must be even")
        self.own = nn.Sequential(nn.Linear(in_features, out_features // 2), nn.ReLU())
        self.shared = nn.Sequential(nn.Linear(in_features, out_features // 2), nn.ReLU())

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x = input.permute(0, 1, 3, 2)                            # [B, C, N, D]
        a = self.own(x)
        s = self.shared(x).mean(dim=1, keepdim=True).expand_as(a)
        return torch.cat([a, s], dim=-1).permute(0, 1, 3, 2)


class TransformAttendConcatenate(NeuralModule):
    """As :class:`TransformAverageConcatenate`, with the average replaced by multi-head attention across channels (each
    channel queries all channels of the same frame)."""

    def __init__(self, in_features: int, out_features: Optional[int] = None, n_head: int = 4, dropout_rate: float = 0.0):
        super().__init__()
        out_features = out_features or in_features
        if out_features % 2:
            raise ValueError("out_features must be even")
        self.own = nn.Sequential(nn.Linear(in_features, out_features // 2), nn.ReLU())
        self.shared = nn.Sequential(nn.Linear(in_features, out_features // 2), nn.ReLU())
        self.attn = nn.MultiheadAttention(out_features // 2, n_head, dropout=dropout_rate, batch_first=True)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        B, C, D, N = input.shape
        x = input.permute(0, 3, 1, 2)                            # [B, N, C, D]
        a = self.own(x)
        s = self.shared(x).reshape(B * N, C, -1)
        s = self.attn(s, s, s, need_weights=False)[0].view(B, N, C, -1)
        return torch.cat([a, s], dim=-1).permute(0, 2, 3, 1)


class ChannelAveragePool(NeuralModule):
    """``[B, C, D, N] -> [B, 1, D, N]`` by the mean over channels."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return input.mean(dim=1, keepdim=True)


class ChannelAttentionPool(NeuralModule):
    """Attention across channels followed by the mean: ``[B, C, D, N] -> [B, 1, D, N]``."""

    def __init__(self, in_features: int, n_head: int = 1, dropout_rate: float = 0.0):
        super().__init__()
        self.attn = nn.MultiheadAttention(in_features, n_head, dropout=dropout_rate, batch_first=True)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        B, C, D, N = input.shape
        x = input.permute(0, 3, 1, 2).reshape(B * N, C, D)
        y = self.attn(x, x, x, need_weights=False)[0].mean(dim=1)
        return y.view(B, N, D).permute(0, 2, 1).unsqueeze(1)


# ---------------------------------------------------------------------------------------------- mask estimators
class MaskEstimatorFlexChannels(NeuralModule):
    """Mask estimator for any number (and order) of input channels.  Blocks alternate a *channel* block (information exchange
    between channels, permutation equivariant) and a *temporal* block (a Conformer stack applied to each channel on its own);
    channels are pooled either after block ``channel_reduction_position`` or at the end; a linear + sigmoid head gives
    ``num_outputs`` masks ``[B, M, F, N]``."""

    def __init__(self, num_outputs: int, num_subbands: int, num_blocks: int, channel_reduction_position: int = -1,
                 channel_reduction_type: str = "attention", channel_block_type: str = "transform_attend_concatenate",
                 temporal_block_type: str = "conformer_encoder", temporal_block_num_layers: int = 5, temporal_block_num_heads: int = 4,
                 temporal_block_dimension: int = 128, temporal_block_self_attention_model: str = "rel_pos",
                 temporal_block_att_context_size: Optional[List[int]] = None, num_input_channels: Optional[int] = None,
                 mag_reduction: Optional[str] = "abs_mean", mag_power: Optional[float] = None, use_ipd: bool = True,
                 mag_normalization: Optional[str] = None, ipd_normalization: Optional[str] = None):
        super().__init__()
        from ..modules.conformer_encoder import ConformerEncoder

        if temporal_block_type != "conformer_encoder":
            raise ValueError(f"unknown temporal block '{temporal_block_type}'")
        self.features = SpectrogramToMultichannelFeatures(num_subbands, num_input_channels, mag_reduction, mag_power, use_ipd,
                                                         mag_normalization, ipd_normalization)
        D = temporal_block_dimension
        self.reduce_at = num_blocks if channel_reduction_position == -1 else channel_reduction_position
        if not 0 <= self.reduce_at <= num_blocks:
            raise ValueError("channel_reduction_position out of range")
        self.channel_blocks, self.temporal_blocks = nn.ModuleList(), nn.ModuleList()
        d_in = self.features.num_features
        for b in range(num_blocks):
            if b < self.reduce_at:
                if channel_block_type == "transform_average_concatenate":
                    cb = TransformAverageConcatenate(d_in, D)
                elif channel_block_type == "transform_attend_concatenate":
                    cb = TransformAttendConcatenate(d_in, D)
                else:
                    raise ValueError(f"unknown channel block '{channel_block_type}'")
            else:
                cb = nn.Linear(d_in, D)                            # channels already pooled: a plain projection
            self.channel_blocks.append(cb)
            self.temporal_blocks.append(ConformerEncoder(
                feat_in=D, n_layers=temporal_block_num_layers, d_model=D, subsampling="stacking", subsampling_factor=1, n_heads=temporal_block_num_heads, self_attention_model=temporal_block_self_attention_model,
                att_context_size=temporal_block_att_context_size, conv_kernel_size=9, conv_norm_type="layer_norm", dropout=0.0,
                dropout_pre_encoder=0.0, dropout_emb=0.0, dropout_att=0.0, ff_expansion_factor=4, feat_out=D))
            d_in = D
        if channel_reduction_type == "average":
            self.pool = ChannelAveragePool()
        elif channel_reduction_type == "attention":
            self.pool = ChannelAttentionPool(D if self.reduce_at > 0 else self.features.num_features)
        else:
            raise ValueError(f"unknown channel reduction '{channel_reduction_type}'")
        self.head = nn.Linear(D if num_blocks > 0 else self.features.num_features, num_outputs * num_subbands)
        self.M, self.F = num_outputs, num_subbands

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        x, _ = self.features(input, input_length)                   # [B, C, D, N]
        B, _, _, N = x.shape
        if input_length is None:
            input_length = torch.full((B,), N, dtype=torch.long, device=x.device)
        for b, (cb, tb) in enumerate(zip(self.channel_blocks, self.temporal_blocks)):
            if b == self.reduce_at:
                x = self.pool(x)
            if isinstance(cb, nn.Linear):
                x = cb(x.permute(0, 1, 3, 2)).permute(0, 1, 3, 2)
            else:
                x = cb(x)
            C = x.shape[1]
            y, _ = tb(audio_signal=x.reshape(B * C, x.shape[2], N), length=input_length.repeat_interleave(C))
            x = y.view(B, C, -1, N)
        if self.reduce_at >= len(self.channel_blocks):
            x = self.pool(x)                                         # reduction at the end
        m = torch.sigmoid(self.head(x[:, 0].transpose(1, 2))).view(B, N, self.M, self.F).permute(0, 2, 3, 1)
        fm = _frame_mask(input_length, N, m.device)
        return m * fm[:, None, None, :].to(m.dtype), input_length


class MaskEstimatorGSS(NeuralModule):
    """Guided source separation: masks from a complex angular-central Gaussian mixture model fitted by EM in every sub-band,
    with the sources' time activity as a prior on the posteriors.

    Model: unit-norm observations ``z_t = x_t / |x_t|``; source n has a Hermitian shape matrix ``B_n``; likelihood
    ``p(z | n) ∝ det(B_n)^-1 (z^H B_n^-1 z)^-C``.  E-step: ``γ_{n,t} ∝ a_{n,t} p(z_t | n)``.  M-step:
    ``B_n = C Σ_t γ_{n,t} z_t z_t^H / (z_t^H B_n^-1 z_t) / Σ_t γ_{n,t}``.  Input ``[B, C, F, N]`` complex and activity
    ``[B, S, N]``; output posteriors ``[B, S, F, N]``."""

    def __init__(self, num_iterations: int = 3, eps: float = 1e-8, dtype: torch.dtype = torch.cdouble):
        super().__init__()
        if num_iterations < 1:
            raise ValueError("num_iterations must be positive")
        self.iters, self.eps, self.dtype = num_iterations, eps, dtype

    def normalize(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        return x / (torch.linalg.vector_norm(x, dim=dim, keepdim=True) + self.eps)

    @torch.no_grad()
    def forward(self, input: torch.Tensor, activity: torch.Tensor):
        B, C, F, N = input.shape
        S = activity.shape[1]
        if activity.shape[-1] != N:
            raise ValueError("activity must have one value per frame")
        z = self.normalize(input.to(self.dtype), dim=1).permute(0, 2, 3, 1)                # [B, F, N, C]
        rdt = z.real.dtype
        a = activity.to(rdt).unsqueeze(1).expand(B, F, S, N)                                 # [B, F, S, N]
        gamma = a / a.sum(dim=2, keepdim=True).clamp(min=self.eps)
        zz = z.unsqueeze(-1) * z.conj().unsqueeze(-2)                                        # [B, F, N, C, C]
        eye = torch.eye(C, dtype=self.dtype, device=input.device)
        quad = torch.ones(B, F, S, N, dtype=rdt, device=input.device)                        # z^H B^-1 z, 1 for B = I
        for _ in range(self.iters):
            w = gamma / quad.clamp(min=self.eps)                                             # [B, F, S, N]
            Bn = C * torch.einsum("bfsn,bfncd->bfscd", w.to(self.dtype), zz) / gamma.sum(-1).clamp(min=self.eps)[..., None, None]
            Bn = 0.5 * (Bn + Bn.conj().transpose(-1, -2))
            tr = Bn.diagonal(dim1=-2, dim2=-1).real.sum(-1)
            Bn = Bn + (1e-6 * tr.clamp(min=self.eps) / C)[..., None, None] * eye
            Binv = torch.linalg.inv(Bn)
            quad = torch.einsum("bfnc,bfscd,bfnd->bfsn", z.conj(), Binv, z).real.clamp(min=self.eps)
            logdet = torch.linalg.slogdet(Bn)[1].real                                        # [B, F, S]
            loglik = -logdet.unsqueeze(-1) - C * torch.log(quad)
            logpost = loglik + torch.log(a.clamp(min=self.eps))
            gamma = torch.softmax(logpost, dim=2) * (a.sum(dim=2, keepdim=True) > 0)
        return gamma.permute(0, 2, 1, 3).to(input.real.dtype)


# ---------------------------------------------------------------------------------------------- filters
class ParametricMultichannelWienerFilter(NeuralModule):
    """Speech-distortion-weighted multichannel Wiener filter with a reference selection.  ``rank='full'``:
    ``W = (Φ_s + β Φ_n)^-1 Φ_s``; ``rank='one'`` (speech covariance of rank one): ``W = Φ_n^-1 Φ_s / (β + tr(Φ_n^-1 Φ_s))``.
    β = 0 keeps the target undistorted (MVDR), β = 1 is the Wiener filter, larger β trades distortion for noise reduction.
    ``ref_channel``: an index, ``'max_snr'`` (:class:`ReferenceChannelEstimatorSNR`) or ``None`` (average of all references)."""

    def __init__(self, beta: float = 1.0, rank: str = "one", postfilter: Optional[str] = None, ref_channel=0, ref_hard: bool = True,
                 ref_hard_use_grad: bool = True, ref_subband_weighting: bool = False, num_subbands: Optional[int] = None,
                 diag_reg: Optional[float] = 1e-6, eps: float = 1e-8):
        super().__init__()
        if rank not in ("one", "full"):
            raise ValueError("rank must be 'one' or 'full'")
        if postfilter not in (None, "ban"):
            raise ValueError("postfilter must be None or 'ban'")
        self.beta, self.rank, self.postfilter, self.reg, self.eps = beta, rank, postfilter, diag_reg, eps
        self.ref_channel = ref_channel
        self.ref_estimator = ReferenceChannelEstimatorSNR(ref_hard, ref_hard_use_grad, ref_subband_weighting, num_subbands, eps) \
            if ref_channel == "max_snr" else None

    def _regularise(self, psd: torch.Tensor) -> torch.Tensor:
        if self.reg is None:
            return psd
        C = psd.shape[-1]
        tr = psd.diagonal(dim1=-2, dim2=-1).real.sum(-1)
        return psd + (self.reg * tr + self.eps)[..., None, None] * torch.eye(C, dtype=psd.dtype, device=psd.device)

    def forward(self, input: torch.Tensor, psd_s: torch.Tensor, psd_n: torch.Tensor) -> torch.Tensor:
        """input ``[B, C, F, N]``, covariances ``[B, F, C, C]`` -> ``[B, 1, F, N]``."""
        if self.rank == "one":
            # rank-one speech model: W = Φ_n^-1 Φ_s / (β + tr(Φ_n^-1 Φ_s)); β = 0 is the distortionless (MVDR) solution
            num = torch.linalg.solve(self._regularise(psd_n), psd_s)
            lam = num.diagonal(dim1=-2, dim2=-1).sum(-1)[..., None, None]
            W = num / (self.beta + lam + self.eps)                                          # [B, F, C, C]; column r: reference r
        else:
            W = torch.linalg.solve(self._regularise(psd_s + self.beta * psd_n), psd_s)
        if self.postfilter == "ban":
            # blind analytic normalisation per candidate reference
            num = torch.sqrt(torch.einsum("bfcr,bfcd,bfde,bfer->bfr", W.conj(), psd_n, psd_n, W).real.clamp(min=0) / W.shape[-1])
            den = torch.einsum("bfcr,bfcd,bfdr->bfr", W.conj(), psd_n, W).real.clamp(min=self.eps)
            W = W * (num / den).unsqueeze(-2)
        if isinstance(self.ref_channel, int):
            w = W[..., self.ref_channel]
        elif self.ref_estimator is not None:
            ref = self.ref_estimator(W, psd_s, psd_n)                                       # [B, F, C] or [B, 1, C] weights
            w = torch.einsum("bfcr,bfr->bfc", W, ref.to(W.dtype))
        else:
            w = W.mean(dim=-1)
        return torch.einsum("bfc,bcfn->bfn", w.conj(), input).unsqueeze(1)


class ReferenceChannelEstimatorSNR(NeuralModule):
    """Reference weights that favour the candidate whose filter gives the best output SNR.  Hard selection takes the arg-max
    (optionally with a straight-through gradient); soft selection is a softmax over the SNRs in dB.  With
    ``ref_subband_weighting`` the per-band SNRs are combined with learned band weights before the selection."""

    def __init__(self, hard: bool = True, hard_use_grad: bool = True, subband_weighting: bool = False, num_subbands: Optional[int] = None,
                 eps: float = 1e-8):
        super().__init__()
        self.hard, self.hard_use_grad, self.eps = hard, hard_use_grad, eps
        if subband_weighting:
            if num_subbands is None:
                raise ValueError("num_subbands is needed for sub-band weighting")
            self.weight = nn.Parameter(torch.zeros(num_subbands))
        else:
            self.weight = None

    def forward(self, W: torch.Tensor, psd_s: torch.Tensor, psd_n: torch.Tensor) -> torch.Tensor:
        ps = torch.einsum("bfcr,bfcd,bfdr->bfr", W.conj(), psd_s, W).real
        pn = torch.einsum("bfcr,bfcd,bfdr->bfr", W.conj(), psd_n, W).real
        if self.weight is not None:
            wts = torch.softmax(self.weight, dim=0).view(1, -1, 1)
            ps, pn = (ps * wts).sum(1, keepdim=True), (pn * wts).sum(1, keepdim=True)
        else:
            ps, pn = ps.sum(1, keepdim=True), pn.sum(1, keepdim=True)
        snr_db = 10 * torch.log10(ps.clamp(min=self.eps) / pn.clamp(min=self.eps))          # [B, 1, C]
        soft = torch.softmax(snr_db, dim=-1)
        if not self.hard:
            return soft.expand(-1, W.shape[1], -1)
        hard = torch.nn.functional.one_hot(snr_db.argmax(dim=-1), snr_db.shape[-1]).to(soft.dtype)
        out = hard + soft - soft.detach() if self.hard_use_grad else hard
        return out.expand(-1, W.shape[1], -1)


class WPEFilter(NeuralModule):
    """Weighted prediction error dereverberation for one iteration: the late reverberation of every channel is predicted from
    ``filter_length`` past frames (``prediction_delay`` frames back) of all channels by a filter that minimises the
    power-weighted residual, and subtracted.  ``G = (Σ_t x̃_t x̃_t^H / λ_t)^-1 (Σ_t x̃_t x_t^H / λ_t)``, ``y_t = x_t - G^H x̃_t``."""

    def __init__(self, filter_length: int, prediction_delay: int, diag_reg: Optional[float] = 1e-6, eps: float = 1e-8):
        super().__init__()
        self.K, self.D, self.reg, self.eps = filter_length, prediction_delay, diag_reg, eps

    def convtensor(self, x: torch.Tensor) -> torch.Tensor:
        """``[B, C, F, N] -> [B, C, F, N, K]``: entry k of frame t is ``x[t - D - k]`` (zero before the start)."""
        N = x.shape[-1]
        pad = torch.nn.functional.pad(x, (self.D + self.K - 1, 0))
        return torch.stack([pad[..., self.K - 1 - k: self.K - 1 - k + N] for k in range(self.K)], dim=-1)

    def forward(self, input: torch.Tensor, power: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        """``power`` ``[B, F, N]``: the (estimated) power of the desired signal per frame."""
        B, C, F, N = input.shape
        w = 1.0 / power.clamp(min=self.eps)
        fm = _frame_mask(input_length, N, input.device)
        if fm is not None:
            w = w * fm[:, None, :].to(w.dtype)
        xt = self.convtensor(input).permute(0, 2, 3, 1, 4).reshape(B, F, N, C * self.K)      # [B, F, N, CK]
        xw = xt * w.unsqueeze(-1).to(xt.dtype)
        R = torch.einsum("bfni,bfnj->bfij", xw, xt.conj())
        P = torch.einsum("bfni,bfnc->bfic", xw, input.permute(0, 2, 3, 1).conj())
        if self.reg is not None:
            tr = R.diagonal(dim1=-2, dim2=-1).real.sum(-1)
            R = R + (self.reg * tr + self.eps)[..., None, None] * torch.eye(C * self.K, dtype=R.dtype, device=R.device)
        G = torch.linalg.solve(R, P)                                                       # [B, F, CK, C]
        late = torch.einsum("bfni,bfic->bfnc", xt, G.conj())
        out = input - late.permute(0, 3, 1, 2)
        if fm is not None:
            out = out * fm[:, None, None, :].to(out.real.dtype)
        return out, input_length


class MaskBasedDereverbWPE(NeuralModule):
    """Iterated WPE.  The power of the desired signal is re-estimated from the current output (mean over channels of ``|y|^2``),
    optionally shaped by a mask from a neural estimator (clamped to ``[mask_min_db, mask_max_db]``)."""

    def __init__(self, filter_length: int, prediction_delay: int, num_iterations: int = 1, mask_min_db: float = -200.0,
                 mask_max_db: float = 0.0, diag_reg: Optional[float] = 1e-6, eps: float = 1e-8, dtype: torch.dtype = torch.cdouble):
        super().__init__()
        self.filter = WPEFilter(filter_length, prediction_delay, diag_reg, eps)
        self.iters, self.dtype = num_iterations, dtype
        self.mask_min, self.mask_max = 10 ** (mask_min_db / 20), 10 ** (mask_max_db / 20)

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None):
        in_dtype = input.dtype
        x = input.to(self.dtype)
        y = x
        for _ in range(self.iters):
            mag = y.abs()
            if mask is not None:
                m = mask.to(mag.dtype).clamp(self.mask_min, self.mask_max)
                mag = mag * (m if m.shape[1] == mag.shape[1] else m[:, :1])
            power = mag.pow(2).mean(dim=1)
            y, _ = self.filter(x, power, input_length)
        return y.to(in_dtype), input_length


class MixtureConsistencyProjection(NeuralModule):
    """Distribute the mismatch between the mixture and the sum of the estimates over the estimates, equally or in proportion to
    their power, so that the estimates add up to the mixture.  ``mixture [B, 1, F, N]``, ``estimate [B, M, F, N]``."""

    def __init__(self, weighting: Optional[str] = None, eps: float = 1e-8):
        super().__init__()
        if weighting not in (None, "power"):
            raise ValueError("weighting must be None or 'power'")
        self.weighting, self.eps = weighting, eps

    def forward(self, mixture: torch.Tensor, estimate: torch.Tensor) -> torch.Tensor:
        M = estimate.shape[1]
        if self.weighting is None:
            w = 1.0 / M
        else:
            p = estimate.abs().pow(2)
            w = p / (p.sum(dim=1, keepdim=True) + self.eps)
        return estimate + w * (mixture - estimate.sum(dim=1, keepdim=True))


class SSLPretrainWithMaskedPatch(NeuralModule):
    """Zero out random time patches of a spectrogram for masked-prediction pre-training: ``patch_size`` frames per patch and
    either a fixed number of patches or a fraction ``mask_fraction`` of every utterance's length."""

    def __init__(self, patch_size: int = 10, mask_fraction: float = 0.7, rng: Optional[random.Random] = None):
        super().__init__()
        if patch_size <= 0 or not 0.0 <= mask_fraction <= 1.0:
            raise ValueError("patch_size must be positive and mask_fraction within [0, 1]")
        self.patch, self.fraction = patch_size, mask_fraction
        self.rng = rng or random.Random()

    def forward(self, input_spec: torch.Tensor, length: torch.Tensor) -> torch.Tensor:
        out = input_spec.clone()
        for b in range(out.shape[0]):
            n = int(length[b])
            n_patches = n // self.patch
            k = int(math.ceil(self.fraction * n / self.patch)) if n_patches else 0
            for p in self.rng.sample(range(n_patches), min(k, n_patches)):
                out[b, ..., p * self.patch:(p + 1) * self.patch] = 0
        return out

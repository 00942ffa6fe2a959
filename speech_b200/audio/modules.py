"""Signal-processing and neural modules of the audio (enhancement / separation) collection.

* ``AudioToSpectrogram`` / ``SpectrogramToAudio`` — multichannel STFT analysis / synthesis with optional magnitude
  compression (``audio/modules/transforms.py``).
* Mask estimators and mask application: ``MaskEstimatorRNN``, ``MaskReferenceChannel``, ``MaskBasedBeamformer`` with MVDR
  (power-iteration-free closed form, reference-channel selection), ``audio/modules/masking.py``.
* Metrics / losses: SI-SDR, SDR, ``SDRLoss``, ``MSELoss`` with length masks (``audio/losses/audio.py``, ``audio/metrics``).
* Backbones: ``SpectrogramConformerUNet`` (``parts/submodules/conformer_unet.py``) and a small ``SpectrogramNCSN`` score
  network with time conditioning (the reference's NCSN++ role, ``parts/submodules/ncsnpp.py``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.module import Loss, NeuralModule


def _len_mask(lens: Optional[torch.Tensor], T: int, device) -> Optional[torch.Tensor]:
    return None if lens is None else (torch.arange(T, device=device)[None, :] < lens[:, None])


class AudioToSpectrogram(NeuralModule):
    def __init__(self, fft_length: int = 512, hop_length: int = 128, magnitude_power: float = 1.0, scale: float = 1.0):
        super().__init__()
        self.n_fft, self.hop, self.mag_power, self.scale = fft_length, hop_length, magnitude_power, scale
        self.register_buffer("window", torch.hann_window(fft_length), persistent=False)

    @property
    def num_subbands(self) -> int:
        return self.n_fft // 2 + 1

    def get_output_length(self, input_length: torch.Tensor) -> torch.Tensor:
        return torch.div(input_length, self.hop, rounding_mode="floor") + 1

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        """[B, C, T] → complex [B, C, F, N], lengths."""
        B, C, T = input.shape
        s = torch.stft(input.reshape(B * C, T).float(), self.n_fft, self.hop, self.n_fft, self.window.to(input.device), center=True,
                       pad_mode="constant", return_complex=True)
        s = s.view(B, C, *s.shape[-2:])
        if self.mag_power != 1.0:
            s = torch.polar(s.abs().clamp(min=1e-8) ** self.mag_power, s.angle())
        s = s * self.scale
        lens = self.get_output_length(input_length) if input_length is not None else None
        if lens is not None:
            s = s * _len_mask(lens, s.shape[-1], s.device).view(B, 1, 1, -1)
        return s, lens


class SpectrogramToAudio(NeuralModule):
    def __init__(self, fft_length: int = 512, hop_length: int = 128, magnitude_power: float = 1.0, scale: float = 1.0):
        super().__init__()
        self.n_fft, self.hop, self.mag_power, self.scale = fft_length, hop_length, magnitude_power, scale
        self.register_buffer("window", torch.hann_window(fft_length), persistent=False)

    def get_output_length(self, input_length: torch.Tensor) -> torch.Tensor:
        return (input_length - 1).clamp(min=0) * self.hop

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        B, C, Fq, N = input.shape
        s = input / self.scale
        if self.mag_power != 1.0:
            s = torch.polar(s.abs().clamp(min=1e-8) ** (1.0 / self.mag_power), s.angle())
        x = torch.istft(s.reshape(B * C, Fq, N), self.n_fft, self.hop, self.n_fft, self.window.to(input.device), center=True)
        x = x.view(B, C, -1)
        lens = self.get_output_length(input_length) if input_length is not None else None
        if lens is not None:
            x = x * _len_mask(lens, x.shape[-1], x.device).view(B, 1, -1)
        return x, lens


class MaskEstimatorRNN(NeuralModule):
    """Magnitude (log-compressed) of the reference channel → stacked RNN → ``num_outputs`` sigmoid masks [B, M, F, N]."""

    def __init__(self, num_outputs: int, num_subbands: int, num_features: int = 256, num_layers: int = 2, rnn_type: str = "lstm",
                 bidirectional: bool = True, num_hidden_features: Optional[int] = None):
        super().__init__()
        rnn = {"lstm": nn.LSTM, "gru": nn.GRU}[rnn_type]
        self.norm = nn.LayerNorm(num_subbands)
        self.rnn = rnn(num_subbands, num_features, num_layers, batch_first=True, bidirectional=bidirectional)
        d = num_features * (2 if bidirectional else 1)
        self.proj = nn.Linear(d, num_hidden_features or d)
        self.out = nn.ModuleList([nn.Linear(num_hidden_features or d, num_subbands) for _ in range(num_outputs)])

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None):
        mag = torch.log1p(input[:, 0].abs()).transpose(1, 2)                 # [B, N, F]
        h, _ = self.rnn(self.norm(mag))
        h = torch.relu(self.proj(h))
        masks = torch.stack([torch.sigmoid(o(h)).transpose(1, 2) for o in self.out], dim=1)
        if input_length is not None:
            masks = masks * _len_mask(input_length, masks.shape[-1], masks.device).view(-1, 1, 1, masks.shape[-1])
        return masks, input_length


class MaskReferenceChannel(NeuralModule):
    def __init__(self, ref_channel: int = 0, mask_min_db: float = -200.0, mask_max_db: float = 0.0):
        super().__init__()
        self.ref = ref_channel
        self.lo, self.hi = 10 ** (mask_min_db / 20), 10 ** (mask_max_db / 20)

    def forward(self, input: torch.Tensor, input_length, mask: torch.Tensor):
        return mask.clamp(self.lo, self.hi) * input[:, self.ref: self.ref + 1], input_length


class MaskBasedBeamformer(NeuralModule):
    """MVDR from mask-weighted spatial covariance matrices: ``w = (Φ_n^{-1} Φ_s) u / trace(Φ_n^{-1} Φ_s)``."""

    def __init__(self, ref_channel: Optional[int] = 0, filter_type: str = "mvdr_souden", diag_reg: float = 1e-6, eps: float = 1e-8,
                 mask_min_db: float = -200.0, mask_max_db: float = 0.0):
        super().__init__()
        self.ref, self.reg, self.eps = ref_channel, diag_reg, eps

    @staticmethod
    def covariance(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """x [B, C, F, N], mask [B, F, N] → [B, F, C, C]."""
        xm = x * mask.unsqueeze(1)
        psd = torch.einsum("bcfn,bdfn->bfcd", xm, x.conj())
        return psd / mask.sum(-1).clamp(min=1e-8).unsqueeze(-1).unsqueeze(-1)

    def forward(self, input: torch.Tensor, input_length, mask: torch.Tensor, mask_undesired: Optional[torch.Tensor] = None):
        """mask [B, M, F, N] (one target per output channel) → beamformed [B, M, F, N]."""
        outs = []
        C = input.shape[1]
        eye = torch.eye(C, device=input.device, dtype=input.dtype)
        for m in range(mask.shape[1]):
            ms = mask[:, m]
            mn = mask_undesired[:, m] if mask_undesired is not None else (1 - ms)
            ps, pn = self.covariance(input, ms.to(input.real.dtype)), self.covariance(input, mn.to(input.real.dtype))
            tr = pn.diagonal(dim1=-2, dim2=-1).real.sum(-1)
            pn = pn + (self.reg * tr + self.eps).unsqueeze(-1).unsqueeze(-1) * eye
            num = torch.linalg.solve(pn, ps)                                             # Φ_n^{-1} Φ_s
            trace = num.diagonal(dim1=-2, dim2=-1).sum(-1).unsqueeze(-1).unsqueeze(-1)
            W = num / (trace + self.eps)
            if self.ref is None:
                snr = (torch.einsum("bfcd,bfde,bfec->bfc", W.conj().transpose(-1, -2), ps, W).real.sum(1) /
                       torch.einsum("bfcd,bfde,bfec->bfc", W.conj().transpose(-1, -2), pn, W).real.sum(1).clamp(min=1e-8))
                ref = snr.argmax(-1)
                w = W[torch.arange(W.shape[0]), :, :, ref]
            else:
                w = W[..., self.ref]                                                     # [B, F, C]
            outs.append(torch.einsum("bfc,bcfn->bfn", w.conj(), input))
        out = torch.stack(outs, dim=1)
        if input_length is not None:
            out = out * _len_mask(input_length, out.shape[-1], out.device).view(-1, 1, 1, out.shape[-1])
        return out, input_length


# ---------------------------------------------------------------------------------------------- metrics / losses
def _masked(x: torch.Tensor, lens: Optional[torch.Tensor]) -> torch.Tensor:
    return x if lens is None else x * _len_mask(lens, x.shape[-1], x.device).view(x.shape[0], *([1] * (x.dim() - 2)), -1)


def sdr(estimate: torch.Tensor, target: torch.Tensor, input_length: Optional[torch.Tensor] = None, scale_invariant: bool = False,
        remove_mean: bool = True, eps: float = 1e-8) -> torch.Tensor:
    """Signal-to-distortion ratio in dB per [B, C]."""
    e, t = _masked(estimate.float(), input_length), _masked(target.float(), input_length)
    if remove_mean:
        n = input_length.view(-1, 1, 1).float() if input_length is not None else float(e.shape[-1])
        e = _masked(e - e.sum(-1, keepdim=True) / n, input_length)
        t = _masked(t - t.sum(-1, keepdim=True) / n, input_length)
    if scale_invariant:
        a = (e * t).sum(-1, keepdim=True) / (t.pow(2).sum(-1, keepdim=True) + eps)
        t = a * t
    return 10 * torch.log10((t.pow(2).sum(-1) + eps) / ((e - t).pow(2).sum(-1) + eps))


def si_sdr(estimate, target, input_length=None):
    return sdr(estimate, target, input_length, scale_invariant=True)


class SDRLoss(Loss):
    def __init__(self, scale_invariant: bool = False, remove_mean: bool = True, sdr_max: Optional[float] = None, eps: float = 1e-8,
                 reduction: str = "mean"):
        super().__init__()
        self.si, self.rm, self.sdr_max, self.eps = scale_invariant, remove_mean, sdr_max, eps

    def forward(self, estimate, target, input_length=None, mask=None):
        v = sdr(estimate, target, input_length, self.si, self.rm, self.eps)
        if self.sdr_max is not None:
            v = -10 * torch.log10(10 ** (-v / 10) + 10 ** (-self.sdr_max / 10))
        return -v.mean()


class MaskedMSELoss(Loss):
    def forward(self, estimate, target, input_length=None):
        d = (estimate - target)
        d = (d.abs() ** 2) if torch.is_complex(d) else d.pow(2)
        if input_length is None:
            return d.mean()
        m = _len_mask(input_length, d.shape[-1], d.device).view(d.shape[0], *([1] * (d.dim() - 2)), -1).to(d.dtype)
        return (d * m).sum() / (m.sum() * (d[0].numel() / d.shape[-1])).clamp(min=1)


# ---------------------------------------------------------------------------------------------- backbones
class _TimeEmbedding(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim
        self.mlp = nn.Sequential(nn.Linear(dim, dim * 2), nn.SiLU(), nn.Linear(dim * 2, dim))

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        half = self.dim // 2
        f = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / max(half - 1, 1))
        a = t.float().view(-1, 1) * 1000.0 * f.view(1, -1)
        return self.mlp(torch.cat([a.sin(), a.cos()], dim=-1))


class SpectrogramConformerUNet(NeuralModule):
    """Conformer over the time axis of (real, imag)-stacked spectrograms with U-Net skip connections between the first and
    second half of the layers; optional conditioning spectrogram and diffusion / flow time."""

    def __init__(self, in_channels: int = 1, out_channels: int = 1, feat_in: int = 257, n_layers: int = 4, d_model: int = 128,
                 n_heads: int = 4, conv_kernel_size: int = 9, dropout: float = 0.0, use_time: bool = True):
        super().__init__()
        from ..modules.conformer_modules import ConformerLayer

        self.in_ch, self.out_ch, self.F = in_channels, out_channels, feat_in
        self.proj_in = nn.Linear(2 * in_channels * feat_in, d_model)
        self.time = _TimeEmbedding(d_model) if use_time else None
        self.layers = nn.ModuleList([ConformerLayer(d_model=d_model, d_ff=4 * d_model, self_attention_model="abs_pos", n_heads=n_heads,
                                                    conv_kernel_size=conv_kernel_size, conv_norm_type="layer_norm", dropout=dropout,
                                                    dropout_att=dropout) for _ in range(n_layers)])
        self.skip = nn.ModuleList([nn.Linear(2 * d_model, d_model) for _ in range(n_layers // 2)])
        self.proj_out = nn.Linear(d_model, 2 * out_channels * feat_in)

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None, condition: Optional[torch.Tensor] = None,
                time: Optional[torch.Tensor] = None):
        """input complex [B, C_in, F, N] (condition is concatenated along channels by the caller) → complex [B, C_out, F, N]."""
        B, C, Fq, N = input.shape
        x = torch.view_as_real(input).permute(0, 3, 1, 4, 2).reshape(B, N, C * 2 * Fq)
        h = self.proj_in(x.float())
        if self.time is not None and time is not None:
            h = h + self.time(time).unsqueeze(1)
        pad = None if input_length is None else ~_len_mask(input_length, N, h.device)
        att = None if pad is None else (pad.unsqueeze(1) | pad.unsqueeze(2))
        stack = []
        half = len(self.layers) // 2
        for i, l in enumerate(self.layers):
            if i >= len(self.layers) - half:
                h = self.skip[i - (len(self.layers) - half)](torch.cat([h, stack.pop()], dim=-1))
            h = l(x=h, att_mask=att, pos_emb=None, pad_mask=pad)
            if i < half:
                stack.append(h)
        y = self.proj_out(h.float()).view(B, N, self.out_ch, 2, Fq).permute(0, 2, 4, 1, 3).contiguous()
        y = torch.view_as_complex(y)
        if input_length is not None:
            y = y * _len_mask(input_length, N, y.device).view(B, 1, 1, N)
        return y, input_length


class SpectrogramNCSN(NeuralModule):
    """Small 2-D convolutional score network over (real, imag) channels with FiLM time conditioning."""

    def __init__(self, in_channels: int = 2, out_channels: int = 1, hidden: int = 32, n_blocks: int = 3):
        super().__init__()
        self.inp = nn.Conv2d(2 * in_channels, hidden, 3, padding=1)
        self.time = _TimeEmbedding(hidden)
        self.blocks = nn.ModuleList([nn.ModuleList([nn.GroupNorm(4, hidden), nn.Conv2d(hidden, hidden, 3, padding=1),
                                                    nn.Linear(hidden, 2 * hidden)]) for _ in range(n_blocks)])
        self.out = nn.Conv2d(hidden, 2 * out_channels, 3, padding=1)
        self.out_ch = out_channels

    def forward(self, input: torch.Tensor, input_length=None, condition=None, time=None):
        B, C, Fq, N = input.shape
        x = torch.view_as_real(input).permute(0, 1, 4, 2, 3).reshape(B, 2 * C, Fq, N).float()
        h = self.inp(x)
        te = self.time(time if time is not None else torch.zeros(B, device=x.device))
        for gn, conv, film in self.blocks:
            s, b = film(te).chunk(2, dim=-1)
            h = h + conv(F.silu(gn(h) * (1 + s.view(B, -1, 1, 1)) + b.view(B, -1, 1, 1)))
        y = self.out(h).view(B, self.out_ch, 2, Fq, N).permute(0, 1, 3, 4, 2).contiguous()
        y = torch.view_as_complex(y)
        if input_length is not None:
            y = y * _len_mask(input_length, N, y.device).view(B, 1, 1, N)
        return y, input_length

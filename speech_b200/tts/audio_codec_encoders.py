"""Spectral encoders and the low-latency residual decoder of the audio codec, with the normalised convolution wrappers they are
made of.  The encoders work on spectral features at the frame rate instead of strided convolutions over samples: a mel
spectrogram encoded full-band or per band by residual networks, or log-magnitude STFTs at several resolutions merged while the
frame rate is halved at each stage.  The decoder does most of its work at the low frame rate and keeps the up-sampling stack
small; it can be causal.
Reference: ``tts/modules/audio_codec_modules.py`` (``CodecActivation``, ``Conv1dNorm`` / ``ConvTranspose1dNorm`` and causal
variants, ``ResidualBlockV2``, ``HiFiGANResBlock`` / ``HiFiGANResLayer``, ``MelSpectrogramProcessor``, ``STFTProcessor``,
``ResNetEncoder``, ``FullBandMelEncoder``, ``MultiBandMelEncoder``, ``STFTResidualBlock``, ``DownSampleResidualBlock``,
``MultiResolutionSTFTEncoder``, ``ResNetDecoder``, ``CausalHiFiGANEncoder``, ``MultiPeriodDiscriminator``, ``PreEmphasis``).
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from .audio_codec import PeriodDiscriminator, mask_by_length
from .audio_codec_extra import CausalConv1d, CausalConvTranspose1d


class _Snake(nn.Module):
    """``x + sin^2(alpha x) / alpha`` with one learned ``alpha`` per channel; ``half`` applies it to the first half of the channels and a
    leaky ReLU to the rest."""

    def __init__(self, channels: int, half: bool = False):
        super().__init__()
        self.half = half
        self.n = channels // 2 if half else channels
        self.alpha = nn.Parameter(torch.ones(1, self.n, 1))

    def forward(self, x):
        a = x[:, :self.n]
        a = a + torch.sin(self.alpha * a).square() / (self.alpha + 1e-9)
        return torch.cat([a, F.leaky_relu(x[:, self.n:], 0.01)], dim=1) if self.half else a


class CodecActivation(nn.Module):
    """``elu``, ``lrelu`` (slope 0.1), ``snake`` or ``half_snake`` by name."""

    def __init__(self, activation: str = "elu", channels: int = 1):
        super().__init__()
        activation = activation.lower()
        if activation == "elu":
            self.activation = nn.ELU()
        elif activation == "lrelu":
            self.activation = nn.LeakyReLU(0.1)
        elif activation == "snake":
            self.activation = _Snake(channels)
        elif activation == "half_snake":
            self.activation = _Snake(channels, half=True)
        else:
            raise ValueError(f"unknown activation {activation!r}: choose elu, lrelu, snake or half_snake")

    def forward(self, x):
        return self.activation(x)


def _wn(m):
    return nn.utils.parametrizations.weight_norm(m)


class _NormConv(nn.Module):
    def remove_weight_norm(self):
        for m in self.modules():
            if isinstance(m, (nn.Conv1d, nn.ConvTranspose1d, nn.Conv2d)) and nn.utils.parametrize.is_parametrized(m, "weight"):
                nn.utils.parametrize.remove_parametrizations(m, "weight")


class Conv1dNorm(_NormConv):
    """Weight-normalised 1-D convolution with ``same``-style padding (``stride`` s maps T frames to ``T // s``), an optional activation
    and masking of the frames past ``input_len``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, dilation: int = 1, padding: Optional[int] = None,
                 pad_mode: str = "reflect", activation: Optional[str] = None):
        super().__init__()
        padding = dilation * (kernel_size - 1) // 2 if padding is None else padding
        self.conv = _wn(nn.Conv1d(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation, padding=padding,
                                  padding_mode={"reflect": "reflect", "replicate": "replicate", "zeros": "zeros"}[pad_mode]))
        self.activation = CodecActivation(activation, out_channels) if activation else None

    def forward(self, inputs, input_len=None):
        y = self.conv(inputs)
        if self.activation is not None:
            y = self.activation(y)
        if input_len is not None:
            y = mask_by_length(y[..., :int(input_len.max())] if y.shape[-1] > int(input_len.max()) else y, input_len.clamp(max=y.shape[-1]))
        return y


class CausalConv1dNorm(_NormConv):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, dilation: int = 1, pad_mode: str = "zeros", activation: Optional[str] = None):
        super().__init__()
        self.inner = CausalConv1d(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation)
        self.inner.conv = _wn(self.inner.conv)
        self.activation = CodecActivation(activation, out_channels) if activation else None

    def forward(self, inputs, input_len=None):
        y = self.inner(inputs)
        if self.activation is not None:
            y = self.activation(y)
        return mask_by_length(y, input_len.clamp(max=y.shape[-1])) if input_len is not None else y


class ConvTranspose1dNorm(_NormConv):
    """Weight-normalised transposed convolution that maps T frames to exactly ``T * stride``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, activation: Optional[str] = None):
        super().__init__()
        pad, out_pad = math.ceil((kernel_size - stride) / 2), (kernel_size - stride) % 2
        self.stride = stride
        self.conv = _wn(nn.ConvTranspose1d(in_channels, out_channels, kernel_size, stride=stride, padding=pad, output_padding=out_pad))
        self.activation = CodecActivation(activation, out_channels) if activation else None

    def forward(self, inputs, input_len=None):
        y = self.conv(inputs)[..., :inputs.shape[-1] * self.stride]
        if self.activation is not None:
            y = self.activation(y)
        return mask_by_length(y, input_len.clamp(max=y.shape[-1])) if input_len is not None else y


class CausalConvTranspose1dNorm(_NormConv):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, activation: Optional[str] = None):
        super().__init__()
        if kernel_size != 2 * stride:
            raise ValueError("the causal up-sampler uses a kernel of twice its stride")
        self.inner = CausalConvTranspose1d(in_channels, out_channels, stride)
        self.inner.tconv = _wn(self.inner.tconv)
        self.activation = CodecActivation(activation, out_channels) if activation else None

    def forward(self, inputs, input_len=None):
        y = self.inner(inputs)
        if self.activation is not None:
            y = self.activation(y)
        return mask_by_length(y, input_len.clamp(max=y.shape[-1])) if input_len is not None else y


class Conv2dNorm(_NormConv):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: Tuple[int, int], stride: Tuple[int, int] = (1, 1), dilation: Tuple[int, int] = (1, 1)):
        super().__init__()
        pad = tuple(d * (k - 1) // 2 for k, d in zip(kernel_size, dilation))
        self.conv = _wn(nn.Conv2d(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation, padding=pad, padding_mode="reflect"))

    def forward(self, inputs):
        return self.conv(inputs)


def _conv(causal: bool):
    return CausalConv1dNorm if causal else Conv1dNorm


class ResidualBlockV1(nn.Module):
    """Pre-activation residual branch: ``x + skip(act(dropout(input(act(x)))))`` with a dilated first convolution."""

    def __init__(self, channels: int, filters: int, kernel_size: int = 3, dilation: int = 1, dropout_rate: float = 0.0, activation: str = "lrelu",
                 is_causal: bool = False, pad_mode: str = "reflect"):
        super().__init__()
        C = _conv(is_causal)
        self.input_activation, self.skip_activation = CodecActivation(activation, channels), CodecActivation(activation, filters)
        self.input_conv = C(channels, filters, kernel_size, dilation=dilation, pad_mode=pad_mode)
        self.skip_conv = C(filters, channels, kernel_size, pad_mode=pad_mode)
        self.dropout = nn.Dropout(dropout_rate)

    def forward(self, inputs, input_len=None):
        r = self.input_conv(self.input_activation(inputs), input_len)
        r = self.skip_conv(self.dropout(self.skip_activation(r)), input_len)
        return inputs + r


class ResidualBlockV2(nn.Module):
    """Post-activation variant: ``act(x + skip(input(x)))`` (the first convolution carries its own activation)."""

    def __init__(self, channels: int, filters: int, kernel_size: int = 3, activation: str = "lrelu", is_causal: bool = False, pad_mode: str = "reflect"):
        super().__init__()
        C = _conv(is_causal)
        self.input_conv = C(channels, filters, kernel_size, activation=activation, pad_mode=pad_mode)
        self.skip_conv = C(filters, channels, kernel_size, pad_mode=pad_mode)
        self.output_activation = CodecActivation(activation, channels)

    def forward(self, inputs, input_len=None):
        out = self.output_activation(inputs + self.skip_conv(self.input_conv(inputs, input_len), input_len))
        return mask_by_length(out, input_len.clamp(max=out.shape[-1])) if input_len is not None else out


class HiFiGANResBlock(nn.Module):
    """One residual block per dilation, applied in sequence."""

    def __init__(self, channels: int, kernel_size: int, dilations: Iterable[int], activation: str = "lrelu", is_causal: bool = False, pad_mode: str = "reflect"):
        super().__init__()
        self.res_blocks = nn.ModuleList(ResidualBlockV1(channels, channels, kernel_size, d, 0.0, activation, is_causal, pad_mode) for d in dilations)

    def forward(self, inputs, input_len=None):
        for b in self.res_blocks:
            inputs = b(inputs, input_len)
        return inputs


class HiFiGANResLayer(nn.Module):
    """The mean of one ``HiFiGANResBlock`` per kernel size (multi-receptive-field fusion)."""

    def __init__(self, channels: int, kernel_sizes: Iterable[int], dilations: Iterable[int], activation: str = "lrelu", is_causal: bool = False, pad_mode: str = "reflect"):
        super().__init__()
        self.res_blocks = nn.ModuleList(HiFiGANResBlock(channels, k, list(dilations), activation, is_causal, pad_mode) for k in kernel_sizes)

    def forward(self, inputs, input_len=None):
        return sum(b(inputs, input_len) for b in self.res_blocks) / len(self.res_blocks)


class CausalHiFiGANEncoder(nn.Module):
    """The HiFi-GAN generator inverted into an encoder with causal convolutions: a residual layer then a strided convolution per
    down-sampling rate, channels doubling each time."""

    def __init__(self, encoded_dim: int, down_sample_rates: Sequence[int] = (2, 4, 5, 8), base_channels: int = 32, in_kernel_size: int = 7, out_kernel_size: int = 7,
                 resblock_kernel_sizes: Sequence[int] = (3, 7, 11), resblock_dilation_sizes: Sequence[int] = (1, 3, 5), activation: str = "lrelu", pad_mode: str = "zeros"):
        super().__init__()
        self.down_sample_rates = list(down_sample_rates)
        self.pre_conv = CausalConv1dNorm(1, base_channels, in_kernel_size)
        ch = base_channels
        self.activations, self.res_layers, self.down_sample_conv_layers = nn.ModuleList(), nn.ModuleList(), nn.ModuleList()
        for r in self.down_sample_rates:
            self.res_layers.append(HiFiGANResLayer(ch, resblock_kernel_sizes, resblock_dilation_sizes, activation, is_causal=True))
            self.activations.append(CodecActivation(activation, ch))
            self.down_sample_conv_layers.append(CausalConv1dNorm(ch, 2 * ch, 2 * r, stride=r))
            ch *= 2
        self.post_activation = CodecActivation(activation, ch)
        self.post_conv = CausalConv1dNorm(ch, encoded_dim, out_kernel_size)

    @property
    def total_stride(self) -> int:
        return int(math.prod(self.down_sample_rates))

    def forward(self, audio: torch.Tensor, audio_len: torch.Tensor):
        x, lens = self.pre_conv(audio.unsqueeze(1), audio_len), audio_len
        for act, res, down, r in zip(self.activations, self.res_layers, self.down_sample_conv_layers, self.down_sample_rates):
            x = act(res(x, lens))
            lens = lens // r
            x = down(x)
            x = mask_by_length(x[..., :max(int(lens.max()), 1)], lens.clamp(max=x.shape[-1]))
        return self.post_conv(self.post_activation(x), lens), lens


# ---------------------------------------------------------------------------------------------------------- spectral front ends
class PreEmphasis(nn.Module):
    """``y[t] = x[t] - coefficient * x[t-1]`` with the first sample reflected."""

    def __init__(self, coefficient: float = 0.97):
        super().__init__()
        self.register_buffer("filter", torch.tensor([-coefficient, 1.0]).view(1, 1, 2))

    def forward(self, audio: torch.Tensor) -> torch.Tensor:
        return F.conv1d(F.pad(audio.unsqueeze(1), (1, 0), "reflect"), self.filter).squeeze(1)


class STFTProcessor(nn.Module):
    """Log-magnitude STFT ``log(|X| + log_guard)`` with exactly ``audio_len // hop_length`` frames (the signal is padded by ``(n_fft - hop) / 2``
    on both sides instead of being centred)."""

    def __init__(self, n_fft: int, win_length: int, hop_length: int, log_guard: float = 1.0, pad_mode: str = "reflect"):
        super().__init__()
        self.n_fft, self.win_length, self.hop_length, self.log_guard, self.pad_mode = n_fft, win_length, hop_length, log_guard, pad_mode
        self.register_buffer("window", torch.hann_window(win_length, periodic=False), persistent=False)
        self.pad = (n_fft - hop_length) // 2

    def magnitude(self, audio: torch.Tensor) -> torch.Tensor:
        x = F.pad(audio.unsqueeze(1), (self.pad, self.pad), self.pad_mode).squeeze(1)
        return torch.stft(x.float(), self.n_fft, self.hop_length, self.win_length, self.window.float(), center=False, return_complex=True).abs()

    def forward(self, audio: torch.Tensor, audio_len: torch.Tensor):
        spec_len = audio_len // self.hop_length
        spec = torch.log(self.magnitude(audio) + self.log_guard)
        spec = spec[..., :max(int(spec_len.max()), 1)]
        return mask_by_length(spec, spec_len.clamp(max=spec.shape[-1])), spec_len


class MelSpectrogramProcessor(nn.Module):
    """Log-mel features for codec training: magnitude STFT (window = FFT size) → HTK-free triangular mel bank → ``log(mel + log_guard)``;
    ``audio_len // hop_length`` frames."""

    def __init__(self, sample_rate: int, win_length: int, hop_length: int, mel_dim: int = 80, log_guard: float = 1.0):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        self.mel_dim, self.hop_length = mel_dim, hop_length
        self.stft = STFTProcessor(win_length, win_length, hop_length, log_guard=0.0)
        self.log_guard = log_guard
        self.register_buffer("fb", torch.as_tensor(np.asarray(mel_filterbank(sample_rate, win_length, mel_dim, 0.0, None, norm=None)), dtype=torch.float32), persistent=False)

    def forward(self, audio: torch.Tensor, audio_len: torch.Tensor):
        spec_len = audio_len // self.hop_length
        mel = torch.log(torch.matmul(self.fb, self.stft.magnitude(audio)) + self.log_guard)
        mel = mel[..., :max(int(spec_len.max()), 1)]
        return mask_by_length(mel, spec_len.clamp(max=mel.shape[-1])), spec_len


class ResNetEncoder(nn.Module):
    """Residual network over frame-rate features; the time axis keeps its length."""

    def __init__(self, in_channels: int, out_channels: int, num_layers: int = 6, hidden_channels: int = 256, filters: int = 768, kernel_size: int = 3,
                 dropout_rate: float = 0.1, activation: str = "lrelu", pad_mode: str = "reflect"):
        super().__init__()
        self.pre_conv = Conv1dNorm(in_channels, hidden_channels, kernel_size, pad_mode=pad_mode)
        self.res_layers = nn.ModuleList(ResidualBlockV1(hidden_channels, filters, kernel_size, 1, dropout_rate, activation, False, pad_mode) for _ in range(num_layers))
        self.post_activation = CodecActivation(activation, hidden_channels)
        self.post_conv = Conv1dNorm(hidden_channels, out_channels, kernel_size, pad_mode=pad_mode)

    def forward(self, inputs, input_len):
        x = self.pre_conv(inputs, input_len)
        for layer in self.res_layers:
            x = layer(x, input_len)
        return self.post_conv(self.post_activation(x), input_len)


class FullBandMelEncoder(nn.Module):
    def __init__(self, mel_processor: nn.Module, encoder: nn.Module):
        super().__init__()
        self.mel_processor, self.encoder = mel_processor, encoder

    @property
    def total_stride(self) -> int:
        return int(self.mel_processor.hop_length)

    def forward(self, audio, audio_len):
        spec, spec_len = self.mel_processor(audio, audio_len)
        return self.encoder(spec, spec_len), spec_len


class MultiBandMelEncoder(nn.Module):
    """Mel channels ``[start, end)`` of each band go through a residual encoder of their own; the outputs are concatenated (one codebook
    group per band when the quantiser has as many groups).  The bands must cover every mel channel."""

    def __init__(self, mel_bands: Sequence[Tuple[int, int]], mel_processor: nn.Module, **encoder_kwargs):
        super().__init__()
        self.validate_mel_bands(mel_processor.mel_dim, mel_bands)
        self.mel_bands, self.mel_processor = [tuple(b) for b in mel_bands], mel_processor
        self.encoders = nn.ModuleList(ResNetEncoder(in_channels=b[1] - b[0], **encoder_kwargs) for b in self.mel_bands)

    @staticmethod
    def validate_mel_bands(mel_dim: int, mel_bands: Sequence[Tuple[int, int]]) -> None:
        used = np.zeros(mel_dim, dtype=bool)
        for a, b in mel_bands:
            used[a:b] = True
        if not used.all():
            raise ValueError(f"mel bands must cover all {mel_dim} channels; missing {np.where(~used)[0].tolist()}")

    @property
    def total_stride(self) -> int:
        return int(self.mel_processor.hop_length)

    def forward(self, audio, audio_len):
        spec, spec_len = self.mel_processor(audio, audio_len)
        return torch.cat([enc(spec[:, a:b], spec_len) for (a, b), enc in zip(self.mel_bands, self.encoders)], dim=1), spec_len


class DownSampleResidualBlock(nn.Module):
    def __init__(self, channels: int, filters: int, kernel_size: int, activation: str, down_sample_rate: int, pad_mode: str):
        super().__init__()
        self.down_sample_rate = down_sample_rate
        self.down_sample_conv = Conv1dNorm(channels, filters, 2 * down_sample_rate + 1, stride=down_sample_rate, activation=activation, pad_mode=pad_mode)
        self.res_block = ResidualBlockV2(filters, filters, kernel_size, activation, pad_mode=pad_mode)

    def forward(self, inputs, input_len):
        out_len = input_len // self.down_sample_rate
        return self.res_block(self.down_sample_conv(inputs, out_len), out_len), out_len


class STFTResidualBlock(nn.Module):
    """Halves (``down_sample_rate``) the frame rate of the running encoding and adds the STFT of the audio at the matching resolution."""

    def __init__(self, resolution: Tuple[int, int, int], input_dim: int, filters: int, kernel_size: int, activation: str, down_sample_rate: int, pad_mode: str):
        super().__init__()
        n_fft, hop, win = resolution
        self.down_sample_rate = down_sample_rate
        self.down_sample_conv = Conv1dNorm(input_dim, filters, 2 * down_sample_rate + 1, stride=down_sample_rate, activation=activation, pad_mode=pad_mode)
        self.spec_processor = STFTProcessor(n_fft, win, hop, pad_mode=pad_mode)
        self.spec_conv = Conv1dNorm(n_fft // 2 + 1, filters, kernel_size, pad_mode=pad_mode)
        self.spec_act = CodecActivation(activation, filters)
        self.res_block = ResidualBlockV2(filters, filters, kernel_size, activation, pad_mode=pad_mode)

    def forward(self, inputs, input_len, audio, audio_len):
        out_len = input_len // self.down_sample_rate
        out = self.down_sample_conv(inputs, out_len)
        spec, _ = self.spec_processor(audio, audio_len)
        res = self.spec_conv(spec, out_len)
        T = min(out.shape[-1], res.shape[-1])
        out = self.spec_act(out[..., :T] + res[..., :T])
        return self.res_block(out, out_len), out_len


class MultiResolutionSTFTEncoder(nn.Module):
    """``resolutions``: ``(n_fft, hop, win)`` triples whose hops double from one to the next; the first sets the input frame rate, every further
    one halves it while adding its STFT, then ``down_sample_rate_list`` reduces it further.  Total stride = last hop × product of the rates."""

    def __init__(self, out_dim: int, resolutions: Sequence[Tuple[int, int, int]], resolution_filter_list: Sequence[int], down_sample_filter_list: Sequence[int] = (),
                 down_sample_rate_list: Sequence[int] = (), kernel_size: int = 3, activation: str = "lrelu", pad_mode: str = "replicate"):
        super().__init__()
        if len(resolutions) < 1 or len(resolutions) != len(resolution_filter_list):
            raise ValueError("one filter count per STFT resolution is needed")
        for a, b in zip(resolutions[:-1], resolutions[1:]):
            if b[1] != 2 * a[1]:
                raise ValueError(f"hop lengths must double between resolutions, got {a[1]} then {b[1]}")
        n_fft, hop, win = resolutions[0]
        f0 = resolution_filter_list[0]
        self.pre_spec_processor = STFTProcessor(n_fft, win, hop, pad_mode=pad_mode)
        self.pre_conv = Conv1dNorm(n_fft // 2 + 1, f0, kernel_size, activation=activation, pad_mode=pad_mode)
        self.pre_res_block = ResidualBlockV2(f0, f0, kernel_size, activation, pad_mode=pad_mode)
        dim = f0
        self.stft_blocks = nn.ModuleList()
        for res, f in zip(resolutions[1:], resolution_filter_list[1:]):
            self.stft_blocks.append(STFTResidualBlock(tuple(res), dim, f, kernel_size, activation, 2, pad_mode))
            dim = f
        if down_sample_filter_list and not down_sample_rate_list:
            down_sample_rate_list = [2] * len(down_sample_filter_list)
        self.down_sample_blocks = nn.ModuleList()
        for f, r in zip(down_sample_filter_list, down_sample_rate_list):
            self.down_sample_blocks.append(DownSampleResidualBlock(dim, f, kernel_size, activation, r, pad_mode))
            dim = f
        self.post_conv = Conv1dNorm(dim, out_dim, kernel_size, pad_mode=pad_mode)
        self._stride = int(resolutions[-1][1] * math.prod(down_sample_rate_list or [1]))

    @property
    def total_stride(self) -> int:
        return self._stride

    def forward(self, audio, audio_len):
        x, lens = self.pre_spec_processor(audio, audio_len)
        x = self.pre_res_block(self.pre_conv(x, lens), lens)
        for b in self.stft_blocks:
            x, lens = b(x, lens, audio, audio_len)
        for b in self.down_sample_blocks:
            x, lens = b(x, lens)
        return self.post_conv(x, lens), lens


class ResNetDecoder(nn.Module):
    """Low-latency decoder: a few up-sampling stages (``pre_up_sample_rates``), then ``n_hidden_layers`` residual blocks at that still-low frame rate
    where most of the parameters sit, then light up-sampling residual stages to the sample rate and a tanh output."""

    def __init__(self, input_dim: int, input_filters: int, pre_up_sample_rates: Sequence[int], pre_up_sample_filters: Sequence[int], n_hidden_layers: int,
                 hidden_filters: int, resblock_up_sample_rates: Sequence[int], resblock_up_sample_filters: Sequence[int], resblock_up_sample_kernel_size: int = 7,
                 kernel_size: int = 3, activation: str = "half_snake", is_causal: bool = False, pad_mode: str = "replicate"):
        super().__init__()
        if len(pre_up_sample_rates) != len(pre_up_sample_filters) or len(resblock_up_sample_rates) != len(resblock_up_sample_filters):
            raise ValueError("one filter count per up-sampling rate is needed")
        C, U = _conv(is_causal), (CausalConvTranspose1dNorm if is_causal else ConvTranspose1dNorm)
        pm = "zeros" if is_causal else pad_mode
        self.pre_conv = C(input_dim, input_filters, kernel_size, pad_mode=pm)
        ch = input_filters
        self.pre_up_sample_rates, self.resblock_up_sample_rates = list(pre_up_sample_rates), list(resblock_up_sample_rates)
        self.pre_resblocks, self.pre_up_sample_layers = nn.ModuleList(), nn.ModuleList()
        for r, f in zip(self.pre_up_sample_rates, pre_up_sample_filters):
            self.pre_resblocks.append(ResidualBlockV2(ch, 2 * ch, kernel_size, activation, is_causal, pm))
            self.pre_up_sample_layers.append(U(ch, f, 2 * r, stride=r, activation=activation))
            ch = f
        self.conv_layers = nn.ModuleList(ResidualBlockV2(ch, hidden_filters, kernel_size, activation, is_causal, pm) for _ in range(n_hidden_layers))
        self.resblock_up_sample_layers, self.resblocks = nn.ModuleList(), nn.ModuleList()
        for r, f in zip(self.resblock_up_sample_rates, resblock_up_sample_filters):
            self.resblock_up_sample_layers.append(U(ch, f, 2 * r, stride=r, activation=activation))
            self.resblocks.append(ResidualBlockV2(f, f, resblock_up_sample_kernel_size, activation, is_causal, pm))
            ch = f
        self.post_conv = C(ch, 1, kernel_size, pad_mode=pm)

    @property
    def total_stride(self) -> int:
        return int(math.prod(self.pre_up_sample_rates) * math.prod(self.resblock_up_sample_rates))

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        lens = input_len
        x = self.pre_conv(inputs, lens)
        for res, up, r in zip(self.pre_resblocks, self.pre_up_sample_layers, self.pre_up_sample_rates):
            x = res(x, lens)
            lens = lens * r
            x = up(x, lens)
        for layer in self.conv_layers:
            x = layer(x, lens)
        for up, res, r in zip(self.resblock_up_sample_layers, self.resblocks, self.resblock_up_sample_rates):
            lens = lens * r
            x = res(up(x, lens), lens)
        audio = torch.tanh(self.post_conv(x, lens)).squeeze(1)
        return mask_by_length(audio, lens.clamp(max=audio.shape[-1])), lens


class MultiPeriodDiscriminator(nn.Module):
    """One period discriminator per period; returns the lists ``(scores_real, scores_gen, fmaps_real, fmaps_gen)``."""

    def __init__(self, periods: Iterable[int] = (2, 3, 5, 7, 11), lrelu_slope: float = 0.1):
        super().__init__()
        self.discriminators = nn.ModuleList(PeriodDiscriminator(p) for p in periods)

    def forward(self, audio_real: torch.Tensor, audio_gen: torch.Tensor):
        sr, sg, fr, fg = [], [], [], []
        for d in self.discriminators:
            a, fa = d(audio_real)
            b, fb = d(audio_gen)
            sr.append(a); sg.append(b); fr.append(fa); fg.append(fb)
        return sr, sg, fr, fg


ENCODERS = {"MultiBandMelEncoder": MultiBandMelEncoder, "FullBandMelEncoder": FullBandMelEncoder, "MultiResolutionSTFTEncoder": MultiResolutionSTFTEncoder,
            "CausalHiFiGANEncoder": CausalHiFiGANEncoder}
DECODERS = {"ResNetDecoder": ResNetDecoder}


def build_encoder(cfg: dict) -> nn.Module:
    """Encoder from a config whose ``_target_`` ends in one of the class names above; a ``mel_processor`` sub-config builds the mel front end
    and an ``encoder`` sub-config the residual network of the full-band variant."""
    cfg = dict(cfg)
    name = str(cfg.pop("_target_")).rsplit(".", 1)[-1]
    if "mel_processor" in cfg:
        mp = dict(cfg.pop("mel_processor"))
        mp.pop("_target_", None)
        cfg["mel_processor"] = MelSpectrogramProcessor(**mp)
    if name == "FullBandMelEncoder":
        ec = dict(cfg.pop("encoder"))
        ec.pop("_target_", None)
        cfg["encoder"] = ResNetEncoder(**ec)
    return ENCODERS[name](**cfg)

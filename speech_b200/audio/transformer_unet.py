"""Transformer U-Net over spectrogram frames: a stack of pre-norm attention / GEGLU blocks whose second half receives skip
connections from the first half, with convolutional position embedding, rotary-free attention and optional adaptive RMS norm
conditioned on a diffusion / flow time (reference ``audio/parts/submodules/transformerunet.py``: ``LearnedSinusoidalPosEmb``,
``ConvPositionEmbed``, ``RMSNorm`` / ``AdaptiveRMSNorm``, ``GEGLU``, ``TransformerUNet``, ``SpectrogramTransformerUNet``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..core.module import NeuralModule


class LearnedSinusoidalPosEmb(nn.Module):
    """Scalar -> ``[x, sin(2π w x), cos(2π w x)]`` with learned frequencies ``w`` (``dim`` even: ``dim / 2`` frequencies)."""

    def __init__(self, dim: int):
        super().__init__()
        if dim % 2:
            raise ValueError("dim must be even")
        self.weights = nn.Parameter(torch.randn(dim // 2))

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        t = t.view(-1, 1).float()
        f = t * self.weights.view(1, -1) * 2 * math.pi
        return torch.cat([t, f.sin(), f.cos()], dim=-1)


class ConvPositionEmbed(nn.Module):
    """Position information from a grouped 1-D convolution over time followed by GELU; padded frames are zeroed before and after."""

    def __init__(self, dim: int, kernel_size: int, groups: Optional[int] = None):
        super().__init__()
        if kernel_size % 2 == 0:
            raise ValueError("kernel_size must be odd")
        self.conv = nn.Conv1d(dim, dim, kernel_size, padding=kernel_size // 2, groups=groups or dim)

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if mask is not None:
            x = x * mask.unsqueeze(-1)
        y = F.gelu(self.conv(x.transpose(1, 2))).transpose(1, 2)
        return y if mask is None else y * mask.unsqueeze(-1)


class RMSNorm(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.scale, self.gamma = dim ** 0.5, nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F.normalize(x, dim=-1) * self.scale * self.gamma


class AdaptiveRMSNorm(nn.Module):
    """RMS norm whose gain and shift are linear functions of a condition vector (zero-initialised: starts as plain RMS norm)."""

    def __init__(self, dim: int, cond_dim: Optional[int] = None):
        super().__init__()
        cond_dim = cond_dim or dim
        self.scale = dim ** 0.5
        self.to_gamma, self.to_beta = nn.Linear(cond_dim, dim), nn.Linear(cond_dim, dim)
        for lin, b in ((self.to_gamma, 1.0), (self.to_beta, 0.0)):
            nn.init.zeros_(lin.weight)
            nn.init.constant_(lin.bias, b)

    def forward(self, x, cond):
        g, b = self.to_gamma(cond).unsqueeze(1), self.to_beta(cond).unsqueeze(1)
        return F.normalize(x, dim=-1) * self.scale * g + b


class GEGLU(nn.Module):
    def forward(self, x):
        a, gate = x.chunk(2, dim=-1)
        return F.gelu(gate) * a


class _Block(nn.Module):
    def __init__(self, dim: int, heads: int, ff_mult: int, dropout: float, adaptive: bool, skip: bool):
        super().__init__()
        norm = (lambda: AdaptiveRMSNorm(dim)) if adaptive else (lambda: RMSNorm(dim))
        self.skip = nn.Linear(2 * dim, dim) if skip else None
        self.n1, self.n2 = norm(), norm()
        self.attn = nn.MultiheadAttention(dim, heads, dropout=dropout, batch_first=True)
        inner = int(dim * ff_mult * 2 / 3)
        self.ff = nn.Sequential(nn.Linear(dim, 2 * inner), GEGLU(), nn.Dropout(dropout), nn.Linear(inner, dim))
        self.adaptive = adaptive

    def forward(self, x, pad, cond, skip_in=None):
        if self.skip is not None:
            x = self.skip(torch.cat([x, skip_in], dim=-1))
        h = self.n1(x, cond) if self.adaptive else self.n1(x)
        x = x + self.attn(h, h, h, key_padding_mask=pad, need_weights=False)[0]
        h = self.n2(x, cond) if self.adaptive else self.n2(x)
        return x + self.ff(h)


class TransformerUNet(NeuralModule):
    """``depth`` blocks (even); block ``depth/2 + i`` concatenates the output of block ``depth/2 - 1 - i``.  ``adaptive_rmsnorm``
    conditions every norm on ``adaptive_rmsnorm_cond`` ``[B, dim]``."""

    def __init__(self, dim: int, depth: int, heads: int = 8, ff_mult: int = 4, attn_dropout: float = 0.0, ff_dropout: float = 0.0,
                 max_positions: int = 6000, adaptive_rmsnorm: bool = False, adaptive_rmsnorm_cond_dim_in: Optional[int] = None,
                 conv_pos_embed_kernel_size: int = 31, conv_pos_embed_groups: Optional[int] = None):
        super().__init__()
        if depth % 2:
            raise ValueError("depth must be even")
        self.pos = ConvPositionEmbed(dim, conv_pos_embed_kernel_size, conv_pos_embed_groups)
        self.blocks = nn.ModuleList([_Block(dim, heads, ff_mult, max(attn_dropout, ff_dropout), adaptive_rmsnorm, i >= depth // 2)
                                     for i in range(depth)])
        self.final = RMSNorm(dim)
        self.adaptive = adaptive_rmsnorm

    def forward(self, x: torch.Tensor, key_padding_mask: Optional[torch.Tensor] = None, adaptive_rmsnorm_cond: Optional[torch.Tensor] = None):
        """x ``[B, N, dim]``; ``key_padding_mask`` ``[B, N]`` True on padding."""
        if self.adaptive and adaptive_rmsnorm_cond is None:
            raise ValueError("adaptive_rmsnorm_cond is required")
        valid = None if key_padding_mask is None else (~key_padding_mask).to(x.dtype)
        x = x + self.pos(x, valid)
        stack = []
        half = len(self.blocks) // 2
        for i, b in enumerate(self.blocks):
            if i < half:
                x = b(x, key_padding_mask, adaptive_rmsnorm_cond)
                stack.append(x)
            else:
                x = b(x, key_padding_mask, adaptive_rmsnorm_cond, skip_in=stack.pop())
        return self.final(x)


class SpectrogramTransformerUNet(NeuralModule):
    """Complex spectrogram ``[B, C_in, F, N]`` (+ optional condition ``[B, C_c, F, N]`` and time ``[B]``) -> ``[B, C_out, F, N]``."""

    def __init__(self, in_channels: int = 1, out_channels: int = 1, freq_dim: int = 256, dim: int = 1024, depth: int = 24, heads: int = 16,
                 ff_mult: int = 4, ff_dropout: float = 0.0, attn_dropout: float = 0.0, max_positions: int = 6000, time_hidden_dim: Optional[int] = None,
                 conv_pos_embed_kernel_size: int = 31, conv_pos_embed_groups: Optional[int] = None, adaptive_rmsnorm: bool = True):
        super().__init__()
        self.in_ch, self.out_ch, self.F = in_channels, out_channels, freq_dim
        self.proj_in = nn.Linear(2 * in_channels * freq_dim, dim)
        th = time_hidden_dim or 4 * dim
        self.time = nn.Sequential(LearnedSinusoidalPosEmb(dim), nn.Linear(dim + 1, th), nn.SiLU(), nn.Linear(th, dim)) if adaptive_rmsnorm else None
        self.net = TransformerUNet(dim, depth, heads, ff_mult, attn_dropout, ff_dropout, max_positions, adaptive_rmsnorm, dim,
                                   conv_pos_embed_kernel_size, conv_pos_embed_groups)
        self.proj_out = nn.Linear(dim, 2 * out_channels * freq_dim)

    def forward(self, input: torch.Tensor, input_length: Optional[torch.Tensor] = None, condition: Optional[torch.Tensor] = None,
                time: Optional[torch.Tensor] = None):
        if condition is not None:
            input = torch.cat([input, condition], dim=1)
        B, C, Fq, N = input.shape
        if C != self.in_ch or Fq != self.F:
            raise ValueError(f"expected [{self.in_ch} channels, {self.F} bands], got [{C}, {Fq}]")
        x = torch.view_as_real(input).permute(0, 3, 1, 4, 2).reshape(B, N, C * 2 * Fq)
        pad = None if input_length is None else torch.arange(N, device=x.device)[None, :] >= input_length[:, None]
        cond = None
        if self.time is not None:
            cond = self.time(time if time is not None else torch.zeros(B, device=x.device))
        h = self.net(self.proj_in(x.float()), pad, cond)
        y = self.proj_out(h).view(B, N, self.out_ch, 2, Fq).permute(0, 2, 4, 1, 3).contiguous()
        y = torch.view_as_complex(y)
        if pad is not None:
            y = y * (~pad).view(B, 1, 1, N)
        return y, input_length

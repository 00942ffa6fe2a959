"""EnCodec-style codec parts: SEANet encoder / decoder (residual conv blocks, strided re-sampling, an LSTM bottleneck) and
residual vector quantisation with Euclidean codebooks trained by exponential moving averages (k-means initialisation on the first
batch, re-seeding of codes that stopped being used), plain and grouped.

Reference: ``tts/modules/encodec_modules.py`` (``SEANetEncoder``, ``SEANetDecoder``, ``EuclideanCodebook``, ``ResidualVectorQuantizer``,
``GroupResidualVectorQuantizer``).  The STFT discriminators of that file live in ``tts/audio_codec_extra.py``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .audio_codec import mask_by_length

__all__ = ["EuclideanCodebook", "GroupResidualVectorQuantizer", "ResidualVectorQuantizer", "SEANetDecoder", "SEANetEncoder"]


def _pad_same(k: int, d: int = 1) -> int:
    return (k - 1) * d // 2


class SEANetResnetBlock(nn.Module):
    """ELU -> conv(k=3) to half the channels -> ELU -> conv(k=1) back, plus a 1x1 convolution shortcut."""

    def __init__(self, channels: int):
        super().__init__()
        self.pre = nn.Conv1d(channels, channels // 2, 3, padding=1)
        self.post = nn.Conv1d(channels // 2, channels, 1)
        self.short = nn.Conv1d(channels, channels, 1)

    def forward(self, x, lens):
        y = self.post(F.elu(self.pre(F.elu(x))))
        return mask_by_length(self.short(x) + y, lens)


class SEANetRNN(nn.Module):
    def __init__(self, dim: int, num_layers: int = 2):
        super().__init__()
        self.rnn = nn.LSTM(dim, dim, num_layers, batch_first=True)

    def forward(self, x, lens):
        packed = nn.utils.rnn.pack_padded_sequence(x.transpose(1, 2), lens.cpu().clamp(min=1), batch_first=True, enforce_sorted=False)
        y, _ = self.rnn(packed)
        y, _ = nn.utils.rnn.pad_packed_sequence(y, batch_first=True, total_length=x.shape[2])
        return mask_by_length(x + y.transpose(1, 2), lens)


class SEANetEncoder(nn.Module):
    """``[B, T]`` audio -> ``[B, encoded_dim, T / prod(down_sample_rates)]``."""

    def __init__(self, down_sample_rates: Sequence[int] = (2, 4, 5, 8), base_channels: int = 32, in_kernel_size: int = 7, out_kernel_size: int = 7,
                 encoded_dim: int = 128, rnn_layers: int = 2):
        super().__init__()
        self.rates = list(down_sample_rates)
        self.pre = nn.Conv1d(1, base_channels, in_kernel_size, padding=_pad_same(in_kernel_size))
        ch = base_channels
        self.res, self.down = nn.ModuleList(), nn.ModuleList()
        for r in self.rates:
            self.res.append(SEANetResnetBlock(ch))
            self.down.append(nn.Conv1d(ch, 2 * ch, 2 * r, stride=r, padding=math.ceil(r / 2)))
            ch *= 2
        self.rnn = SEANetRNN(ch, rnn_layers)
        self.post = nn.Conv1d(ch, encoded_dim, out_kernel_size, padding=_pad_same(out_kernel_size))
        self.total_stride = int(math.prod(self.rates))

    def forward(self, audio: torch.Tensor, audio_len: torch.Tensor):
        x, lens = mask_by_length(self.pre(mask_by_length(audio, audio_len).unsqueeze(1)), audio_len), audio_len
        for res, down, r in zip(self.res, self.down, self.rates):
            x = res(x, lens)
            lens = torch.div(lens, r, rounding_mode="floor")
            x = down(F.elu(x))[..., : int(lens.max()) if lens.numel() else 0]
            x = mask_by_length(x, lens)
        x = self.rnn(x, lens)
        return mask_by_length(self.post(F.elu(x)), lens), lens


class SEANetDecoder(nn.Module):
    def __init__(self, up_sample_rates: Sequence[int] = (8, 5, 4, 2), base_channels: int = 512, in_kernel_size: int = 7, out_kernel_size: int = 3,
                 encoded_dim: int = 128, rnn_layers: int = 2):
        super().__init__()
        self.rates = list(up_sample_rates)
        self.pre = nn.Conv1d(encoded_dim, base_channels, in_kernel_size, padding=_pad_same(in_kernel_size))
        self.rnn = SEANetRNN(base_channels, rnn_layers)
        ch = base_channels
        self.up, self.res = nn.ModuleList(), nn.ModuleList()
        for r in self.rates:
            self.up.append(nn.ConvTranspose1d(ch, ch // 2, 2 * r, stride=r, padding=r // 2 + r % 2, output_padding=r % 2))
            ch //= 2
            self.res.append(SEANetResnetBlock(ch))
        self.post = nn.Conv1d(ch, 1, out_kernel_size, padding=_pad_same(out_kernel_size))

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        x, lens = mask_by_length(self.pre(mask_by_length(inputs, input_len)), input_len), input_len
        x = self.rnn(x, lens)
        for up, res, r in zip(self.up, self.res, self.rates):
            lens = lens * r
            x = up(F.elu(x))
            x = F.pad(x, (0, max(0, int(lens.max()) - x.shape[-1])))[..., : int(lens.max())]
            x = res(mask_by_length(x, lens), lens)
        audio = torch.tanh(self.post(F.elu(x))).squeeze(1)
        return mask_by_length(audio, lens), lens


# ------------------------------------------------------------------------------------------------ quantisation
def _k_means(samples: torch.Tensor, k: int, iters: int = 10) -> Tuple[torch.Tensor, torch.Tensor]:
    n = samples.shape[0]
    idx = torch.randperm(n, device=samples.device)[:k] if n >= k else torch.randint(0, n, (k,), device=samples.device)
    means = samples[idx].clone()
    counts = torch.ones(k, device=samples.device)
    for _ in range(iters):
        assign = torch.cdist(samples, means).argmin(dim=1)
        counts = torch.bincount(assign, minlength=k).float()
        sums = torch.zeros_like(means).index_add_(0, assign, samples)
        means = torch.where(counts[:, None] > 0, sums / counts.clamp(min=1)[:, None], means)
    return means, counts


class EuclideanCodebook(nn.Module):
    """Nearest-neighbour codebook.  In training, ``cluster_size`` and ``embed_sum`` follow the assignments by exponential moving
    average and the codes are their (Laplace-smoothed) ratio — no gradient reaches the codebook; the encoder receives a
    commitment loss and the straight-through estimate.  Codes whose smoothed usage falls under ``threshold_ema_dead_code`` are
    re-seeded from the current batch."""

    def __init__(self, codebook_size: int, codebook_dim: int, decay: float = 0.99, threshold_ema_dead_code: Optional[float] = 2.0,
                 kmeans_iters: Optional[int] = 10, epsilon: float = 1e-5):
        super().__init__()
        self.K, self.D, self.decay, self.dead, self.kmeans_iters, self.eps = codebook_size, codebook_dim, decay, threshold_ema_dead_code, kmeans_iters, epsilon
        self.register_buffer("initialized", torch.tensor(0.0 if kmeans_iters else 1.0))
        self.register_buffer("cluster_size", torch.zeros(codebook_size))
        init = torch.zeros(codebook_size, codebook_dim) if kmeans_iters else torch.randn(codebook_size, codebook_dim) / math.sqrt(codebook_dim)
        self.register_buffer("codes", init.clone())
        self.register_buffer("codes_avg", init.clone())

    @torch.no_grad()
    def _init_codes(self, flat: torch.Tensor):
        if bool(self.initialized):
            return
        means, counts = _k_means(flat.float(), self.K, self.kmeans_iters)
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.broadcast(means, 0)
            torch.distributed.broadcast(counts, 0)
        self.codes.copy_(means)
        self.codes_avg.copy_(means)
        self.cluster_size.copy_(counts)
        self.initialized.fill_(1.0)

    @torch.no_grad()
    def _update(self, flat: torch.Tensor, idx: torch.Tensor):
        onehot = F.one_hot(idx, self.K).float()
        counts, sums = onehot.sum(0), onehot.t() @ flat.float()
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.all_reduce(counts)
            torch.distributed.all_reduce(sums)
        self.cluster_size.mul_(self.decay).add_(counts, alpha=1 - self.decay)
        self.codes_avg.mul_(self.decay).add_(sums, alpha=1 - self.decay)
        n = self.cluster_size.sum()
        smooth = (self.cluster_size + self.eps) / (n + self.K * self.eps) * n
        self.codes.copy_(self.codes_avg / smooth.unsqueeze(1))
        if self.dead is not None:
            dead = self.cluster_size < self.dead
            if bool(dead.any()) and flat.shape[0] > 0:
                pick = flat[torch.randint(0, flat.shape[0], (int(dead.sum()),), device=flat.device)].float()
                if torch.distributed.is_available() and torch.distributed.is_initialized():
                    torch.distributed.broadcast(pick, 0)
                self.codes[dead] = pick
                self.codes_avg[dead] = pick * self.dead
                self.cluster_size[dead] = self.dead

    def encode(self, x: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        """[B, D, T] -> indices [B, T] (0 beyond the lengths)."""
        flat = x.transpose(1, 2).reshape(-1, self.D).float()
        idx = torch.cdist(flat, self.codes).argmin(dim=1).view(x.shape[0], x.shape[2])
        return idx * (torch.arange(x.shape[2], device=x.device)[None, :] < lens[:, None])

    def decode(self, idx: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        return mask_by_length(F.embedding(idx, self.codes).transpose(1, 2), lens)

    def forward(self, x: torch.Tensor, lens: torch.Tensor):
        """-> (dequantised with straight-through gradient [B, D, T], indices [B, T], commitment loss)."""
        valid = (torch.arange(x.shape[2], device=x.device)[None, :] < lens[:, None])
        flat_valid = x.transpose(1, 2)[valid]
        if self.training:
            self._init_codes(flat_valid.detach())
        idx = self.encode(x, lens)
        if self.training:
            self._update(flat_valid.detach(), idx[valid])
        deq = self.decode(idx, lens)
        commit = ((x - deq.detach()).pow(2).mean(dim=1) * valid).sum() / valid.sum().clamp(min=1)
        return x + (deq - x).detach(), idx, commit


class ResidualVectorQuantizer(nn.Module):
    """``num_codebooks`` codebooks on successive residuals; ``forward`` returns ``(dequantised [B, D, T], indices [N, B, T], commit
    loss)`` — the index layout of ``GroupFiniteScalarQuantizer``, so the codec model can use either."""

    def __init__(self, num_codebooks: int = 8, codebook_size: int = 1024, codebook_dim: int = 128, decay: float = 0.99, threshold_ema_dead_code: Optional[float] = 2.0,
                 kmeans_iters: Optional[int] = 10, commit_loss_scale: float = 1.0):
        super().__init__()
        self.books = nn.ModuleList([EuclideanCodebook(codebook_size, codebook_dim, decay, threshold_ema_dead_code, kmeans_iters) for _ in range(num_codebooks)])
        self.num_groups = self.num_codebooks = num_codebooks
        self.codebook_size, self.commit_scale = codebook_size, commit_loss_scale
        self.commit_loss = torch.tensor(0.0)

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        res, out, ids, commit = inputs, 0, [], 0.0
        for b in self.books:
            q, i, c = b(res, input_len)
            res = res - q.detach()
            out = out + q
            ids.append(i)
            commit = commit + c
        self.commit_loss = self.commit_scale * commit / len(self.books)
        # straight-through over the whole stack: value = sum of the levels, gradient = identity to the input
        return inputs + (out - inputs).detach(), torch.stack(ids, dim=0)

    def encode(self, inputs, input_len):
        res, ids = inputs, []
        for b in self.books:
            i = b.encode(res, input_len)
            res = res - b.decode(i, input_len)
            ids.append(i)
        return torch.stack(ids, dim=0)

    def decode(self, indices, input_len):
        return sum(b.decode(indices[k], input_len) for k, b in enumerate(self.books))


class GroupResidualVectorQuantizer(nn.Module):
    """The channels are split into ``num_groups`` groups, each with its own residual quantiser; indices are concatenated along
    the codebook axis."""

    def __init__(self, num_codebooks: int = 8, num_groups: int = 2, codebook_size: int = 1024, codebook_dim: int = 128, **kw):
        super().__init__()
        if num_codebooks % num_groups or codebook_dim % num_groups:
            raise ValueError("num_codebooks and codebook_dim must be divisible by num_groups")
        self.groups = nn.ModuleList([ResidualVectorQuantizer(num_codebooks // num_groups, codebook_size, codebook_dim // num_groups, **kw) for _ in range(num_groups)])
        self.num_groups, self.num_codebooks, self.codebook_size = num_groups, num_codebooks, codebook_size
        self.per = num_codebooks // num_groups

    @property
    def commit_loss(self):
        return sum(g.commit_loss for g in self.groups) / len(self.groups)

    def forward(self, inputs, input_len):
        outs, ids = zip(*[g(x, input_len) for g, x in zip(self.groups, inputs.chunk(len(self.groups), dim=1))])
        return torch.cat(outs, dim=1), torch.cat(ids, dim=0)

    def encode(self, inputs, input_len):
        return torch.cat([g.encode(x, input_len) for g, x in zip(self.groups, inputs.chunk(len(self.groups), dim=1))], dim=0)

    def decode(self, indices, input_len):
        return torch.cat([g.decode(indices[k * self.per:(k + 1) * self.per], input_len) for k, g in enumerate(self.groups)], dim=1)

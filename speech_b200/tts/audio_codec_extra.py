"""More parts of the neural audio codec: causal (streamable) convolutions and decoder, multi-band and multi-resolution STFT
discriminators, a discriminator on the features of a speech foundation model, the loss classes of codec training, a speaker
encoder, and conversion of codec indices between quantizer layouts.

References (behaviour): ``tts/modules/audio_codec_modules.py`` (``CausalConv1dNorm`` :704, ``CausalConvTranspose1dNorm`` :642,
``CausalHiFiGANDecoder`` :2200, ``MultiBandDiscriminatorSTFT`` :1128, ``MultiResolutionDiscriminatorSTFT`` :1197,
``SLMDiscriminator`` :92, ``ResNetSpeakerEncoder`` :433, ``VectorQuantizerIndexConverter`` :3022), ``tts/losses/audio_codec_loss.py``
(``TimeDomainLoss``, ``MultiResolutionMelLoss``, ``SISDRLoss``, ``RelativeFeatureMatchingLoss``, hinged / squared GAN losses, MMD
losses).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .audio_codec import FiniteScalarQuantizer, GroupFiniteScalarQuantizer, mask_by_length


# ------------------------------------------------------------------------------------------------ causal layers
class CausalConv1d(nn.Module):
    """Convolution that sees no future sample: ``(k - 1) * dilation - (stride - 1)`` zeros on the left.  ``forward_stream`` carries
    the left context between chunks so that chunked and whole-signal outputs are equal."""

    def __init__(self, cin: int, cout: int, kernel_size: int, stride: int = 1, dilation: int = 1):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, kernel_size, stride=stride, dilation=dilation)
        self.left = (kernel_size - 1) * dilation - (stride - 1)
        self.stride = stride

    def forward(self, x):
        return self.conv(F.pad(x, (self.left, 0)))

    def forward_stream(self, x, state: Optional[torch.Tensor]):
        if state is None:
            state = x.new_zeros(x.shape[0], x.shape[1], self.left)
        z = torch.cat([state, x], dim=-1)
        y = self.conv(z)
        consumed = y.shape[-1] * self.stride
        return y, z[..., consumed:]


class CausalConvTranspose1d(nn.Module):
    """Up-sampling by ``stride`` without look-ahead: a transposed convolution of kernel ``2 * stride`` whose trailing ``stride``
    outputs (which later inputs would still add to) are held back; in streaming they are carried as an overlap."""

    def __init__(self, cin: int, cout: int, stride: int):
        super().__init__()
        self.tconv = nn.ConvTranspose1d(cin, cout, 2 * stride, stride=stride)
        self.stride = stride

    def forward(self, x):
        return self.tconv(x)[..., : x.shape[-1] * self.stride]

    def forward_stream(self, x, state: Optional[torch.Tensor]):
        y = self.tconv(x)                                            # [.., (T + 1) * stride]
        if state is not None:
            head = y[..., : self.stride] + (state - self.tconv.bias.view(1, -1, 1) if self.tconv.bias is not None else state)
            y = torch.cat([head, y[..., self.stride:]], dim=-1)
        return y[..., : x.shape[-1] * self.stride], y[..., x.shape[-1] * self.stride:]


class _CausalResBlock(nn.Module):
    def __init__(self, ch: int, kernel_size: int, dilations: Sequence[int]):
        super().__init__()
        self.c1 = nn.ModuleList([CausalConv1d(ch, ch, kernel_size, dilation=d) for d in dilations])
        self.c2 = nn.ModuleList([CausalConv1d(ch, ch, kernel_size) for _ in dilations])

    def forward(self, x):
        for a, b in zip(self.c1, self.c2):
            x = x + b(F.leaky_relu(a(F.leaky_relu(x, 0.1)), 0.1))
        return x

    def forward_stream(self, x, state):
        state = state or [None] * (2 * len(self.c1))
        new = []
        for i, (a, b) in enumerate(zip(self.c1, self.c2)):
            y, s1 = a.forward_stream(F.leaky_relu(x, 0.1), state[2 * i])
            y, s2 = b.forward_stream(F.leaky_relu(y, 0.1), state[2 * i + 1])
            x = x + y
            new += [s1, s2]
        return x, new


class CausalHiFiGANDecoder(nn.Module):
    """Latents ``[B, D, T]`` -> audio ``[B, T * prod(rates)]`` with causal layers only.  ``decode_stream(latents_chunk, state)``
    produces exactly the samples the whole-sequence ``forward`` would produce for those frames, so codec tokens can be turned into
    sound as they are generated."""

    def __init__(self, input_dim: int = 32, up_sample_rates=(8, 4, 4, 2), base_channels: int = 256, in_kernel_size: int = 7,
                 out_kernel_size: int = 3, resblock_kernel_sizes=(3, 7), resblock_dilation_sizes=(1, 3)):
        super().__init__()
        self.rates = list(up_sample_rates)
        self.pre = CausalConv1d(input_dim, base_channels, in_kernel_size)
        ch = base_channels
        self.up, self.res = nn.ModuleList(), nn.ModuleList()
        for r in self.rates:
            self.up.append(CausalConvTranspose1d(ch, ch // 2, r))
            ch //= 2
            self.res.append(nn.ModuleList([_CausalResBlock(ch, k, resblock_dilation_sizes) for k in resblock_kernel_sizes]))
        self.post = CausalConv1d(ch, 1, out_kernel_size)

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        x = self.pre(inputs)
        for up, blocks in zip(self.up, self.res):
            x = up(F.leaky_relu(x, 0.1))
            x = sum(b(x) for b in blocks) / len(blocks)
        audio = torch.tanh(self.post(F.leaky_relu(x, 0.1))).squeeze(1)
        lens = input_len * int(math.prod(self.rates))
        return mask_by_length(audio, lens.clamp(max=audio.shape[-1])), lens.clamp(max=audio.shape[-1])

    def decode_stream(self, inputs: torch.Tensor, state: Optional[dict] = None) -> Tuple[torch.Tensor, dict]:
        st = state or {}
        new: dict = {}
        x, new["pre"] = self.pre.forward_stream(inputs, st.get("pre"))
        for i, (up, blocks) in enumerate(zip(self.up, self.res)):
            x, new[f"up{i}"] = up.forward_stream(F.leaky_relu(x, 0.1), st.get(f"up{i}"))
            outs = []
            for j, b in enumerate(blocks):
                y, new[f"res{i}_{j}"] = b.forward_stream(x, st.get(f"res{i}_{j}"))
                outs.append(y)
            x = sum(outs) / len(outs)
        y, new["post"] = self.post.forward_stream(F.leaky_relu(x, 0.1), st.get("post"))
        return torch.tanh(y).squeeze(1), new


# ------------------------------------------------------------------------------------------------ discriminators
class DiscriminatorSTFT(nn.Module):
    """2-D convolutions over a (real, imag) spectrogram restricted to frequency bands ``[lo, hi)`` given as fractions of the
    spectrum; one convolution stack per band, outputs concatenated along frequency."""

    def __init__(self, resolution=(1024, 256, 1024), bands=((0.0, 1.0),), ch: int = 32):
        super().__init__()
        self.n_fft, self.hop, self.win = resolution
        self.bands = [tuple(b) for b in bands]

        def stack():
            return nn.ModuleList([nn.Conv2d(2, ch, (3, 9), padding=(1, 4)), nn.Conv2d(ch, ch, (3, 9), stride=(1, 2), dilation=(1, 1), padding=(1, 4)),
                                  nn.Conv2d(ch, ch, (3, 9), stride=(1, 2), dilation=(2, 1), padding=(2, 4)),
                                  nn.Conv2d(ch, ch, (3, 3), padding=(1, 1))])
        self.stacks = nn.ModuleList([stack() for _ in self.bands])
        self.post = nn.Conv2d(ch, 1, (3, 3), padding=(1, 1))

    def spectrogram(self, audio: torch.Tensor) -> torch.Tensor:
        w = torch.hann_window(self.win, device=audio.device)
        s = torch.stft(audio.float(), self.n_fft, self.hop, self.win, w, return_complex=True)       # [B, F, T]
        return torch.view_as_real(s).permute(0, 3, 2, 1)                                           # [B, 2, T, F]

    def forward(self, audio: torch.Tensor):
        spec = self.spectrogram(audio)
        Fq = spec.shape[-1]
        outs, fmaps = [], []
        for (lo, hi), stack in zip(self.bands, self.stacks):
            x = spec[..., int(lo * Fq): max(int(lo * Fq) + 1, int(hi * Fq))]
            for c in stack:
                x = F.leaky_relu(c(x), 0.1)
                fmaps.append(x)
            outs.append(x)
        x = self.post(torch.cat(outs, dim=-1))
        fmaps.append(x)
        return x.flatten(1), fmaps


class MultiBandDiscriminatorSTFT(DiscriminatorSTFT):
    def __init__(self, resolution=(1024, 256, 1024), stft_bands=((0.0, 0.1), (0.1, 0.25), (0.25, 0.5), (0.5, 0.75), (0.75, 1.0)), ch: int = 32):
        super().__init__(resolution, stft_bands, ch)


class MultiResolutionDiscriminatorSTFT(nn.Module):
    def __init__(self, resolutions=((512, 128, 512), (1024, 256, 1024), (2048, 512, 2048)), stft_bands=((0.0, 0.1), (0.1, 0.25), (0.25, 0.5), (0.5, 0.75), (0.75, 1.0)),
                 ch: int = 32):
        super().__init__()
        self.discs = nn.ModuleList([MultiBandDiscriminatorSTFT(r, stft_bands, ch) for r in resolutions])

    def forward(self, audio_real: torch.Tensor, audio_gen: torch.Tensor):
        outs = [(d(audio_real), d(audio_gen)) for d in self.discs]
        return ([o[0][0] for o in outs], [o[1][0] for o in outs], [o[0][1] for o in outs], [o[1][1] for o in outs])


class SLMDiscriminator(nn.Module):
    """Discriminator on the hidden states of a frozen speech foundation model: ``feature_extractor(audio_16k) -> [B, L, T, D]``
    (all layers stacked) or ``[B, T, D]``; the layers are flattened into channels and scored by 1-D convolutions.  Judging speech
    in a learned feature space pushes the codec towards intelligible output."""

    def __init__(self, feature_extractor: Callable[[torch.Tensor], torch.Tensor], slm_hidden: int = 768, slm_layers: int = 13,
                 initial_channel: int = 64, input_sr: int = 22050, slm_sr: int = 16000):
        super().__init__()
        object.__setattr__(self, "_extract", feature_extractor)           # frozen, not a sub-module
        self.input_sr, self.slm_sr = input_sr, slm_sr
        c = initial_channel
        self.pre = nn.Conv1d(slm_hidden * slm_layers, c, 1)
        self.convs = nn.ModuleList([nn.Conv1d(c, 2 * c, 5, padding=2), nn.Conv1d(2 * c, 4 * c, 5, padding=2), nn.Conv1d(4 * c, 4 * c, 5, padding=2)])
        self.post = nn.Conv1d(4 * c, 1, 3, padding=1)

    def _features(self, audio: torch.Tensor) -> torch.Tensor:
        if self.input_sr != self.slm_sr:
            n = int(round(audio.shape[-1] * self.slm_sr / self.input_sr))
            audio = F.interpolate(audio.unsqueeze(1), size=n, mode="linear", align_corners=False).squeeze(1)
        with torch.no_grad():
            h = self._extract(audio)
        if h.dim() == 4:
            B, L, T, D = h.shape
            h = h.permute(0, 1, 3, 2).reshape(B, L * D, T)
        else:
            h = h.transpose(1, 2)
        return h

    def _score(self, h):
        fmaps = []
        x = self.pre(h)
        for c in self.convs:
            x = F.leaky_relu(c(x), 0.1)
            fmaps.append(x)
        x = self.post(x)
        return x.flatten(1), fmaps

    def forward(self, audio_real, audio_gen):
        (sr, fr), (sg, fg) = self._score(self._features(audio_real)), self._score(self._features(audio_gen))
        return [sr], [sg], [fr], [fg]


# ------------------------------------------------------------------------------------------------ speaker encoder
class _SEBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False), nn.BatchNorm2d(cout)
        self.c2, self.b2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False), nn.BatchNorm2d(cout)
        self.se = nn.Sequential(nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(cout, max(1, cout // 8)), nn.ReLU(), nn.Linear(max(1, cout // 8), cout), nn.Sigmoid())
        self.skip = None if (stride == 1 and cin == cout) else nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        y = self.b2(self.c2(F.relu(self.b1(self.c1(x)))))
        y = y * self.se(y)[:, :, None, None]
        return F.relu(y + (x if self.skip is None else self.skip(x)))


class ResNetSpeakerEncoder(nn.Module):
    """Squeeze-excitation ResNet over log-mel frames with attentive statistics pooling -> an L2-normalised speaker vector."""

    def __init__(self, n_mels: int = 64, channels=(32, 64, 128, 256), proj_dim: int = 512, sample_rate: int = 16000):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        self.n_fft, self.hop = 512, 160
        self.register_buffer("fb", torch.as_tensor(mel_filterbank(sample_rate, self.n_fft, n_mels), dtype=torch.float32), persistent=False)
        self.stem = nn.Sequential(nn.Conv2d(1, channels[0], 3, 1, 1, bias=False), nn.BatchNorm2d(channels[0]), nn.ReLU())
        blocks, cin = [], channels[0]
        for i, c in enumerate(channels):
            blocks.append(_SEBlock(cin, c, 1 if i == 0 else 2))
            cin = c
        self.blocks = nn.Sequential(*blocks)
        fdim = channels[-1] * math.ceil(n_mels / 2 ** (len(channels) - 1))
        self.att = nn.Sequential(nn.Conv1d(fdim, 128, 1), nn.ReLU(), nn.BatchNorm1d(128), nn.Conv1d(128, fdim, 1), nn.Softmax(dim=2))
        self.fc = nn.Linear(2 * fdim, proj_dim)

    def forward(self, audio: torch.Tensor, audio_len: Optional[torch.Tensor] = None) -> torch.Tensor:
        w = torch.hann_window(400, device=audio.device)
        p = torch.stft(audio.float(), self.n_fft, self.hop, 400, w, return_complex=True).abs().pow(2)
        mel = torch.log(torch.matmul(self.fb.to(p.dtype), p) + 1e-6)
        mel = mel - mel.mean(dim=-1, keepdim=True)
        x = self.blocks(self.stem(mel.unsqueeze(1)))                 # [B, C, F', T']
        x = x.flatten(1, 2)
        a = self.att(x)
        mu = (x * a).sum(2)
        sd = ((x.pow(2) * a).sum(2) - mu.pow(2)).clamp(min=1e-5).sqrt()
        return F.normalize(self.fc(torch.cat([mu, sd], dim=1)), dim=-1)


# ------------------------------------------------------------------------------------------------ losses
def _time_mask(lens: Optional[torch.Tensor], T: int, device) -> Optional[torch.Tensor]:
    return None if lens is None else (torch.arange(T, device=device)[None, :] < lens[:, None]).float()


class TimeDomainLoss(nn.Module):
    """Mean absolute error between waveforms over the valid samples."""

    def forward(self, audio_real, audio_gen, audio_len=None):
        T = min(audio_real.shape[-1], audio_gen.shape[-1])
        d = (audio_real[..., :T] - audio_gen[..., :T]).abs()
        m = _time_mask(audio_len, T, d.device)
        return d.mean() if m is None else (d * m).sum() / m.sum().clamp(min=1)


class MultiResolutionMelLoss(nn.Module):
    """L1 + L2 distance between log-mel spectrograms at several STFT resolutions (window lengths ``resolutions``, mel bins
    ``mel_dims``), averaged over resolutions."""

    def __init__(self, sample_rate: int, resolutions=((32, 8), (64, 16), (128, 32), (256, 64), (512, 128), (1024, 256), (2048, 512)),
                 mel_dims=(5, 10, 20, 40, 80, 160, 320), log_guard: float = 1.0, l1_scale: float = 1.0, l2_scale: float = 1.0):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        if len(resolutions) != len(mel_dims):
            raise ValueError("one mel dimension per resolution")
        self.res = [tuple(r) for r in resolutions]
        self.guard, self.l1, self.l2 = log_guard, l1_scale, l2_scale
        for i, ((win, hop), n) in enumerate(zip(self.res, mel_dims)):
            self.register_buffer(f"fb{i}", torch.as_tensor(mel_filterbank(sample_rate, win, min(n, win // 2)), dtype=torch.float32), persistent=False)

    def _mel(self, x, i):
        win, hop = self.res[i]
        w = torch.hann_window(win, device=x.device)
        s = torch.stft(x.float(), win, hop, win, w, return_complex=True).abs()
        return torch.log(torch.matmul(getattr(self, f"fb{i}").to(s.dtype), s) + self.guard)

    def forward(self, audio_real, audio_gen, audio_len=None):
        T = min(audio_real.shape[-1], audio_gen.shape[-1])
        if audio_len is not None:
            m = _time_mask(audio_len, T, audio_real.device)
            audio_real, audio_gen = audio_real[..., :T] * m, audio_gen[..., :T] * m
        loss = 0.0
        for i in range(len(self.res)):
            a, b = self._mel(audio_real[..., :T], i), self._mel(audio_gen[..., :T], i)
            loss = loss + self.l1 * (a - b).abs().mean() + self.l2 * (a - b).pow(2).mean()
        return loss / len(self.res)


class SISDRLoss(nn.Module):
    """Negative scale-invariant signal-to-distortion ratio in dB (clipped at ``clip_max``), mean over the batch."""

    def __init__(self, epsilon: float = 1e-8, clip_max: Optional[float] = 30.0):
        super().__init__()
        self.eps, self.clip = epsilon, clip_max

    def forward(self, audio_real, audio_gen, audio_len=None):
        T = min(audio_real.shape[-1], audio_gen.shape[-1])
        t, e = audio_real[..., :T].float(), audio_gen[..., :T].float()
        m = _time_mask(audio_len, T, t.device)
        if m is not None:
            n = m.sum(-1, keepdim=True).clamp(min=1)
            t, e = (t - (t * m).sum(-1, keepdim=True) / n) * m, (e - (e * m).sum(-1, keepdim=True) / n) * m
        else:
            t, e = t - t.mean(-1, keepdim=True), e - e.mean(-1, keepdim=True)
        proj = (e * t).sum(-1, keepdim=True) / (t.pow(2).sum(-1, keepdim=True) + self.eps) * t
        sdr = 10 * torch.log10(proj.pow(2).sum(-1) / ((e - proj).pow(2).sum(-1) + self.eps) + self.eps)
        if self.clip is not None:
            sdr = sdr.clamp(max=self.clip)
        return -sdr.mean()


class RelativeFeatureMatchingLoss(nn.Module):
    """Feature matching where every feature map's L1 distance is divided by the mean magnitude of the real features, so that deep
    and shallow layers weigh alike."""

    def __init__(self, div_guard: float = 1e-3):
        super().__init__()
        self.g = div_guard

    def forward(self, fmaps_real, fmaps_gen):
        loss, n = 0.0, 0
        for fr, fg in zip(fmaps_real, fmaps_gen):
            for a, b in zip(fr, fg):
                loss = loss + (b - a.detach()).abs().mean() / (a.detach().abs().mean() + self.g)
                n += 1
        return loss / max(n, 1)


class GeneratorHingedLoss(nn.Module):
    def forward(self, disc_scores_gen):
        return sum(F.relu(1 - s).mean() for s in disc_scores_gen) / len(disc_scores_gen)


class GeneratorSquaredLoss(nn.Module):
    def forward(self, disc_scores_gen):
        return sum((1 - s).pow(2).mean() for s in disc_scores_gen) / len(disc_scores_gen)


class DiscriminatorHingedLoss(nn.Module):
    def forward(self, disc_scores_real, disc_scores_gen):
        return sum(F.relu(1 - r).mean() + F.relu(1 + g).mean() for r, g in zip(disc_scores_real, disc_scores_gen)) / len(disc_scores_real)


class DiscriminatorSquaredLoss(nn.Module):
    def forward(self, disc_scores_real, disc_scores_gen):
        return sum((1 - r).pow(2).mean() + g.pow(2).mean() for r, g in zip(disc_scores_real, disc_scores_gen)) / len(disc_scores_real)


class MMDLoss(nn.Module):
    """Maximum mean discrepancy between two sets of vectors with a mixture of Gaussian kernels (bandwidths as multiples of the
    median pairwise distance): zero when the sets follow the same distribution.  Used to keep codebook usage / embeddings of
    different domains aligned."""

    def __init__(self, kernel_scales=(0.25, 0.5, 1.0, 2.0, 4.0)):
        super().__init__()
        self.scales = list(kernel_scales)

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        x, y = x.reshape(-1, x.shape[-1]).float(), y.reshape(-1, y.shape[-1]).float()
        z = torch.cat([x, y], 0)
        d2 = torch.cdist(z, z).pow(2)
        med = d2[d2 > 0].median().detach().clamp(min=1e-6) if bool((d2 > 0).any()) else d2.new_tensor(1.0)
        k = sum(torch.exp(-d2 / (s * med)) for s in self.scales) / len(self.scales)
        n, m = x.shape[0], y.shape[0]
        kxx, kyy, kxy = k[:n, :n], k[n:, n:], k[:n, n:]
        off = lambda a, c: (a.sum() - a.diagonal().sum()) / max(1, c * (c - 1))  # noqa: E731
        return off(kxx, n) + off(kyy, m) - 2 * kxy.mean()


# ------------------------------------------------------------------------------------------------ index conversion
class VectorQuantizerIndexConverter(nn.Module):
    """Re-express codec indices of one finite-scalar-quantizer layout in another with the same total number of scalar dimensions
    (e.g. 8 groups x 4 levels -> 4 groups x 8 levels): indices -> per-dimension codes -> indices, without touching audio."""

    def __init__(self, vector_quantizer_original: GroupFiniteScalarQuantizer, vector_quantizer_new: GroupFiniteScalarQuantizer):
        super().__init__()
        self.vo, self.vn = vector_quantizer_original, vector_quantizer_new
        lo = [l for q in self.vo.fsqs for l in self._levels(q)]
        ln = [l for q in self.vn.fsqs for l in self._levels(q)]
        if lo != ln:
            raise ValueError(f"the quantizers do not share their per-dimension levels: {lo} vs {ln}")

    @staticmethod
    def _levels(q: FiniteScalarQuantizer) -> List[int]:
        return [int(v) for v in q.num_levels.flatten().tolist()]

    @classmethod
    def _digits(cls, q: FiniteScalarQuantizer, idx: torch.Tensor) -> torch.Tensor:
        out = []
        for l in cls._levels(q):
            out.append(idx % l)
            idx = idx // l
        return torch.stack(out, dim=1)                                # [B, D, T]

    @classmethod
    def _index(cls, q: FiniteScalarQuantizer, digits: torch.Tensor) -> torch.Tensor:
        idx, mul = torch.zeros_like(digits[:, 0]), 1
        for d, l in enumerate(cls._levels(q)):
            idx = idx + digits[:, d] * mul
            mul *= l
        return idx

    def convert_original_to_new(self, audio_tokens: torch.Tensor, audio_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[G_old, B, T] -> [G_new, B, T]`` (the layout the quantizers' ``encode`` / ``decode`` use)."""
        digits = torch.cat([self._digits(q, audio_tokens[g]) for g, q in enumerate(self.vo.fsqs)], dim=1)
        out, o = [], 0
        for q in self.vn.fsqs:
            out.append(self._index(q, digits[:, o:o + q.dim]))
            o += q.dim
        return torch.stack(out, dim=0)

    def convert_new_to_original(self, audio_tokens: torch.Tensor, audio_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
        return VectorQuantizerIndexConverter(self.vn, self.vo).convert_original_to_new(audio_tokens, audio_lens)

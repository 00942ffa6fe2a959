"""Residual-VQ variational audio codec of the EAR-TTS speech generator: waveform <-> continuous latents <-> residual codes.

``Wav2Latent`` (STFT -> causal ConvNeXt stages with strided down-sampling -> latent), ``ProbabilisticRVQ`` (``depth`` codebooks
applied to successive residuals, with a tracked residual variance: the quantiser is read as a mixture of isotropic Gaussians whose
``log_std`` the speech LM's mixture-of-Gaussians head uses), ``Latent2Wav`` (mirror image ending in an inverse STFT).  Every layer
is causal, so ``RVQVAEModel.decode_stream`` turns latents into sound chunk by chunk with the samples of a whole-sequence decode.

Reference: ``speechlm2/modules/ear_tts_vae_codec.py`` (``ConvNeXt1d``, ``PreTrainedProbabilisticVQ``, ``Wav2Latent``, ``Latent2Wav``,
``RVQVAEModel``).  The reference loads frozen pre-trained weights; here the model also trains (``training_loss``, ``update_codebooks``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..tts.audio_codec_extra import CausalConv1d, CausalConvTranspose1d

__all__ = ["ConvNeXt1d", "Latent2Wav", "ProbabilisticRVQ", "RVQVAEModel", "Wav2Latent"]


class ConvNeXt1d(nn.Module):
    """Depthwise causal convolution -> LayerNorm over channels -> 4x pointwise expansion with GELU -> projection scaled by a
    learned per-channel factor, added to the input."""

    def __init__(self, channels: int, kernel_size: int = 7, expansion: int = 4, layer_scale: float = 1e-2):
        super().__init__()
        self.dw = CausalConv1d(channels, channels, kernel_size)
        self.dw.conv = nn.Conv1d(channels, channels, kernel_size, groups=channels)
        self.norm = nn.LayerNorm(channels)
        self.pw1, self.pw2 = nn.Linear(channels, expansion * channels), nn.Linear(expansion * channels, channels)
        self.gamma = nn.Parameter(torch.full((channels,), layer_scale))

    def _rest(self, x, y):
        y = self.pw2(F.gelu(self.pw1(self.norm(y.transpose(1, 2)))))
        return x + (self.gamma * y).transpose(1, 2)

    def forward(self, x):
        return self._rest(x, self.dw(x))

    def forward_stream(self, x, state):
        y, state = self.dw.forward_stream(x, state)
        return self._rest(x, y), state


def _stft_causal(wav: torch.Tensor, n_fft: int, hop: int) -> torch.Tensor:
    """[B, T] -> [B, n_fft + 2, T / hop]: real and imaginary parts; frame t ends at sample (t + 1) * hop (left zero padding)."""
    w = torch.hann_window(n_fft, device=wav.device, dtype=torch.float32)
    x = F.pad(wav.float(), (n_fft - hop, 0))
    s = torch.stft(x, n_fft, hop, n_fft, w, center=False, return_complex=True)
    return torch.cat([s.real, s.imag], dim=1)


class Wav2Latent(nn.Module):
    def __init__(self, latent_size: int = 64, n_fft: int = 32, hop_length: int = 8, base_hidden_size: int = 64, channel_mult: Sequence[int] = (1, 2, 4),
                 rates: Sequence[int] = (4, 4, 4), num_blocks: int = 2, kernel_size: int = 7):
        super().__init__()
        if len(channel_mult) != len(rates):
            raise ValueError("one channel multiplier per down-sampling rate")
        self.n_fft, self.hop = n_fft, hop_length
        ch = base_hidden_size * channel_mult[0]
        self.inp = CausalConv1d(n_fft + 2, ch, 3)
        stages = []
        for i, r in enumerate(rates):
            stages += [ConvNeXt1d(ch, kernel_size) for _ in range(num_blocks)]
            nxt = base_hidden_size * channel_mult[min(i + 1, len(channel_mult) - 1)]
            stages.append(CausalConv1d(ch, nxt, 2 * r, stride=r))
            ch = nxt
        self.stages = nn.ModuleList(stages)
        self.out = nn.Sequential(nn.GroupNorm(1, ch), nn.Conv1d(ch, latent_size, 1))
        self.ratio = hop_length * int(math.prod(rates))

    def forward(self, wav: torch.Tensor) -> torch.Tensor:
        """[B, 1, T] (T a multiple of ``ratio``) -> [B, T / ratio, latent]."""
        x = self.inp(_stft_causal(wav[:, 0], self.n_fft, self.hop))
        for m in self.stages:
            x = m(x)
        return self.out(x).transpose(1, 2)


class Latent2Wav(nn.Module):
    def __init__(self, latent_size: int = 64, n_fft: int = 32, hop_length: int = 8, base_hidden_size: int = 64, channel_mult: Sequence[int] = (4, 2, 1),
                 rates: Sequence[int] = (4, 4, 4), num_blocks: int = 2, kernel_size: int = 7):
        super().__init__()
        self.n_fft, self.hop = n_fft, hop_length
        ch = base_hidden_size * channel_mult[0]
        self.inp = CausalConv1d(latent_size, ch, 3)
        stages = []
        for i, r in enumerate(rates):
            nxt = base_hidden_size * channel_mult[min(i + 1, len(channel_mult) - 1)]
            stages.append(CausalConvTranspose1d(ch, nxt, r))
            ch = nxt
            stages += [ConvNeXt1d(ch, kernel_size) for _ in range(num_blocks)]
        self.stages = nn.ModuleList(stages)
        self.norm = nn.LayerNorm(ch)
        self.out = nn.Linear(ch, n_fft + 2)
        self.ratio = hop_length * int(math.prod(rates))

    # .............................................................. inverse STFT by overlap-add, streamable
    def _frames(self, spec: torch.Tensor) -> torch.Tensor:
        F_ = self.n_fft // 2 + 1
        c = torch.complex(spec[:, :F_].float(), spec[:, F_:].float())
        w = torch.hann_window(self.n_fft, device=spec.device, dtype=torch.float32)
        return torch.fft.irfft(c, n=self.n_fft, dim=1) * w[None, :, None]           # [B, n_fft, T]

    def _overlap_add(self, frames: torch.Tensor, carry: Optional[Tuple[torch.Tensor, torch.Tensor]]):
        B, N, T = frames.shape
        L = (T - 1) * self.hop + N
        w = torch.hann_window(N, device=frames.device, dtype=torch.float32)
        y = F.fold(frames, (1, L), (1, N), stride=(1, self.hop)).reshape(B, L)
        env = F.fold((w * w)[None, :, None].expand(1, N, T), (1, L), (1, N), stride=(1, self.hop)).reshape(1, L)
        if carry is not None:
            k = carry[0].shape[-1]
            y = torch.cat([y[:, :k] + carry[0], y[:, k:]], dim=1)
            env = torch.cat([env[:, :k] + carry[1], env[:, k:]], dim=1)
        n = T * self.hop
        return y[:, :n] / env[:, :n].clamp(min=1e-3), (y[:, n:], env[:, n:])

    def _net(self, z, state: Optional[dict]):
        st, new = state or {}, {}
        stream = state is not None
        x = z.transpose(1, 2)
        if stream:
            x, new["inp"] = self.inp.forward_stream(x, st.get("inp"))
        else:
            x = self.inp(x)
        for i, m in enumerate(self.stages):
            if stream:
                x, new[i] = m.forward_stream(x, st.get(i))
            else:
                x = m(x)
        return self.out(self.norm(x.transpose(1, 2))).transpose(1, 2), new

    def forward(self, z: torch.Tensor, constrain_value_range: bool = True) -> torch.Tensor:
        """[B, T', latent] -> [B, 1, T' * ratio]."""
        spec, _ = self._net(z, None)
        wav, _ = self._overlap_add(self._frames(spec), None)
        return (wav.clamp(-1, 1) if constrain_value_range else wav).unsqueeze(1)

    def forward_stream(self, z: torch.Tensor, state: Optional[dict] = None, constrain_value_range: bool = True):
        state = state if state is not None else {"ola": None}
        spec, new = self._net(z, state)
        wav, new["ola"] = self._overlap_add(self._frames(spec), state.get("ola"))
        return (wav.clamp(-1, 1) if constrain_value_range else wav).unsqueeze(1), new


class ProbabilisticRVQ(nn.Module):
    """``depth`` codebooks of ``num_mixtures`` vectors; level i starts at norm ``(depth - i) / depth`` so that later levels model
    ever smaller residuals.  ``encode`` picks the nearest vector of each level for the running residual.  ``variance[i]`` follows
    the mean squared residual left after level i (exponential moving average during training)."""

    def __init__(self, channels: int, num_mixtures: int, depth: int = 1, ema_decay: float = 0.99):
        super().__init__()
        self.channels, self.num_mixtures, self.depth, self.decay = channels, num_mixtures, depth, ema_decay
        self.mus_list = nn.ParameterList([nn.Parameter(F.normalize(torch.randn(num_mixtures, channels), dim=1) * ((depth - i) / depth), requires_grad=False)
                                          for i in range(depth)])
        self.register_buffer("variance", torch.ones(depth))
        self.register_buffer("usage", torch.ones(depth, num_mixtures))

    @property
    def log_std(self) -> torch.Tensor:
        return 0.5 * torch.log(self.variance[-1])

    @staticmethod
    def _nearest(r: torch.Tensor, mus: torch.Tensor) -> torch.Tensor:
        d = r.pow(2).sum(-1, keepdim=True) + mus.pow(2).sum(-1) - 2 * r @ mus.t()
        return d.argmin(-1)

    def encode(self, z: torch.Tensor, return_z_q: bool = False):
        r, ids = z.float(), []
        for mus in self.mus_list:
            i = self._nearest(r, mus)
            r = r - F.embedding(i, mus)
            ids.append(i)
        return (ids, z - r.to(z.dtype)) if return_z_q else ids

    def decode(self, ids: Sequence[torch.Tensor]) -> torch.Tensor:
        z = 0
        for i, mus in zip(ids, self.mus_list):
            z = z + F.embedding(i, mus)
        return z

    @torch.no_grad()
    def update_codebooks(self, z: torch.Tensor):
        """One EMA k-means step per level on a batch of latents ``[..., C]`` (training only)."""
        r = z.detach().float().reshape(-1, self.channels)
        for lvl, mus in enumerate(self.mus_list):
            i = self._nearest(r, mus)
            onehot = F.one_hot(i, self.num_mixtures).float()
            cnt = onehot.sum(0)
            mean = (onehot.t() @ r) / cnt.clamp(min=1).unsqueeze(1)
            hit = cnt > 0
            mus.data[hit] = self.decay * mus.data[hit] + (1 - self.decay) * mean[hit]
            self.usage[lvl] = self.decay * self.usage[lvl] + (1 - self.decay) * cnt
            r = r - F.embedding(i, mus)
            self.variance[lvl] = self.decay * self.variance[lvl] + (1 - self.decay) * r.pow(2).mean()


class RVQVAEModel(nn.Module):
    """Config keys: ``latent_size, n_fft, hop_length, base_hidden_size, channel_mult, rates, num_blocks, kernel_size, codebook_size,
    num_quantizers``; ``wav_to_token_ratio`` = hop_length * prod(rates)."""

    defaults = dict(latent_size=64, n_fft=32, hop_length=8, base_hidden_size=64, channel_mult=(1, 2, 4), rates=(4, 4, 4), num_blocks=2, kernel_size=7,
                    codebook_size=256, num_quantizers=4, sample_rate=22050)

    def __init__(self, config: Optional[Dict[str, Any]] = None, trainable: bool = False):
        super().__init__()
        c = dict(self.defaults)
        c.update(dict(config or {}))
        self.config = c
        common = dict(latent_size=c["latent_size"], n_fft=c["n_fft"], hop_length=c["hop_length"], base_hidden_size=c["base_hidden_size"],
                      num_blocks=c["num_blocks"], kernel_size=c["kernel_size"])
        self.encoder = Wav2Latent(channel_mult=tuple(c["channel_mult"]), rates=tuple(c["rates"]), **common)
        self.prvq = ProbabilisticRVQ(c["latent_size"], c["codebook_size"], c["num_quantizers"])
        self.decoder = Latent2Wav(channel_mult=tuple(reversed(tuple(c["channel_mult"]))), rates=tuple(reversed(tuple(c["rates"]))), **common)
        self.wav_to_token_ratio = self.encoder.ratio
        if not trainable:
            for p in self.parameters():
                p.requires_grad = False

    def pad_to_ratio(self, wav: torch.Tensor) -> torch.Tensor:
        pad = (-wav.shape[-1]) % self.wav_to_token_ratio
        return F.pad(wav, (0, pad)) if pad else wav

    def ae_encode(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 3 or x.shape[1] != 1:
            raise ValueError(f"expected mono audio [B, 1, T], got {tuple(x.shape)}")
        if x.shape[2] % self.wav_to_token_ratio:
            raise ValueError(f"audio length {x.shape[2]} is not a multiple of wav_to_token_ratio {self.wav_to_token_ratio}: pad it (pad_to_ratio)")
        return self.encoder(x)

    def ae_decode(self, z: torch.Tensor, constrain_value_range: bool = True) -> torch.Tensor:
        return self.decoder(z, constrain_value_range)

    def encode(self, x: torch.Tensor) -> List[torch.Tensor]:
        """Waveform -> ``num_quantizers`` index tensors ``[B, T']``."""
        return self.prvq.encode(self.ae_encode(x))

    @property
    def rvq_codebooks(self) -> torch.Tensor:
        """[num_quantizers, codebook_size, latent]: what the speech generator adopts as its code embeddings."""
        return torch.stack([m.data for m in self.prvq.mus_list])

    def decode(self, ids: Optional[Sequence[torch.Tensor]] = None, constrain_value_range: bool = True, tokens: Optional[torch.Tensor] = None,
               tokens_len: Optional[torch.Tensor] = None):
        """From per-level index tensors -> ``[B, 1, T]``; or, codec-model style, ``tokens`` [B, K, T'] (+ ``tokens_len``) ->
        ``(audio [B, T], audio_len)``."""
        if tokens is not None:
            wav = self.ae_decode(self.prvq.decode(list(tokens.long().unbind(1))), constrain_value_range)[:, 0]
            lens = tokens_len * self.wav_to_token_ratio if tokens_len is not None else torch.full((wav.shape[0],), wav.shape[1], device=wav.device)
            return wav, lens
        return self.ae_decode(self.prvq.decode(ids), constrain_value_range)

    def decode_stream(self, z: torch.Tensor, state: Optional[dict] = None, constrain_value_range: bool = True):
        """Latents (or de-quantised codes) of the next frames ``[B, t, latent]`` -> their ``t * ratio`` samples and the new state."""
        return self.decoder.forward_stream(z, state, constrain_value_range)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        z = self.ae_encode(x)
        ids, z_q = self.prvq.encode(z, return_z_q=True)
        z_st = z + (z_q - z).detach()                                   # straight-through
        return self.ae_decode(z_st, constrain_value_range=False), z, z_q

    def training_loss(self, x: torch.Tensor, commitment: float = 0.25) -> Dict[str, torch.Tensor]:
        """Multi-resolution spectral L1 + waveform L1 + commitment of the latents to their quantised values; the codebooks follow
        the latents by EMA (no gradient)."""
        y, z, z_q = self.forward(x)
        if self.training:
            self.prvq.update_codebooks(z)
        rec = (y - x).abs().mean()
        spec = 0.0
        for n in (64, 256, 1024):
            if x.shape[-1] < n:
                continue
            w = torch.hann_window(n, device=x.device)
            a = torch.stft(x[:, 0].float(), n, n // 4, n, w, return_complex=True).abs()
            b = torch.stft(y[:, 0].float(), n, n // 4, n, w, return_complex=True).abs()
            spec = spec + (torch.log1p(a) - torch.log1p(b)).abs().mean()
        commit = (z - z_q.detach()).pow(2).mean()
        return {"loss": rec + spec + commitment * commit, "rec": rec.detach(), "commit": commit.detach()}

"""Neural audio codec: waveform ↔ discrete tokens.

``AudioCodecModel``: strided convolutional encoder → finite scalar quantiser (FSQ, optionally grouped: one code index per
group = per codebook) → HiFi-GAN style decoder; trained with mel / multi-resolution STFT reconstruction losses and
multi-period + multi-resolution-STFT discriminators (feature matching + least-squares GAN).  The TTS models use a frozen
instance through ``encode`` / ``decode``.
Reference: ``tts/models/audio_codec.py``, ``tts/modules/audio_codec_modules.py:1347 (FSQ), 1550 (GroupFSQ)``,
``tts/losses/audio_codec_loss.py``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, OmegaConf, cfg_get, to_container
from ..core.modelpt import ModelPT


def mask_by_length(x: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    m = torch.arange(x.shape[-1], device=x.device)[None, :] < lens[:, None]
    return x * m.view(x.shape[0], *([1] * (x.dim() - 2)), x.shape[-1]).to(x.dtype)


class FiniteScalarQuantizer(nn.Module):
    """Each latent dim ``d`` is squashed to ``(-1, 1)``, rounded to ``num_levels[d]`` levels (straight-through) and the
    tuple of levels is read as one mixed-radix index."""

    def __init__(self, num_levels: Sequence[int], eps: float = 1e-3):
        super().__init__()
        self.register_buffer("num_levels", torch.tensor(list(num_levels), dtype=torch.long).view(1, -1, 1), persistent=False)
        basis = torch.cumprod(torch.tensor([1] + list(num_levels[:-1]), dtype=torch.long), dim=0)
        self.register_buffer("dim_base_index", basis.view(1, -1, 1), persistent=False)
        self.eps = eps
        self.dim = len(num_levels)
        self.codebook_size = int(torch.tensor(list(num_levels)).prod())

    def _bound(self, x):
        L = self.num_levels.to(x.dtype)
        scale = (L - 1) * (1 - self.eps) / 2
        offset = torch.where(self.num_levels % 2 == 0, torch.full_like(scale, 0.5), torch.zeros_like(scale))
        shift = torch.tan(offset / scale)
        return scale * torch.tanh(x + shift) - offset

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        """[B, D, T] → (dequantised [B, D, T] with straight-through gradient, indices [1, B, T])."""
        b = self._bound(inputs.float())
        r = b + (torch.round(b) - b).detach()
        scale = (self.num_levels // 2).to(r.dtype)
        deq = mask_by_length((r / scale).to(inputs.dtype), input_len)
        return deq, self.codes_to_indices(r, input_len)

    def codes_to_indices(self, r, input_len):
        nn_ = (r + (self.num_levels // 2).to(r.dtype)).round().long()
        idx = (nn_ * self.dim_base_index).sum(dim=1)
        return (idx * (torch.arange(idx.shape[-1], device=idx.device)[None] < input_len[:, None])).unsqueeze(0)

    def decode(self, indices: torch.Tensor, input_len: torch.Tensor) -> torch.Tensor:
        """indices [1, B, T] → dequantised [B, D, T]."""
        idx = indices[0].unsqueeze(1)
        nn_ = (idx // self.dim_base_index) % self.num_levels
        scale = (self.num_levels // 2).float()
        return mask_by_length((nn_.float() - scale) / scale, input_len)


class GroupFiniteScalarQuantizer(nn.Module):
    def __init__(self, num_groups: int, num_levels_per_group: Sequence[int], **kw):
        super().__init__()
        self.num_groups = num_groups
        self.fsqs = nn.ModuleList([FiniteScalarQuantizer(num_levels_per_group, **kw) for _ in range(num_groups)])
        self.codebook_dim_per_group = len(num_levels_per_group)
        self.codebook_size = self.fsqs[0].codebook_size

    def forward(self, inputs, input_len):
        outs, ids = [], []
        for g, x in zip(self.fsqs, inputs.chunk(self.num_groups, dim=1)):
            d, i = g(x, input_len)
            outs.append(d)
            ids.append(i)
        return torch.cat(outs, dim=1), torch.cat(ids, dim=0)          # [B, D, T], [G, B, T]

    def encode(self, inputs, input_len):
        return self.forward(inputs, input_len)[1]

    def decode(self, indices, input_len):
        return torch.cat([g.decode(indices[i:i + 1], input_len) for i, g in enumerate(self.fsqs)], dim=1)


def _same_pad(k: int, d: int = 1) -> int:
    return (k - 1) * d // 2


class ResidualBlock(nn.Module):
    def __init__(self, ch: int, kernel_size: int = 3, dilations=(1, 3, 5), causal: bool = False):
        super().__init__()
        self.causal, self.k, self.dil = causal, kernel_size, list(dilations)
        self.convs1 = nn.ModuleList([nn.Conv1d(ch, ch, kernel_size, dilation=d, padding=0 if causal else _same_pad(kernel_size, d))
                                     for d in dilations])
        self.convs2 = nn.ModuleList([nn.Conv1d(ch, ch, kernel_size, padding=0 if causal else _same_pad(kernel_size)) for _ in dilations])

    def _c(self, conv, x, d):
        if self.causal:
            x = F.pad(x, ((self.k - 1) * d, 0))
        return conv(x)

    def forward(self, x):
        for c1, c2, d in zip(self.convs1, self.convs2, self.dil):
            y = self._c(c1, F.leaky_relu(x, 0.1), d)
            y = self._c(c2, F.leaky_relu(y, 0.1), 1)
            x = x + y
        return x


class HiFiGANEncoder(nn.Module):
    def __init__(self, encoded_dim: int = 32, down_sample_rates=(2, 4, 4, 8), base_channels: int = 32, in_kernel_size: int = 7,
                 out_kernel_size: int = 7, resblock_kernel_sizes=(3,), resblock_dilation_sizes=(1, 3), causal: bool = False):
        super().__init__()
        self.rates = list(down_sample_rates)
        self.pre = nn.Conv1d(1, base_channels, in_kernel_size, padding=_same_pad(in_kernel_size))
        ch = base_channels
        self.res, self.down = nn.ModuleList(), nn.ModuleList()
        for r in self.rates:
            self.res.append(nn.ModuleList([ResidualBlock(ch, k, resblock_dilation_sizes, causal) for k in resblock_kernel_sizes]))
            self.down.append(nn.Conv1d(ch, ch * 2, 2 * r, stride=r, padding=(2 * r - r + 1) // 2))
            ch *= 2
        self.post = nn.Conv1d(ch, encoded_dim, out_kernel_size, padding=_same_pad(out_kernel_size))

    @property
    def total_stride(self) -> int:
        return int(math.prod(self.rates))

    def forward(self, audio: torch.Tensor, audio_len: torch.Tensor):
        x = self.pre(audio.unsqueeze(1))
        lens = audio_len
        for blocks, down, r in zip(self.res, self.down, self.rates):
            x = sum(b(x) for b in blocks) / len(blocks)
            x = down(F.leaky_relu(x, 0.1))
            lens = torch.div(lens + r - 1, r, rounding_mode="floor")
            x = mask_by_length(x[..., : int(lens.max())] if x.shape[-1] >= int(lens.max()) else x, lens.clamp(max=x.shape[-1]))
        x = self.post(F.leaky_relu(x, 0.1))
        lens = lens.clamp(max=x.shape[-1])
        return mask_by_length(x, lens), lens


class HiFiGANDecoder(nn.Module):
    def __init__(self, input_dim: int = 32, up_sample_rates=(8, 4, 4, 2), base_channels: int = 512, in_kernel_size: int = 7,
                 out_kernel_size: int = 3, resblock_kernel_sizes=(3, 7, 11), resblock_dilation_sizes=(1, 3, 5),
                 activation: str = "lrelu", output_activation: str = "tanh", causal: bool = False):
        super().__init__()
        self.rates = list(up_sample_rates)
        self.pre = nn.Conv1d(input_dim, base_channels, in_kernel_size, padding=_same_pad(in_kernel_size))
        ch = base_channels
        self.up, self.res = nn.ModuleList(), nn.ModuleList()
        for r in self.rates:
            self.up.append(nn.ConvTranspose1d(ch, ch // 2, 2 * r, stride=r, padding=r // 2 + r % 2, output_padding=r % 2))
            ch //= 2
            self.res.append(nn.ModuleList([ResidualBlock(ch, k, resblock_dilation_sizes, causal) for k in resblock_kernel_sizes]))
        self.post = nn.Conv1d(ch, 1, out_kernel_size, padding=_same_pad(out_kernel_size))
        self.out_act = torch.tanh if output_activation == "tanh" else (lambda z: z.clamp(-1, 1))

    def forward(self, inputs: torch.Tensor, input_len: torch.Tensor):
        x = self.pre(inputs)
        lens = input_len
        for up, blocks, r in zip(self.up, self.res, self.rates):
            x = up(F.leaky_relu(x, 0.1))
            lens = lens * r
            x = x[..., : int(lens.max())]
            x = sum(b(x) for b in blocks) / len(blocks)
        audio = self.out_act(self.post(F.leaky_relu(x, 0.1))).squeeze(1)
        return mask_by_length(audio, lens.clamp(max=audio.shape[-1])), lens.clamp(max=audio.shape[-1])


# ---------------------------------------------------------------------------------------------- losses / discriminators
def _stft_mag(x, n_fft, hop, win):
    w = torch.hann_window(win, device=x.device, dtype=torch.float32)
    s = torch.stft(x.float(), n_fft, hop, win, w, return_complex=True, center=True, pad_mode="reflect")
    return s.abs().clamp(min=1e-5)


class MultiResolutionSTFTLoss(nn.Module):
    def __init__(self, resolutions=((512, 128, 512), (1024, 256, 1024), (2048, 512, 2048)), log_guard: float = 1e-5):
        super().__init__()
        self.res = [tuple(r) for r in resolutions]

    def forward(self, audio_real, audio_gen, audio_len):
        loss = 0.0
        for n_fft, hop, win in self.res:
            a, b = _stft_mag(audio_real, n_fft, hop, win), _stft_mag(audio_gen, n_fft, hop, win)
            loss = loss + F.l1_loss(a.log(), b.log()) + (torch.linalg.norm(a - b) / torch.linalg.norm(a).clamp(min=1e-5))
        return loss / len(self.res)


class MelLoss(nn.Module):
    def __init__(self, sample_rate: int = 22050, n_mels: int = 80, n_fft: int = 1024, hop: int = 256, win: int = 1024):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        fb = mel_filterbank(sample_rate, n_fft, n_mels)
        self.register_buffer("fb", torch.as_tensor(fb, dtype=torch.float32), persistent=False)
        self.n_fft, self.hop, self.win = n_fft, hop, win

    def mel(self, x):
        return torch.log(torch.matmul(self.fb.to(x.device), _stft_mag(x, self.n_fft, self.hop, self.win)).clamp(min=1e-5))

    def forward(self, audio_real, audio_gen, audio_len):
        return F.l1_loss(self.mel(audio_real), self.mel(audio_gen))


class PeriodDiscriminator(nn.Module):
    def __init__(self, period: int, ch=(32, 64, 128)):
        super().__init__()
        self.period = period
        chans = [1] + list(ch)
        self.convs = nn.ModuleList([nn.Conv2d(a, b, (5, 1), (3, 1), padding=(2, 0)) for a, b in zip(chans[:-1], chans[1:])])
        self.post = nn.Conv2d(chans[-1], 1, (3, 1), padding=(1, 0))

    def forward(self, x):
        B, T = x.shape
        pad = (-T) % self.period
        x = F.pad(x.unsqueeze(1), (0, pad), mode="reflect" if pad < T else "constant").view(B, 1, -1, self.period)
        fmaps = []
        for c in self.convs:
            x = F.leaky_relu(c(x), 0.1)
            fmaps.append(x)
        x = self.post(x)
        fmaps.append(x)
        return x.flatten(1), fmaps


class STFTDiscriminator(nn.Module):
    def __init__(self, resolution=(1024, 256, 1024), ch: int = 32):
        super().__init__()
        self.resolution = tuple(resolution)
        self.convs = nn.ModuleList([nn.Conv2d(1, ch, (3, 9), padding=(1, 4)), nn.Conv2d(ch, ch, (3, 9), stride=(1, 2), padding=(1, 4)),
                                    nn.Conv2d(ch, ch, (3, 9), stride=(1, 2), padding=(1, 4))])
        self.post = nn.Conv2d(ch, 1, 3, padding=1)

    def forward(self, x):
        s = _stft_mag(x, *self.resolution).unsqueeze(1).transpose(2, 3)
        fmaps = []
        for c in self.convs:
            s = F.leaky_relu(c(s), 0.1)
            fmaps.append(s)
        s = self.post(s)
        fmaps.append(s)
        return s.flatten(1), fmaps


class Discriminator(nn.Module):
    """Period + STFT sub-discriminators; ``multiband_stft_resolutions`` adds banded STFT discriminators, and ``add_slm`` one on the
    features of a frozen speech foundation model."""

    def __init__(self, periods=(2, 3, 5, 7, 11), stft_resolutions=((512, 128, 512), (1024, 256, 1024)), multiband_stft_resolutions=(),
                 stft_bands=((0.0, 0.1), (0.1, 0.25), (0.25, 0.5), (0.5, 0.75), (0.75, 1.0))):
        super().__init__()
        from .audio_codec_extra import MultiBandDiscriminatorSTFT

        self.discs = nn.ModuleList([PeriodDiscriminator(p) for p in periods] + [STFTDiscriminator(tuple(r)) for r in stft_resolutions]
                                   + [MultiBandDiscriminatorSTFT(tuple(r), stft_bands) for r in multiband_stft_resolutions])
        self.slm = None

    def add_slm(self, feature_extractor, **kw):
        from .audio_codec_extra import SLMDiscriminator

        self.slm = SLMDiscriminator(feature_extractor, **kw)
        return self.slm

    def forward(self, audio_real, audio_gen):
        outs = [(d(audio_real), d(audio_gen)) for d in self.discs]
        res = ([o[0][0] for o in outs], [o[1][0] for o in outs], [o[0][1] for o in outs], [o[1][1] for o in outs])
        if self.slm is not None:
            for acc, extra in zip(res, self.slm(audio_real, audio_gen)):
                acc.extend(extra)
        return res


def gan_update(model, loss: torch.Tensor, optimizer, standalone_step: bool) -> None:
    """Applies ``loss`` to ``optimizer``: through the trainer when the model runs under ``fit`` (gradient averaging over ranks,
    clipping, callbacks); directly when ``standalone_step`` (the discriminator update of a hand-driven loop).  A hand-driven
    generator update is left to the caller, who gets the loss back from ``training_step``."""
    tr = getattr(model, "_trainer", None)
    if tr is not None and getattr(tr, "in_manual_step", False):
        tr.manual_step(loss, optimizer)
    elif standalone_step:
        optimizer.zero_grad()
        loss.backward()
        optimizer.step()


def generator_adv_loss(scores_gen):
    return sum(((1 - s) ** 2).mean() for s in scores_gen) / len(scores_gen)


def discriminator_loss(scores_real, scores_gen):
    return sum(((1 - r) ** 2).mean() + (g ** 2).mean() for r, g in zip(scores_real, scores_gen)) / len(scores_real)


def feature_matching_loss(fmaps_real, fmaps_gen):
    loss, n = 0.0, 0
    for fr, fg in zip(fmaps_real, fmaps_gen):
        for a, b in zip(fr, fg):
            loss = loss + F.l1_loss(b, a.detach())
            n += 1
    return loss / max(n, 1)


class AudioCodecModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.sample_rate = cfg_get(cfg, "sample_rate", 22050)
        enc = dict(cfg_get(cfg, "audio_encoder", {}) or {})
        dec = dict(cfg_get(cfg, "audio_decoder", {}) or {})
        vq = dict(cfg_get(cfg, "vector_quantizer", {}) or {})
        from . import audio_codec_encoders as E

        enc_kind, dec_kind = str(enc.get("_target_", "")).rsplit(".", 1)[-1], str(dec.get("_target_", "")).rsplit(".", 1)[-1]
        enc = to_container(cfg_get(cfg, "audio_encoder"), resolve=True) if enc_kind in E.ENCODERS else enc
        for d in (dec, vq):
            d.pop("_target_", None)
        if enc_kind in E.ENCODERS:                                   # spectral / causal encoders named by class
            self.audio_encoder = E.build_encoder(enc)
        else:
            enc.pop("_target_", None)
            self.audio_encoder = HiFiGANEncoder(**enc)
        self.vector_quantizer = GroupFiniteScalarQuantizer(**vq) if vq else None
        if dec_kind in E.DECODERS:
            self.audio_decoder = E.DECODERS[dec_kind](**{k: (list(v) if hasattr(v, "__iter__") and not isinstance(v, str) else v) for k, v in dec.items()})
        elif dec.pop("causal", False):
            from .audio_codec_extra import CausalHiFiGANDecoder

            self.audio_decoder = CausalHiFiGANDecoder(**dec)
        else:
            self.audio_decoder = HiFiGANDecoder(**dec)
        self.samples_per_frame = self.audio_encoder.total_stride
        self.num_codebooks = self.vector_quantizer.num_groups if self.vector_quantizer is not None else 0
        self.codebook_size = self.vector_quantizer.codebook_size if self.vector_quantizer is not None else 0
        self.discriminator = Discriminator(**dict(cfg_get(cfg, "discriminator", {}) or {})) if cfg_get(cfg, "train_discriminator", True) else None
        self.mel_loss = MelLoss(self.sample_rate, **dict(cfg_get(cfg, "mel_loss", {}) or {}))
        self.stft_loss = MultiResolutionSTFTLoss()
        self.w = {"mel": cfg_get(cfg, "mel_loss_l1_scale", 15.0), "stft": cfg_get(cfg, "stft_loss_scale", 1.0),
                  "gen": cfg_get(cfg, "gen_loss_scale", 1.0), "fm": cfg_get(cfg, "feature_loss_scale", 1.0)}
        from . import audio_codec_extra as X

        kind = cfg_get(cfg, "gan_loss", "squared")
        if kind not in ("squared", "hinged"):
            raise ValueError(f"gan_loss must be 'squared' or 'hinged', got {kind!r}")
        self.gen_loss = X.GeneratorHingedLoss() if kind == "hinged" else X.GeneratorSquaredLoss()
        self.disc_loss = X.DiscriminatorHingedLoss() if kind == "hinged" else X.DiscriminatorSquaredLoss()
        self.feature_loss = X.RelativeFeatureMatchingLoss() if cfg_get(cfg, "feature_loss_type", "absolute") == "relative" else None
        self.w["time"] = cfg_get(cfg, "time_domain_loss_scale", 0.0)
        self.w["sisdr"] = cfg_get(cfg, "si_sdr_loss_scale", 0.0)
        self.time_loss, self.sisdr_loss = X.TimeDomainLoss(), X.SISDRLoss()
        self.automatic_optimization = False
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "audio_decoder"):
            return
        super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ data: batches of (audio, audio_len)
    def _loader(self, config):
        if config is None:
            return None
        from ..data.audio_to_text import SyntheticSpeechDataset, get_dataloader_from_config

        syn = config.get("synthetic", None)
        if syn is None:
            from ..data.audio_to_text import build_speech_dataset

            ds = build_speech_dataset(config, labels=[" "])
        else:
            ds = SyntheticSpeechDataset(vocab_size=2, **dict(syn))
        return get_dataloader_from_config(config, ds, 0, 1)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    # ------------------------------------------------------------------ codec API
    def pad_audio(self, audio, audio_len):
        pad = (-audio.shape[-1]) % self.samples_per_frame
        return (F.pad(audio, (0, pad)) if pad else audio), audio_len

    def encode_audio(self, audio, audio_len):
        audio, audio_len = self.pad_audio(audio, audio_len)
        return self.audio_encoder(audio, audio_len)

    def quantize(self, encoded, encoded_len):
        return self.vector_quantizer.encode(encoded, encoded_len).permute(1, 0, 2)       # [B, C, T]

    def dequantize(self, tokens, tokens_len):
        return self.vector_quantizer.decode(tokens.permute(1, 0, 2), tokens_len)

    @torch.no_grad()
    def encode(self, audio, audio_len):
        """→ tokens [B, C, T_frames], lengths."""
        enc, enc_len = self.encode_audio(audio, audio_len)
        return self.quantize(enc, enc_len), enc_len

    @torch.no_grad()
    def decode(self, tokens, tokens_len):
        return self.audio_decoder(self.dequantize(tokens, tokens_len).to(next(self.audio_decoder.parameters()).dtype), tokens_len)

    @torch.no_grad()
    def decode_stream(self, tokens, state=None):
        """Chunk of tokens ``[B, C, t]`` -> the next ``t * samples_per_frame`` samples; needs ``audio_decoder.causal: true``."""
        if not hasattr(self.audio_decoder, "decode_stream"):
            raise RuntimeError("streaming decode needs a causal decoder (audio_decoder.causal: true)")
        lens = torch.full((tokens.shape[0],), tokens.shape[-1], device=tokens.device, dtype=torch.long)
        z = self.dequantize(tokens, lens).to(next(self.audio_decoder.parameters()).dtype)
        return self.audio_decoder.decode_stream(z, state)

    def add_slm_discriminator(self, feature_extractor, **kw):
        """Adds a discriminator over the features of a frozen speech foundation model (``feature_extractor(audio) -> [B, L, T, D]``);
        call before ``configure_optimizers``."""
        if self.discriminator is None:
            raise RuntimeError("train_discriminator is off")
        kw.setdefault("input_sr", self.sample_rate)
        return self.discriminator.add_slm(feature_extractor, **kw)

    def forward(self, audio, audio_len):
        enc, enc_len = self.encode_audio(audio, audio_len)
        if self.vector_quantizer is not None:
            enc, _ = self.vector_quantizer(enc, enc_len)
        return self.audio_decoder(enc, enc_len)

    # ------------------------------------------------------------------ training (generator / discriminator alternate)
    def configure_optimizers(self):
        lr = cfg_get(cfg_get(self._cfg, "optim", {}), "lr", 2e-4)
        gen = [p for n, p in self.named_parameters() if not n.startswith("discriminator.")]
        opt_g = torch.optim.AdamW(gen, lr=lr, betas=(0.8, 0.99))
        if self.discriminator is None:
            self._optimizers = [opt_g]
            return opt_g
        opt_d = torch.optim.AdamW(self.discriminator.parameters(), lr=lr, betas=(0.8, 0.99))
        self._optimizers = [opt_g, opt_d]
        return [opt_g, opt_d]

    def training_step(self, batch, batch_idx):
        audio, audio_len = batch[0], batch[1]
        gen, gen_len = self.forward(audio, audio_len)
        n = min(audio.shape[-1], gen.shape[-1])
        audio, gen = audio[..., :n], gen[..., :n]
        logs = {}
        opts = getattr(self, "_optimizers", None)
        manual = opts is not None and len(opts) == 2 and self.discriminator is not None
        if manual:
            sr, sg, _, _ = self.discriminator(audio, gen.detach())
            d_loss = self.disc_loss(sr, sg)
            gan_update(self, d_loss, opts[1], standalone_step=True)
            logs["d_loss"] = d_loss.detach()
        loss = self.w["mel"] * self.mel_loss(audio, gen, audio_len) + self.w["stft"] * self.stft_loss(audio, gen, audio_len)
        if self.w["time"]:
            loss = loss + self.w["time"] * self.time_loss(audio, gen, audio_len)
        if self.w["sisdr"]:
            loss = loss + self.w["sisdr"] * self.sisdr_loss(audio, gen, audio_len)
        if self.discriminator is not None:
            sr, sg, fr, fg = self.discriminator(audio, gen)
            fm = self.feature_loss(fr, fg) if self.feature_loss is not None else feature_matching_loss(fr, fg)
            loss = loss + self.w["gen"] * self.gen_loss(sg) + self.w["fm"] * fm
        logs["train_loss"] = loss.detach()
        self.log_dict(logs)
        if opts:
            gan_update(self, loss, opts[0], standalone_step=False)
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        audio, audio_len = batch[0], batch[1]
        gen, _ = self.forward(audio, audio_len)
        n = min(audio.shape[-1], gen.shape[-1])
        return {"val_loss": self.mel_loss(audio[..., :n], gen[..., :n], audio_len)}

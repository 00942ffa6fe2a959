"""Audio-to-audio models: enhancement, separation and generative restoration.

* ``AudioToAudioModel`` — base class: ``(input, input_len, target, target_len)`` batches, SI-SDR / SDR validation metrics,
  ``process()`` for inference on files or arrays, gradient sanitising when a rank sees non-finite values
  (``audio/models/audio_to_audio.py``; NaN-grad all-reduce ``:567``).
* ``EncMaskDecAudioToAudioModel`` — encoder (STFT) → mask estimator → mask processor (reference-channel masking or
  mask-based beamformer) → decoder (iSTFT).
* ``PredictiveAudioToAudioModel`` — encoder → estimator network that predicts the clean spectrogram → decoder.
* ``ScoreBasedGenerativeAudioToAudioModel`` — OUVE SDE score matching with a predictor-corrector sampler.
* ``SchroedingerBridgeAudioToAudioModel`` — data-prediction Schrödinger bridge (VE noise schedule) with an SDE / ODE sampler.
* ``FlowMatchingAudioToAudioModel`` — conditional optimal-transport flow matching with an Euler ODE sampler.
(``audio/models/enhancement.py``.)
"""
from __future__ import annotations

import math
import os
from typing import Any, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from ..core.instantiate import from_config_dict
from ..core.modelpt import ModelPT
from .modules import MaskedMSELoss, SDRLoss, sdr, si_sdr


class AudioToAudioModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self.sample_rate = cfg_get(self._cfg, "sample_rate", 16000)
        self.skip_nan_grad = cfg_get(self._cfg, "skip_nan_grad", False)

    def _finish_init(self):
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not getattr(self, "_ready", False):
            return
        super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ data
    def _loader(self, config):
        if config is None:
            return None
        from .data import build_audio_to_target_dataloader

        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        return build_audio_to_target_dataloader(config, rank, ws)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def setup_test_data(self, c):
        self._test_dl = self._loader(c)

    # ------------------------------------------------------------------ hooks
    def on_after_backward(self):
        """Zero all gradients of this step when any rank produced a non-finite one (keeps ranks in lock-step)."""
        if not self.skip_nan_grad:
            return
        ok = torch.ones(1, device=self.device)
        for p in self.parameters():
            if p.grad is not None and not torch.isfinite(p.grad).all():
                ok.zero_()
                break
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) < 1:
            self.zero_grad()

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        x, xl, y, yl = batch[:4]
        est, el = self.forward(input_signal=x, input_length=xl)
        n = min(est.shape[-1], y.shape[-1])
        return {"val_loss": self._eval_loss(est[..., :n], y[..., :n], yl.clamp(max=n)),
                "val_sisdr": si_sdr(est[..., :n], y[..., :n], yl.clamp(max=n)).mean(),
                "val_sdr": sdr(est[..., :n], y[..., :n], yl.clamp(max=n)).mean()}

    def _eval_loss(self, est, tgt, lens):
        return -si_sdr(est, tgt, lens).mean()

    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0):
        if not outputs:
            return {}
        avg = {k: torch.stack([torch.as_tensor(o[k]).float() for o in outputs]).mean() for k in outputs[0]}
        return {"val_loss": avg["val_loss"], "log": avg}

    # ------------------------------------------------------------------ inference
    @torch.no_grad()
    def process(self, audio: Sequence[Any], output_dir: Optional[str] = None, batch_size: int = 1, **kw) -> List[np.ndarray]:
        from ..data.audio_to_text import load_audio, save_wav

        self.eval()
        outs = []
        for i, a in enumerate(audio):
            x = torch.as_tensor(load_audio(a, target_sr=self.sample_rate) if isinstance(a, str) else a, dtype=torch.float32)
            x = x.reshape(1, 1, -1) if x.dim() == 1 else x.unsqueeze(0)
            est, _ = self.forward(input_signal=x.to(self.device), input_length=torch.tensor([x.shape[-1]], device=self.device), **kw)
            y = est[0].cpu().numpy()
            outs.append(y)
            if output_dir:
                os.makedirs(output_dir, exist_ok=True)
                name = os.path.basename(a) if isinstance(a, str) else f"processed_{i}.wav"
                save_wav(os.path.join(output_dir, name), y[0], self.sample_rate)
        return outs


class EncMaskDecAudioToAudioModel(AudioToAudioModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.encoder = from_config_dict(cfg.encoder)
        self.mask_estimator = from_config_dict(cfg.mask_estimator)
        self.mask_processor = from_config_dict(cfg.mask_processor)
        self.decoder = from_config_dict(cfg.decoder)
        self.mixture_consistency = from_config_dict(cfg.mixture_consistency) if cfg.get("mixture_consistency") is not None else None
        self.loss = from_config_dict(cfg.loss) if cfg.get("loss") is not None else SDRLoss(scale_invariant=True)
        self._ready = True
        self._finish_init()

    def forward(self, input_signal, input_length=None):
        if input_signal.dim() == 2:
            input_signal = input_signal.unsqueeze(1)
        T = input_signal.shape[-1]
        enc, enc_len = self.encoder(input=input_signal, input_length=input_length)
        mask, _ = self.mask_estimator(input=enc, input_length=enc_len)
        proc, proc_len = self.mask_processor(input=enc, input_length=enc_len, mask=mask)
        out, out_len = self.decoder(input=proc, input_length=proc_len)
        out = torch.nn.functional.pad(out, (0, max(0, T - out.shape[-1])))[..., :T]
        return out, input_length

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        est, _ = self.forward(input_signal=x, input_length=xl)
        if y.dim() == 2:
            y = y.unsqueeze(1)
        loss = self.loss(estimate=est, target=y, input_length=xl)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}


class PredictiveAudioToAudioModel(AudioToAudioModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.encoder = from_config_dict(cfg.encoder)
        self.estimator = from_config_dict(cfg.estimator)
        self.decoder = from_config_dict(cfg.decoder)
        self.loss = from_config_dict(cfg.loss) if cfg.get("loss") is not None else MaskedMSELoss()
        self.normalize_input = cfg_get(cfg, "normalize_input", False)
        self._ready = True
        self._finish_init()

    def forward(self, input_signal, input_length=None):
        if input_signal.dim() == 2:
            input_signal = input_signal.unsqueeze(1)
        T = input_signal.shape[-1]
        norm = input_signal.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1e-8) if self.normalize_input else 1.0
        enc, enc_len = self.encoder(input=input_signal / norm, input_length=input_length)
        est, _ = self.estimator(input=enc, input_length=enc_len)
        out, _ = self.decoder(input=est, input_length=enc_len)
        out = torch.nn.functional.pad(out, (0, max(0, T - out.shape[-1])))[..., :T]
        return out * norm, input_length

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        if y.dim() == 2:
            y = y.unsqueeze(1)
        est, _ = self.forward(input_signal=x, input_length=xl)
        loss = self.loss(estimate=est, target=y, input_length=xl)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}


class _GenerativeBase(AudioToAudioModel):
    """Shared plumbing: STFT encoder / decoder, estimator taking (state ⊕ noisy condition, time)."""

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.encoder = from_config_dict(cfg.encoder)
        self.estimator = from_config_dict(cfg.estimator)
        self.decoder = from_config_dict(cfg.decoder)
        self.num_steps = cfg_get(cfg_get(cfg, "sampler", {}) or {}, "num_steps", 8)
        self.normalize_input = cfg_get(cfg, "normalize_input", True)

    def _encode(self, signal, length):
        if signal.dim() == 2:
            signal = signal.unsqueeze(1)
        return self.encoder(input=signal, input_length=length)

    def _net(self, state, cond, time, lens):
        return self.estimator(input=torch.cat([state, cond], dim=1), input_length=lens, time=time)[0]

    def _decode(self, spec, lens, T):
        out, _ = self.decoder(input=spec, input_length=lens)
        return torch.nn.functional.pad(out, (0, max(0, T - out.shape[-1])))[..., :T]

    def _norm(self, x):
        return x.abs().amax(dim=tuple(range(1, x.dim())), keepdim=True).clamp(min=1e-8) if self.normalize_input else 1.0


def _cnoise(like: torch.Tensor) -> torch.Tensor:
    return torch.complex(torch.randn_like(like.real), torch.randn_like(like.real)) / math.sqrt(2.0)


class FlowMatchingAudioToAudioModel(_GenerativeBase):
    """``x_t = (1 - (1 - σ_min) t) x_0 + t x_1`` with ``x_0 ~ N(y, σ²)``; the network regresses the velocity ``x_1 - (1-σ_min) x_0``."""

    def __init__(self, cfg, trainer=None):
        super().__init__(cfg, trainer)
        f = cfg_get(self._cfg, "flow", {}) or {}
        self.sigma_min, self.sigma_start = cfg_get(f, "sigma_min", 1e-4), cfg_get(f, "sigma_start", 0.5)
        self._ready = True
        self._finish_init()

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        n = self._norm(x)
        noisy, lens = self._encode(x / n, xl)
        clean, _ = self._encode(y / n, xl)
        t = torch.rand(noisy.shape[0], device=noisy.device)
        x0 = noisy + self.sigma_start * _cnoise(noisy)
        tt = t.view(-1, 1, 1, 1)
        xt = (1 - (1 - self.sigma_min) * tt) * x0 + tt * clean
        v = self._net(xt, noisy, t, lens)
        loss = MaskedMSELoss()(v, clean - (1 - self.sigma_min) * x0, lens)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def forward(self, input_signal, input_length=None, num_steps: Optional[int] = None):
        T = input_signal.shape[-1]
        n = self._norm(input_signal if input_signal.dim() == 3 else input_signal.unsqueeze(1))
        noisy, lens = self._encode(input_signal / n, input_length)
        x = noisy + self.sigma_start * _cnoise(noisy)
        steps = num_steps or self.num_steps
        for i in range(steps):
            t = torch.full((x.shape[0],), i / steps, device=x.device)
            x = x + self._net(x, noisy, t, lens) / steps
        return self._decode(x, lens, T) * n, input_length


class ScoreBasedGenerativeAudioToAudioModel(_GenerativeBase):
    """Ornstein-Uhlenbeck variance-exploding SDE: ``dx = γ (y - x) dt + g(t) dw``, ``g(t) = σ_min (σ_max/σ_min)^t sqrt(2 log(σ_max/σ_min))``."""

    def __init__(self, cfg, trainer=None):
        super().__init__(cfg, trainer)
        s = cfg_get(self._cfg, "sde", {}) or {}
        self.gamma, self.smin, self.smax = cfg_get(s, "stiffness", 1.5), cfg_get(s, "std_min", 0.05), cfg_get(s, "std_max", 0.5)
        self.t_eps = cfg_get(s, "time_min", 0.03)
        self._ready = True
        self._finish_init()

    def _std(self, t):
        lr = math.log(self.smax / self.smin)
        num = self.smin ** 2 * (torch.exp(2 * lr * t) - torch.exp(-2 * self.gamma * t)) * lr
        return torch.sqrt(num / (self.gamma + lr))

    def _mean(self, x0, y, t):
        e = torch.exp(-self.gamma * t).view(-1, 1, 1, 1)
        return e * x0 + (1 - e) * y

    def _g(self, t):
        lr = math.log(self.smax / self.smin)
        return self.smin * (self.smax / self.smin) ** t * math.sqrt(2 * lr)

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        n = self._norm(x)
        noisy, lens = self._encode(x / n, xl)
        clean, _ = self._encode(y / n, xl)
        t = torch.rand(noisy.shape[0], device=noisy.device) * (1 - self.t_eps) + self.t_eps
        std = self._std(t).view(-1, 1, 1, 1)
        z = _cnoise(noisy)
        xt = self._mean(clean, noisy, t) + std * z
        score = self._net(xt, noisy, t, lens)
        loss = MaskedMSELoss()(score * std, -z, lens)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def forward(self, input_signal, input_length=None, num_steps: Optional[int] = None, corrector_snr: float = 0.5):
        T = input_signal.shape[-1]
        n = self._norm(input_signal if input_signal.dim() == 3 else input_signal.unsqueeze(1))
        noisy, lens = self._encode(input_signal / n, input_length)
        steps = num_steps or self.num_steps
        ts = torch.linspace(1.0, self.t_eps, steps + 1, device=noisy.device)
        x = noisy + self._std(ts[:1]).view(1, 1, 1, 1) * _cnoise(noisy)
        for i in range(steps):
            t = ts[i].expand(x.shape[0])
            dt = ts[i] - ts[i + 1]
            s = self._net(x, noisy, t, lens)
            z = _cnoise(x)                                           # corrector: one annealed Langevin step
            eps = 2 * (corrector_snr * self._std(t).view(-1, 1, 1, 1)) ** 2
            x = x + eps * s + torch.sqrt(2 * eps) * z
            s = self._net(x, noisy, t, lens)                         # predictor: reverse diffusion
            g = self._g(t).view(-1, 1, 1, 1)
            x = x - (self.gamma * (noisy - x) - g ** 2 * s) * dt + g * torch.sqrt(dt) * _cnoise(x)
        return self._decode(x, lens, T) * n, input_length


class SchroedingerBridgeAudioToAudioModel(_GenerativeBase):
    """Bridge between clean (t=0) and noisy (t=1) spectrograms under a VE schedule; the network predicts the clean data."""

    def __init__(self, cfg, trainer=None):
        super().__init__(cfg, trainer)
        s = cfg_get(self._cfg, "noise_schedule", {}) or {}
        self.k, self.c = cfg_get(s, "k", 2.6), cfg_get(s, "c", 0.4)
        self.t_min = cfg_get(s, "time_min", 1e-4)
        self.time_loss_weight = cfg_get(self._cfg, "estimator_output_time_loss_weight", 0.0)
        self._ready = True
        self._finish_init()

    def _sigma2(self, t):
        return self.c * (self.k ** (2 * t) - 1) / (2 * math.log(self.k))

    def _coeffs(self, t):
        s2t, s21 = self._sigma2(t), self._sigma2(torch.ones_like(t))
        sbar2 = s21 - s2t
        wx, wy = sbar2 / s21, s2t / s21
        return wx, wy, torch.sqrt(s2t * sbar2 / s21)

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        n = self._norm(x)
        noisy, lens = self._encode(x / n, xl)
        clean, _ = self._encode(y / n, xl)
        t = torch.rand(noisy.shape[0], device=noisy.device) * (1 - self.t_min) + self.t_min
        wx, wy, std = (v.view(-1, 1, 1, 1) for v in self._coeffs(t))
        xt = wx * clean + wy * noisy + std * _cnoise(noisy)
        est = self._net(xt, noisy, t, lens)
        loss = MaskedMSELoss()(est, clean, lens)
        if self.time_loss_weight > 0:
            T = x.shape[-1]
            y3 = y if y.dim() == 3 else y.unsqueeze(1)
            loss = loss + self.time_loss_weight * (self._decode(est, lens, T) - y3 / n).abs().mean()
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def forward(self, input_signal, input_length=None, num_steps: Optional[int] = None, process: str = "sde"):
        T = input_signal.shape[-1]
        n = self._norm(input_signal if input_signal.dim() == 3 else input_signal.unsqueeze(1))
        noisy, lens = self._encode(input_signal / n, input_length)
        steps = num_steps or self.num_steps
        ts = torch.linspace(1.0, self.t_min, steps + 1, device=noisy.device)
        x = noisy.clone()
        for i in range(steps):
            t, tn = ts[i].expand(x.shape[0]), ts[i + 1].expand(x.shape[0])
            est = self._net(x, noisy, t, lens)
            s2t, s2n = self._sigma2(t).view(-1, 1, 1, 1), self._sigma2(tn).view(-1, 1, 1, 1)
            w = s2n / s2t.clamp(min=1e-12)
            x = w * x + (1 - w) * est
            if process == "sde" and i < steps - 1:
                x = x + torch.sqrt((s2n * (1 - w)).clamp(min=0)) * _cnoise(x)
        return self._decode(x, lens, T) * n, input_length


# ---------------------------------------------------------------------------------------------- time-domain denoiser
class _Seasr(nn.Module):
    """Learned analysis filterbank (strided convolution) -> three convolution stages, each summarised by a GRU -> a stack of
    residual GRUs over the concatenated summaries -> a sigmoid mask on the analysis coefficients -> learned synthesis
    (transposed convolution) with tanh."""

    def __init__(self, hidden_nodes: int = 128, kernel_size: int = 320, f1: int = 1024, f2: int = 512, stride: int = 160, dropout: float = 0.0):
        super().__init__()
        f3 = 2 * hidden_nodes
        self.kernel, self.stride = kernel_size, stride
        self.analysis = nn.Conv1d(1, f1, kernel_size, stride=stride, bias=False)
        self.bn0 = nn.BatchNorm1d(f1, eps=1e-3)
        self.convs = nn.ModuleList([nn.Conv1d(f1, f2, 3, padding=1), nn.Conv1d(f2, f2, 3, padding=1), nn.Conv1d(f2, f2, 3, padding=1)])
        self.bns = nn.ModuleList([nn.BatchNorm1d(f2, eps=1e-3) for _ in range(3)])
        self.feat_gru = nn.ModuleList([nn.GRU(f1, f3, batch_first=True), nn.GRU(f2, f3, batch_first=True), nn.GRU(f2, f3, batch_first=True)])
        self.den = nn.ModuleList([nn.GRU(3 * f3 + f2, f1, batch_first=True), nn.GRU(f1, f1, batch_first=True), nn.GRU(f1, f1, batch_first=True),
                                  nn.GRU(f1, f1, batch_first=True)])
        self.drop = nn.Dropout(dropout)
        self.mask = nn.Linear(f1, f1)
        self.synthesis = nn.ConvTranspose1d(f1, 1, kernel_size, stride=stride)

    def forward(self, x0: torch.Tensor) -> torch.Tensor:
        """[B, 1, T] -> [B, 1, T]."""
        T = x0.shape[-1]
        pad = (-(T - self.kernel)) % self.stride if T >= self.kernel else self.kernel - T
        x0 = F.pad(x0, (0, pad))
        a = F.relu(self.analysis(x0))
        c0 = self.bn0(a)
        c1 = self.bns[0](F.leaky_relu(self.convs[0](c0)))
        c2 = self.bns[1](F.leaky_relu(self.convs[1](c1)))
        c3 = self.bns[2](F.leaky_relu(self.convs[2](c2)))
        g0, _ = self.feat_gru[0](c0.transpose(1, 2))
        g1, _ = self.feat_gru[1](c1.transpose(1, 2))
        g2, _ = self.feat_gru[2](c2.transpose(1, 2))
        h, _ = self.den[0](torch.cat([g0, g1, g2, c3.transpose(1, 2)], dim=2))
        h = self.drop(h) + c0.transpose(1, 2)
        h1, _ = self.den[1](h)
        h1 = self.drop(h1) + h
        h2, _ = self.den[2](h1)
        h, _ = self.den[3](h1 + self.drop(h2))
        m = torch.sigmoid(self.mask(h)).transpose(1, 2)
        return torch.tanh(self.synthesis(a * m))[..., :T]


class BNR2(AudioToAudioModel):
    """Background-noise removal in the time domain at 16 kHz with a combined loss (SI-SDR + spectral + recogniser features).
    Reference: ``audio/models/maxine/bnr.py`` (``BNR2``)."""

    def __init__(self, cfg: DictConfig, trainer=None, feature_extractor=None):
        super().__init__(cfg=cfg, trainer=trainer)
        from .losses import CombinedLoss

        cfg = self._cfg
        if int(self.sample_rate) != 16000:
            raise ValueError("this model is defined for 16 kHz audio")
        self.seasr = _Seasr(**{k: v for k, v in dict(cfg_get(cfg, "seasr", {}) or {}).items() if k != "_target_"})
        self.loss = CombinedLoss(sample_rate=self.sample_rate, feature_extractor=feature_extractor,
                                 **{k: v for k, v in dict(cfg_get(cfg, "loss", {}) or {}).items() if k != "_target_"})
        self._ready = True
        self._finish_init()

    def forward(self, input_signal, input_length=None):
        x = input_signal if input_signal.dim() == 3 else input_signal.unsqueeze(1)
        if x.shape[1] != 1:
            raise ValueError("single-channel input expected")
        y = self.seasr(x)
        if input_length is not None:
            y = y * (torch.arange(y.shape[-1], device=y.device)[None, None, :] < input_length[:, None, None])
        return y, input_length

    def training_step(self, batch, batch_idx):
        x, xl, y, yl = batch[:4]
        est, _ = self.forward(x, xl)
        n = min(est.shape[-1], y.shape[-1])
        loss = self.loss(est[..., :n], y[..., :n] if y.dim() == 3 else y[:, None, :n], xl.clamp(max=n))
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    def _eval_loss(self, est, tgt, lens):
        return self.loss(est, tgt, lens)

"""Abstract model kinds of the TTS collection — what a pipeline may rely on when it chains a spectrogram generator and a vocoder:
``SpectrogramGenerator`` (``parse`` text → tokens, ``generate_spectrogram`` tokens → mel), ``Vocoder`` (``convert_spectrogram_to_audio``),
``MelToSpec`` (mel → linear spectrogram), ``TextToWaveform`` (end-to-end), and ``NeedsNormalizer`` (optional text normalisation before
tokenising).  ``GriffinLimVocoder`` is a parameter-free vocoder (pseudo-inverse of the mel bank + phase reconstruction) for checking a
spectrogram generator without a trained neural vocoder.
Reference: ``tts/models/base.py``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Optional

import numpy as np
import torch

from ..core.modelpt import ModelPT


class NeedsNormalizer:
    """Mixin: ``_setup_normalizer(cfg)`` builds ``self.normalizer`` from ``cfg.text_normalizer`` (a ``_target_`` config or a callable);
    ``normalize_text`` applies it when ``text_normalizer_call_kwargs`` / a normaliser is set, and is the identity otherwise."""

    normalizer = None
    text_normalizer_call = None
    text_normalizer_call_kwargs: dict = {}

    def _setup_normalizer(self, cfg) -> None:
        tn = cfg.get("text_normalizer", None) if hasattr(cfg, "get") else None
        if tn is None:
            return
        if callable(tn):
            self.normalizer = tn
            self.text_normalizer_call = tn
        else:
            from ..core.instantiate import instantiate

            self.normalizer = instantiate(tn)
            self.text_normalizer_call = getattr(self.normalizer, "normalize", self.normalizer)
        kw = cfg.get("text_normalizer_call_kwargs", None)
        self.text_normalizer_call_kwargs = dict(kw) if kw else {}

    def normalize_text(self, text: str) -> str:
        if self.text_normalizer_call is None:
            return text
        return self.text_normalizer_call(text, **self.text_normalizer_call_kwargs)


class SpectrogramGenerator(ModelPT, NeedsNormalizer, ABC):
    @abstractmethod
    def parse(self, str_input: str, **kwargs) -> torch.Tensor:
        """Text → token tensor ``[1, T]`` that ``generate_spectrogram`` takes."""

    @abstractmethod
    def generate_spectrogram(self, tokens: torch.Tensor, **kwargs) -> torch.Tensor:
        """Tokens ``[B, T]`` → spectrogram ``[B, n_mels, frames]``."""


class Vocoder(ModelPT, ABC):
    @abstractmethod
    def convert_spectrogram_to_audio(self, spec: torch.Tensor, **kwargs) -> torch.Tensor:
        """Spectrogram ``[B, n_mels, frames]`` → audio ``[B, samples]``."""


class GlowVocoder(Vocoder):
    """Vocoders that share an invertible-flow formulation keep their mode (training / evaluation / inference) explicit and own an STFT pair."""

    OperationMode = type("OperationMode", (), {"training": 0, "validation": 1, "infer": 2})

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._mode = self.OperationMode.infer

    @property
    def mode(self):
        return self._mode

    def temp_mode(self, mode):
        outer = self

        class _Ctx:
            def __enter__(self_inner):
                self_inner.old, outer._mode = outer._mode, mode

            def __exit__(self_inner, *exc):
                outer._mode = self_inner.old
        return _Ctx()


class MelToSpec(ModelPT, ABC):
    @abstractmethod
    def convert_mel_spectrogram_to_linear(self, mel: torch.Tensor, **kwargs) -> torch.Tensor:
        """Mel ``[B, n_mels, frames]`` → linear magnitude ``[B, n_fft // 2 + 1, frames]``."""


class TextToWaveform(ModelPT, NeedsNormalizer, ABC):
    @abstractmethod
    def parse(self, str_input: str, **kwargs) -> torch.Tensor:
        """Text → token tensor."""

    @abstractmethod
    def convert_text_to_waveform(self, *, tokens: torch.Tensor, **kwargs) -> List[torch.Tensor]:
        """Tokens ``[B, T]`` → list of waveforms."""


class GriffinLimVocoder(torch.nn.Module):
    """Mel (log or linear) → waveform without learned parameters: least-squares inverse of the mel filter bank, then Griffin–Lim phase
    iterations with momentum.  A plain module (no trainer state): ``convert_spectrogram_to_audio(spec)``."""

    def __init__(self, sample_rate: int = 22050, n_fft: int = 1024, hop_length: int = 256, win_length: Optional[int] = None, n_mels: int = 80,
                 fmin: float = 0.0, fmax: Optional[float] = None, n_iters: int = 32, momentum: float = 0.99, log_input: bool = True, power: float = 1.0, mel_norm: Optional[str] = "slaney"):
        super().__init__()
        from ..modules.preprocessor import mel_filterbank

        fb = torch.as_tensor(np.asarray(mel_filterbank(sample_rate, n_fft, n_mels, fmin, fmax, norm=mel_norm)), dtype=torch.float32)
        self.register_buffer("fb_pinv", torch.linalg.pinv(fb), persistent=False)
        self.n_fft, self.hop, self.win = n_fft, hop_length, win_length or n_fft
        self.n_iters, self.momentum, self.log_input, self.power = n_iters, momentum, log_input, power
        self.register_buffer("window", torch.hann_window(self.win), persistent=False)

    def convert_mel_spectrogram_to_linear(self, mel: torch.Tensor) -> torch.Tensor:
        m = torch.exp(mel.float()) if self.log_input else mel.float()
        lin = torch.matmul(self.fb_pinv, m).clamp(min=1e-10)
        return lin if self.power == 1.0 else lin.pow(1.0 / self.power)

    @torch.no_grad()
    def convert_spectrogram_to_audio(self, spec: torch.Tensor, **_) -> torch.Tensor:
        mag = self.convert_mel_spectrogram_to_linear(spec)
        g = torch.Generator(device="cpu").manual_seed(0)
        ang = torch.exp(2j * torch.pi * torch.rand(mag.shape, generator=g)).to(mag.device)
        prev = torch.zeros_like(ang)
        for _ in range(self.n_iters):
            x = torch.istft(mag * ang, self.n_fft, self.hop, self.win, self.window)
            rebuilt = torch.stft(x, self.n_fft, self.hop, self.win, self.window, return_complex=True)
            ang = rebuilt - prev * (self.momentum / (1 + self.momentum))
            prev = rebuilt
            ang = ang / ang.abs().clamp(min=1e-16)
        return torch.istft(mag * ang, self.n_fft, self.hop, self.win, self.window)

    forward = convert_spectrogram_to_audio

"""Audio perception for speech-LLMs: waveform → features → ASR encoder → optional rotary time embedding → modality adapter
→ projection to the LLM width (reference: ``speechlm2/modules/perception.py:28-470``, ``modules/rote.py``)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..core.config import cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.module import NeuralModule


class IdentityConnector(nn.Module):
    def __init__(self, d_model: int = 0, **_):
        super().__init__()
        self.d_model = d_model

    def forward(self, audio_signal, length=None):
        return audio_signal, length


class ConformerMultiLayerFeatureExtractor(nn.Module):
    """Weighted sum of the outputs of several encoder layers (captured with forward hooks)."""

    def __init__(self, encoder, layer_idx_list, aggregator: str = "mean"):
        super().__init__()
        self.layer_idx_list = list(layer_idx_list)
        self.weights = nn.Parameter(torch.zeros(len(self.layer_idx_list))) if aggregator == "weighted" else None
        self._feats = {}
        for i in self.layer_idx_list:
            encoder.layers[i].register_forward_hook(self._hook(i))

    def _hook(self, i):
        def fn(module, inp, out):
            self._feats[i] = out[0] if isinstance(out, tuple) else out
        return fn

    def aggregate(self):
        xs = torch.stack([self._feats[i] for i in self.layer_idx_list], dim=0)
        if self.weights is None:
            return xs.mean(0)
        return (torch.softmax(self.weights, 0).view(-1, 1, 1, 1) * xs).sum(0)


class MultiLayerProjectionConnector(nn.Module):
    """Concatenate ``stack`` neighbouring frames (time reduction) and project with an MLP."""

    def __init__(self, d_model: int, output_dim: Optional[int] = None, hidden: Optional[int] = None, stack: int = 1, layers: int = 2):
        super().__init__()
        self.stack = stack
        dims = [d_model * stack] + [hidden or d_model * 2] * (layers - 1) + [output_dim or d_model]
        mods = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            mods.append(nn.Linear(a, b))
            if i < len(dims) - 2:
                mods.append(nn.GELU())
        self.net = nn.Sequential(*mods)

    def forward(self, audio_signal, length=None):
        x = audio_signal.transpose(1, 2)             # [B, T, D]
        B, T, D = x.shape
        T2 = T // self.stack
        x = x[:, : T2 * self.stack].reshape(B, T2, D * self.stack)
        x = self.net(x)
        if length is not None:
            length = torch.div(length, self.stack, rounding_mode="floor")
        return x.transpose(1, 2), length


class QformerConnector(nn.Module):
    """Window-level Q-Former: ``num_queries`` learnt queries cross-attend to every window of ``window`` encoder frames."""

    def __init__(self, d_model: int, num_queries: int = 1, window: int = 4, num_heads: int = 8, num_layers: int = 2):
        super().__init__()
        self.window, self.nq = window, num_queries
        self.query = nn.Parameter(torch.randn(num_queries, d_model) * 0.02)
        self.layers = nn.ModuleList([nn.TransformerDecoderLayer(d_model, num_heads, d_model * 4, dropout=0.0, batch_first=True,
                                                                norm_first=True) for _ in range(num_layers)])

    def forward(self, audio_signal, length=None):
        x = audio_signal.transpose(1, 2)
        B, T, D = x.shape
        W = self.window
        n = -(-T // W)
        x = torch.nn.functional.pad(x, (0, 0, 0, n * W - T)).reshape(B * n, W, D)
        q = self.query.unsqueeze(0).expand(B * n, -1, -1).to(x.dtype)
        for l in self.layers:
            q = l(q, x)
        out = q.reshape(B, n * self.nq, D)
        if length is not None:
            length = torch.div(length + W - 1, W, rounding_mode="floor") * self.nq
        return out.transpose(1, 2), length


class RotaryTimeEmbedding(nn.Module):
    """Rotate a fraction of the channels by an angle proportional to absolute time (RoTE)."""

    def __init__(self, dim: int, theta: float = 1200.0, rotary_fraction: float = 0.2, frame_seconds: float = 0.08):
        super().__init__()
        r = int(dim * rotary_fraction) // 2 * 2
        self.r, self.frame_seconds = r, frame_seconds
        self.register_buffer("inv_freq", 1.0 / (theta ** (torch.arange(0, r, 2).float() / max(r, 1))), persistent=False)

    def forward(self, x: torch.Tensor, offset_seconds: float = 0.0) -> torch.Tensor:
        """x: [B, T, D]."""
        if self.r == 0:
            return x
        t = torch.arange(x.shape[1], device=x.device).float() * self.frame_seconds + offset_seconds
        ang = t[:, None] * self.inv_freq[None, :]
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        a, b = x[..., : self.r: 2], x[..., 1: self.r: 2]
        rot = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
        return torch.cat([rot, x[..., self.r:]], dim=-1)


class AudioPerceptionModule(NeuralModule):
    def __init__(self, cfg=None, preprocessor=None, encoder=None, modality_adapter=None, output_dim: Optional[int] = None,
                 spec_augment=None, rote=None, **kw):
        super().__init__()
        if cfg is not None:
            preprocessor = preprocessor or cfg_get(cfg, "preprocessor", None)
            encoder = encoder or cfg_get(cfg, "encoder", None)
            modality_adapter = modality_adapter or cfg_get(cfg, "modality_adapter", None)
            output_dim = output_dim or cfg_get(cfg, "output_dim", None)
            spec_augment = spec_augment or cfg_get(cfg, "spec_augment", None)
            rote = rote or cfg_get(cfg, "rote", None)
        build = lambda c: c if isinstance(c, nn.Module) or c is None else from_config_dict(c)  # noqa: E731
        self.preprocessor = build(preprocessor)
        self.encoder = build(encoder)
        self.spec_augmentation = build(spec_augment)
        d_enc = self.encoder._feat_out if hasattr(self.encoder, "_feat_out") else self.encoder.d_model
        self.modality_adapter = build(modality_adapter) if modality_adapter is not None else IdentityConnector(d_enc)
        self.rote = build(rote)
        d_out = getattr(self.modality_adapter, "d_model", None) or getattr(self.modality_adapter, "_feat_out", None) or d_enc
        self.proj = nn.Linear(d_out, output_dim or d_out)
        self.output_dim = output_dim or d_out

    @property
    def token_equivalent_duration(self) -> float:
        feat = getattr(self.preprocessor, "featurizer", self.preprocessor)
        return feat.hop_length / feat.sample_rate * getattr(self.encoder, "subsampling_factor", 1)

    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns embeddings [B, T', output_dim] and their lengths."""
        if processed_signal is None:
            with torch.no_grad():
                processed_signal, processed_signal_length = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.spec_augmentation is not None and self.training:
            processed_signal = self.spec_augmentation(input_spec=processed_signal, length=processed_signal_length)
        enc, enc_len = self.encoder(audio_signal=processed_signal, length=processed_signal_length)[:2]
        if self.rote is not None:
            enc = self.rote(enc.transpose(1, 2)).transpose(1, 2)
        out = self.modality_adapter(audio_signal=enc, length=enc_len)
        enc, enc_len = out[0], out[1]
        x = enc.transpose(1, 2)
        x = ops.linear(x, self.proj.weight, self.proj.bias)
        return x, enc_len


class AudioTranscriptionPerceptionModule(AudioPerceptionModule):
    """Perception built around a complete ASR model (CTC, transducer or hybrid): its encoder feeds the modality adapter as usual,
    and its decoder transcribes the same encoder output, so that a speech-LLM can read the recogniser's hypothesis next to the
    audio embeddings (reference ``speechlm2/modules/perception.py`` ``AudioTranscriptionPerceptionModule``).

    ``asr``: an ASR model instance, a ``.nemo`` path, or a config dictionary ``{"_target_": <model class>, ...model cfg}``."""

    def __init__(self, cfg=None, asr=None, modality_adapter=None, output_dim: Optional[int] = None, freeze_asr_decoder: bool = True, **kw):
        if cfg is not None:
            asr = asr if asr is not None else cfg_get(cfg, "asr", None) or cfg_get(cfg, "pretrained_asr", None)
            modality_adapter = modality_adapter or cfg_get(cfg, "modality_adapter", None)
            output_dim = output_dim or cfg_get(cfg, "output_dim", None)
        if asr is None:
            raise ValueError("an ASR model (instance, .nemo path or config with _target_) is required")
        if isinstance(asr, str):
            from ..models.asr_model import ASRModel

            asr = ASRModel.restore_from(asr)
        elif not isinstance(asr, nn.Module):
            from ..core.config import to_container
            from ..core.instantiate import locate

            c = to_container(asr, resolve=True) if not isinstance(asr, dict) else dict(asr)
            asr = locate(c.pop("_target_"))(OmegaConfCreate(c))
        super().__init__(preprocessor=asr.preprocessor, encoder=asr.encoder, modality_adapter=modality_adapter, output_dim=output_dim,
                         spec_augment=getattr(asr, "spec_augmentation", None))
        self.asr = asr
        if freeze_asr_decoder:
            for name in ("decoder", "joint", "ctc_decoder"):
                m = getattr(asr, name, None)
                if isinstance(m, nn.Module):
                    for p in m.parameters():
                        p.requires_grad = False

    def forward_encoder(self, input_signal, input_signal_length):
        with torch.no_grad():
            feats, flen = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.spec_augmentation is not None and self.training:
            feats = self.spec_augmentation(input_spec=feats, length=flen)
        enc, enc_len = self.encoder(audio_signal=feats, length=flen)[:2]
        return enc, enc_len

    @torch.no_grad()
    def transcribe_encoded(self, encoded: torch.Tensor, encoded_len: torch.Tensor):
        """Hypotheses of the ASR model's own decoder for encoder output ``[B, D, T]`` (objects with ``.text``)."""
        asr = self.asr
        was = asr.training
        asr.eval()
        try:
            if hasattr(asr, "joint") and hasattr(asr, "decoding") and hasattr(asr.decoding, "rnnt_decoder_predictions_tensor"):
                hyps = asr.decoding.rnnt_decoder_predictions_tensor(encoded.detach(), encoded_len, return_hypotheses=True)
            else:
                dec = getattr(asr, "decoder", None) or getattr(asr, "ctc_decoder")
                logp = dec(encoder_output=encoded.detach())
                hyps = asr.decoding.ctc_decoder_predictions_tensor(logp, decoder_lengths=encoded_len, return_hypotheses=True)
            hyps = hyps[0] if isinstance(hyps, tuple) else hyps
        finally:
            asr.train(was)
        return hyps

    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None, encoded=None,
                encoded_len=None):
        if encoded is None:
            return super().forward(input_signal, input_signal_length, processed_signal, processed_signal_length)
        enc = encoded
        if self.rote is not None:
            enc = self.rote(enc.transpose(1, 2)).transpose(1, 2)
        out = self.modality_adapter(audio_signal=enc, length=encoded_len)
        x = ops.linear(out[0].transpose(1, 2), self.proj.weight, self.proj.bias)
        return x, out[1]


def OmegaConfCreate(d):
    from ..core.config import OmegaConf

    return OmegaConf.create(d)

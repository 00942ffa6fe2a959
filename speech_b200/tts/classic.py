"""Classic two-stage TTS: FastPitch (text → mel with explicit duration / pitch), HiFi-GAN vocoder (mel → waveform), the
alignment model (text ↔ mel attention trained with the forward-sum loss) and dictionary grapheme-to-phoneme conversion.

Reference: ``tts/models/fastpitch.py`` + ``modules/fastpitch.py`` / ``modules/transformer.py`` (FFTransformer),
``tts/models/hifigan.py``, ``tts/models/aligner.py`` + ``modules/aligner.py``, ``tts/g2p/models/en_us_arpabet.py`` /
``i18n_ipa.py``; monotonic alignment search ``tts/parts/utils/helpers.py:192-260`` (``binarize_attention``).
"""
from __future__ import annotations

import math
import re
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get, to_container
from ..core.modelpt import ModelPT
from ..core.adapters import AdapterModelPTMixin
from .base import SpectrogramGenerator, Vocoder
from .audio_codec import Discriminator, HiFiGANDecoder, MelLoss, discriminator_loss, feature_matching_loss, gan_update, generator_adv_loss
from .magpietts import ForwardSumLoss, beta_binomial_prior
from .transformer_2501 import Transformer


# ---------------------------------------------------------------------------------------------- G2P
class DictG2p:
    """Word → phoneme lookup with a CMUdict-style dictionary (``WORD  P1 P2 ...``); unknown words fall back to graphemes
    (or are spelled with ``oov_fn``).  ``phoneme_probability`` < 1 mixes graphemes in during training, as the reference does."""

    PUNCT = ",.!?;:'\"()-"

    def __init__(self, phoneme_dict, phoneme_probability: Optional[float] = None, apply_to_oov_word=None, ignore_ambiguous_words: bool = True,
                 seed: int = 0, grapheme_prefix: str = ""):
        self.dict: Dict[str, List[List[str]]] = {}
        if isinstance(phoneme_dict, dict):
            for w, p in phoneme_dict.items():
                self.dict[w.lower()] = [list(x) for x in p] if p and isinstance(p[0], (list, tuple)) else [list(p)]
        else:
            with open(phoneme_dict, encoding="latin-1") as f:
                for line in f:
                    if not line.strip() or line.startswith(";;;"):
                        continue
                    parts = line.split()
                    w = re.sub(r"\(\d+\)$", "", parts[0]).lower()
                    self.dict.setdefault(w, []).append(parts[1:])
        self.p, self.oov_fn, self.ignore_ambiguous = phoneme_probability, apply_to_oov_word, ignore_ambiguous_words
        self.rng = np.random.default_rng(seed)
        self.grapheme_prefix = grapheme_prefix

    def __call__(self, text: str) -> List[str]:
        out: List[str] = []
        for tok in re.findall(r"[\w']+|[^\w\s]|\s+", text):
            if tok.isspace():
                out.append(" ")
                continue
            w = tok.lower()
            prons = self.dict.get(w)
            use_phon = prons is not None and (self.p is None or self.rng.random() < self.p) and \
                not (self.ignore_ambiguous and len(prons) > 1)
            if use_phon:
                out.extend(prons[0])
            elif prons is None and self.oov_fn is not None and tok not in self.PUNCT:
                out.extend(self.oov_fn(w))
            else:
                out.extend(self.grapheme_prefix + ch for ch in w)
        return out


class PhonemeTokenizer:
    def __init__(self, g2p: DictG2p, symbols: Optional[Sequence[str]] = None, pad: str = "<pad>", blank: str = "<blank>", oov: str = "<oov>"):
        syms = list(symbols) if symbols is not None else sorted({p for prons in g2p.dict.values() for pr in prons for p in pr})
        chars = list("abcdefghijklmnopqrstuvwxyz' ") + list(DictG2p.PUNCT)
        self.tokens = [pad, blank, oov] + [s for s in dict.fromkeys(syms + chars)]
        self._t2i = {t: i for i, t in enumerate(self.tokens)}
        self.g2p, self.pad, self.blank, self.oov = g2p, 0, 1, 2

    @property
    def vocab_size(self):
        return len(self.tokens)

    def text_to_ids(self, text: str) -> List[int]:
        return [self._t2i.get(p, self.oov) for p in self.g2p(text)]

    encode = text_to_ids

    def ids_to_tokens(self, ids):
        return [self.tokens[int(i)] for i in ids]


def build_text_tokenizer(cfg):
    """``text_tokenizer`` block of a TTS model config -> tokenizer.  ``type``: ``char`` (``chars``: the alphabet), ``phoneme``
    (CMUdict-style ``phoneme_dict`` path or mapping, optional ``phoneme_probability``) or ``ipa`` (``phoneme_dict`` of IPA
    strings, ``locale``, ``heteronyms``); ids 0..2 are pad / blank / oov for the phoneme kinds."""
    if cfg is None:
        return None
    get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
    if get("_target_", None):
        # a tokenizer class by path (e.g. speech_b200.tokenizers.tts.IPATokenizer) with a nested ``g2p`` block built first
        from ..core.instantiate import instantiate

        return instantiate(cfg)
    kind = get("type", "char")
    if kind == "char":
        from ..tokenizers import CharTokenizer

        return CharTokenizer(list(get("chars", "abcdefghijklmnopqrstuvwxyz' .,?!-")))
    if kind == "phoneme":
        d = get("phoneme_dict")
        return PhonemeTokenizer(DictG2p(dict(d) if not isinstance(d, str) else d, phoneme_probability=get("phoneme_probability", None)))
    if kind == "ipa":
        from .g2p import IpaG2p

        d = get("phoneme_dict")
        g2p = IpaG2p(dict(d) if not isinstance(d, str) else d, locale=get("locale", "en-US"), heteronyms=get("heteronyms", None),
                     phoneme_probability=get("phoneme_probability", None), grapheme_prefix=get("grapheme_prefix", ""), use_chars=True)
        tok = PhonemeTokenizer.__new__(PhonemeTokenizer)
        chars = sorted({g2p.prefix + c for c in (get("chars", None) or "ABCDEFGHIJKLMNOPQRSTUVWXYZ'")}) + [" "] + list(DictG2p.PUNCT)
        tok.tokens = ["<pad>", "<blank>", "<oov>"] + list(dict.fromkeys(sorted(g2p.symbols) + chars))
        tok._t2i = {t: i for i, t in enumerate(tok.tokens)}
        tok.g2p, tok.pad, tok.blank, tok.oov = g2p, 0, 1, 2
        return tok
    raise ValueError(f"unknown text tokenizer type {kind!r}")


def _tts_loader(model, c, audio_only: bool = False):
    """Text + audio batches for the acoustic models; ``audio_only`` drops the text (vocoder)."""
    if c is None or (c.get("manifest_filepath", None) is None and c.get("synthetic", None) is None):
        return None
    from .data import build_tts_dataloader

    return build_tts_dataloader(c, model.tokenizer if not audio_only else (model.tokenizer or _NoText()), cfg_get(model._cfg, "sample_rate", 22050),
                                audio_only=audio_only)


class _NoText:
    vocab_size = 0

    def text_to_ids(self, text):
        return []


# ---------------------------------------------------------------------------------------------- alignment utilities
def binarize_attention(attn: torch.Tensor, in_lens: torch.Tensor, out_lens: torch.Tensor) -> torch.Tensor:
    """Monotonic alignment search: hard 0/1 path [B, T_out, T_in] maximising the sum of log attention."""
    B = attn.shape[0]
    out = torch.zeros_like(attn)
    la = torch.log(attn.detach().float().clamp(min=1e-12)).cpu().numpy()
    for b in range(B):
        T, N = int(out_lens[b]), int(in_lens[b])
        a = la[b, :T, :N]
        Q = np.full((T, N), -np.inf)
        Q[0, 0] = a[0, 0]
        for t in range(1, T):
            for n in range(min(N, t + 1)):
                prev = Q[t - 1, n] if n == 0 else max(Q[t - 1, n], Q[t - 1, n - 1])
                Q[t, n] = prev + a[t, n]
        n = N - 1
        for t in range(T - 1, -1, -1):
            out[b, t, n] = 1.0
            if t > 0 and n > 0 and (n == t or Q[t - 1, n - 1] >= Q[t - 1, n]):
                n -= 1
    return out


def regulate_len(durations: torch.Tensor, enc: torch.Tensor, pace: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Repeat every encoder step ``round(duration / pace)`` times.  durations [B, N], enc [B, N, D] → ([B, T, D], lens)."""
    reps = torch.round(durations.float() / pace).long().clamp(min=0)
    lens = reps.sum(1)
    T = int(lens.max()) if lens.numel() else 0
    out = enc.new_zeros((enc.shape[0], T, enc.shape[2]))
    for b in range(enc.shape[0]):
        r = torch.repeat_interleave(enc[b], reps[b], dim=0)
        out[b, : r.shape[0]] = r
    return out, lens


class ConvAttention(nn.Module):
    """Aligner attention: conv-encoded text keys and mel queries, distance-based soft attention (+ optional prior)."""

    def __init__(self, n_mel: int = 80, n_text: int = 256, n_att: int = 80, temperature: float = 0.0005):
        super().__init__()
        self.temperature = temperature
        self.key_proj = nn.Sequential(nn.Conv1d(n_text, n_text * 2, 3, padding=1), nn.ReLU(), nn.Conv1d(n_text * 2, n_att, 1))
        self.query_proj = nn.Sequential(nn.Conv1d(n_mel, n_mel * 2, 3, padding=1), nn.ReLU(), nn.Conv1d(n_mel * 2, n_mel, 1), nn.ReLU(),
                                        nn.Conv1d(n_mel, n_att, 1))

    def forward(self, queries, keys, mask=None, attn_prior=None):
        """queries [B, n_mel, T], keys [B, n_text, N], mask [B, N] True at padding → (soft attention [B, 1, T, N], log-probs)."""
        k, q = self.key_proj(keys), self.query_proj(queries)
        d = ((q.unsqueeze(3) - k.unsqueeze(2)) ** 2).sum(1, keepdim=True)
        logp = -self.temperature * d
        if attn_prior is not None:
            logp = torch.log_softmax(logp, dim=3) + torch.log(attn_prior.unsqueeze(1) + 1e-8)
        if mask is not None:
            logp = logp.masked_fill(mask.unsqueeze(1).unsqueeze(1), -float("inf"))
        return torch.softmax(logp, dim=3), logp


class TemporalPredictor(nn.Module):
    def __init__(self, d_in: int, d_hidden: int = 256, kernel: int = 3, dropout: float = 0.1, n_layers: int = 2):
        super().__init__()
        layers, c = [], d_in
        for _ in range(n_layers):
            layers.append(nn.ModuleList([nn.Conv1d(c, d_hidden, kernel, padding=kernel // 2), nn.LayerNorm(d_hidden), nn.Dropout(dropout)]))
            c = d_hidden
        self.layers = nn.ModuleList(layers)
        self.fc = nn.Linear(d_hidden, 1)

    def forward(self, x, mask):
        """x [B, N, D], mask [B, N] True at valid positions → [B, N]."""
        h = x * mask.unsqueeze(-1)
        for conv, ln, dr in self.layers:
            h = dr(ln(F.relu(conv(h.transpose(1, 2)).transpose(1, 2))))
        return self.fc(h).squeeze(-1) * mask


class FastPitchModel(SpectrogramGenerator, AdapterModelPTMixin):
    adapter_module_names = ("encoder", "decoder")
    default_adapter_module_name = "encoder"

    def __init__(self, cfg: DictConfig, trainer=None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.tokenizer = tokenizer if tokenizer is not None else build_text_tokenizer(cfg_get(cfg, "text_tokenizer", None))
        self._setup_normalizer(cfg)
        # the datasets append <bos> / <eos> as vocab_size and vocab_size + 1
        n_sym = cfg_get(cfg, "n_symbols", None) or (self.tokenizer.vocab_size + 2 if self.tokenizer is not None else 128)
        d = cfg_get(cfg, "symbols_embedding_dim", 384)
        self.n_mel = cfg_get(cfg, "n_mel_channels", 80)
        self.embedding = nn.Embedding(n_sym, d, padding_idx=0)
        tf = dict(d_model=d, d_ffn=cfg_get(cfg, "d_inner", 1536), sa_n_heads=cfg_get(cfg, "n_heads", 1), kernel_size=3, p_dropout=0.1,
                  is_causal=False, use_learnable_pos_emb=True, max_length_causal_mask=2048)
        self.encoder = Transformer(n_layers=cfg_get(cfg, "encoder_layers", 6), **tf)
        self.decoder = Transformer(n_layers=cfg_get(cfg, "decoder_layers", 6), **tf)
        self.duration_predictor = TemporalPredictor(d)
        self.pitch_predictor = TemporalPredictor(d)
        self.pitch_emb = nn.Conv1d(1, d, 3, padding=1)
        self.proj = nn.Linear(d, self.n_mel)
        self.aligner = ConvAttention(self.n_mel, d)
        self.forward_sum = ForwardSumLoss()
        n_spk = cfg_get(cfg, "n_speakers", 1)
        self.speaker_emb = nn.Embedding(n_spk, d) if n_spk > 1 else None
        # optional speaker encoder (look-up table + global style tokens of a reference spectrogram + pre-computed embedding)
        self.speaker_encoder = None
        if cfg_get(cfg, "speaker_encoder", None):
            from .submodules import SpeakerEncoder

            self.speaker_encoder = SpeakerEncoder.from_config(to_container(cfg_get(cfg, "speaker_encoder"), resolve=True), d)
        self.mel = MelLoss(cfg_get(cfg, "sample_rate", 22050), self.n_mel, cfg_get(cfg, "n_fft", 1024), cfg_get(cfg, "hop_length", 256),
                           cfg_get(cfg, "win_length", 1024))
        self.w = {"dur": cfg_get(cfg, "dur_loss_scale", 0.1), "pitch": cfg_get(cfg, "pitch_loss_scale", 0.1), "align": cfg_get(cfg, "align_loss_scale", 1.0)}
        self.bin_loss_start = cfg_get(cfg, "bin_loss_warmup_epochs", 100)
        self.restore_adapters_from_cfg()
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "forward_sum"):                             # the base constructor calls this before the layers exist
            super()._setup_dataloaders_from_cfg()

    def setup_training_data(self, c):
        self._train_dl = _tts_loader(self, c)

    def setup_validation_data(self, c):
        self._validation_dl = _tts_loader(self, c)

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        with torch.no_grad():
            return {"val_loss": self.training_step(batch, batch_idx)["loss"]}

    @staticmethod
    def estimate_pitch(audio: torch.Tensor, hop: int, sr: int, fmin: float = 60.0, fmax: float = 400.0) -> torch.Tensor:
        """Frame-wise f0 by autocorrelation peak picking (0 where unvoiced)."""
        B, n = audio.shape
        win = 4 * hop
        T = n // hop + 1
        x = F.pad(audio, (win // 2, win // 2 + hop))
        fr = x.unfold(1, win, hop)[:, :T]
        fr = fr - fr.mean(-1, keepdim=True)
        spec = torch.fft.rfft(fr, 2 * win)
        ac = torch.fft.irfft(spec.abs() ** 2)[..., :win]
        lo, hi = int(sr / fmax), min(win - 1, int(sr / fmin))
        seg = ac[..., lo:hi]
        peak, idx = seg.max(-1)
        f0 = sr / (idx + lo).float()
        return torch.where(peak > 0.3 * ac[..., 0].clamp(min=1e-8), f0, torch.zeros_like(f0))

    def forward(self, text, text_len, mel=None, mel_len=None, pitch=None, speaker=None, pace: float = 1.0, reference_spec=None, reference_spec_lens=None):
        mask = torch.arange(text.shape[1], device=text.device)[None] < text_len[:, None]
        x = self.embedding(text)
        if self.speaker_emb is not None and speaker is not None:
            x = x + self.speaker_emb(speaker).unsqueeze(1)
        if self.speaker_encoder is not None:
            if reference_spec is None and mel is not None and self.speaker_encoder.gst_module is not None:
                reference_spec, reference_spec_lens = mel, mel_len          # training: the target utterance is its own style reference
            cond = self.speaker_encoder(batch_size=text.shape[0], speaker=speaker, reference_spec=reference_spec, reference_spec_lens=reference_spec_lens)
            if cond is not None:
                x = x + cond.to(x.dtype)
        enc = self.encoder(x, mask)["output"].float()
        log_dur = self.duration_predictor(enc, mask)
        pitch_pred = self.pitch_predictor(enc, mask)
        attn_soft = attn_logp = attn_hard = None
        if mel is not None:
            T = mel.shape[2]
            prior = torch.zeros((text.shape[0], T, text.shape[1]), device=text.device)
            for b in range(text.shape[0]):
                prior[b, : int(mel_len[b]), : int(text_len[b])] = beta_binomial_prior(int(text_len[b]), int(mel_len[b])).to(text.device)
            attn_soft, attn_logp = self.aligner(mel, x.transpose(1, 2).float(), ~mask, prior)
            attn_hard = binarize_attention(attn_soft.squeeze(1), text_len, mel_len)
            dur = attn_hard.sum(1)
            pitch_tok = (torch.bmm(attn_hard.transpose(1, 2), pitch.unsqueeze(-1)).squeeze(-1) / dur.clamp(min=1)) if pitch is not None else pitch_pred
        else:
            dur = torch.clamp(torch.exp(log_dur) - 1, min=0) * mask
            pitch_tok = pitch_pred
        enc = enc + self.pitch_emb(pitch_tok.unsqueeze(1)).transpose(1, 2)
        frames, flen = regulate_len(dur, enc, pace)
        fmask = torch.arange(frames.shape[1], device=text.device)[None] < flen[:, None]
        dec = self.decoder(frames, fmask)["output"].float()
        return {"mel": self.proj(dec).transpose(1, 2), "mel_len": flen, "log_dur": log_dur, "pitch_pred": pitch_pred, "dur": dur,
                "pitch_tok": pitch_tok, "attn_soft": attn_soft, "attn_logp": attn_logp, "attn_hard": attn_hard, "mask": mask}

    def training_step(self, batch, batch_idx):
        text, text_len, audio, audio_len = batch[:4]
        hop = self.mel.hop
        with torch.no_grad():
            mel = self.mel.mel(audio)
            mel_len = torch.div(audio_len, hop, rounding_mode="floor") + 1
            pitch = self.estimate_pitch(audio, hop, cfg_get(self._cfg, "sample_rate", 22050))[:, : mel.shape[2]]
            pitch = F.pad(pitch, (0, mel.shape[2] - pitch.shape[1])) / 100.0
        o = self.forward(text, text_len, mel, mel_len, pitch)
        T = min(o["mel"].shape[2], mel.shape[2])
        fm = (torch.arange(T, device=mel.device)[None] < mel_len[:, None]).unsqueeze(1)
        mel_loss = ((o["mel"][..., :T] - mel[..., :T]) ** 2 * fm).sum() / (fm.sum() * self.n_mel).clamp(min=1)
        m = o["mask"]
        dur_loss = ((o["log_dur"] - torch.log(o["dur"] + 1)) ** 2 * m).sum() / m.sum()
        pitch_loss = ((o["pitch_pred"] - o["pitch_tok"].detach()) ** 2 * m).sum() / m.sum()
        align = self.forward_sum(o["attn_logp"].squeeze(1), text_len, mel_len)
        loss = mel_loss + self.w["dur"] * dur_loss + self.w["pitch"] * pitch_loss + self.w["align"] * align
        if self.current_epoch >= self.bin_loss_start:
            loss = loss - (o["attn_hard"] * torch.log(o["attn_soft"].squeeze(1).clamp(min=1e-12))).sum() / o["attn_hard"].sum().clamp(min=1)
        self.log_dict({"train_loss": loss.detach(), "mel_loss": mel_loss.detach(), "dur_loss": dur_loss.detach(), "align_loss": align.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def generate_spectrogram(self, tokens: torch.Tensor, speaker=None, pace: float = 1.0, reference_spec=None, reference_spec_lens=None) -> torch.Tensor:
        self.eval()
        lens = torch.tensor([tokens.shape[1]] * tokens.shape[0], device=tokens.device)
        return self.forward(tokens, lens, speaker=speaker, pace=pace, reference_spec=reference_spec, reference_spec_lens=reference_spec_lens)["mel"]

    def parse(self, text: str, normalize: bool = True, **kwargs) -> torch.Tensor:
        if normalize:
            text = self.normalize_text(text)
        return torch.tensor([self.tokenizer.text_to_ids(text)], dtype=torch.long, device=self.device)


class HifiGanModel(Vocoder):
    """Vocoder: mel spectrogram → waveform (generator = ``HiFiGANDecoder``; multi-period + STFT discriminators)."""

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.sample_rate = cfg_get(cfg, "sample_rate", 22050)
        g = dict(cfg_get(cfg, "generator", {}) or {})
        self.n_mel = g.pop("input_dim", 80)
        self.generator = HiFiGANDecoder(input_dim=self.n_mel, **g)
        self.discriminator = Discriminator(**dict(cfg_get(cfg, "discriminator", {}) or {}))
        self.mel = MelLoss(self.sample_rate, self.n_mel, **dict(cfg_get(cfg, "mel", {}) or {}))
        self.l1_factor = cfg_get(cfg, "l1_loss_factor", 45.0)
        self.tokenizer = None
        self.automatic_optimization = False
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "l1_factor"):
            super()._setup_dataloaders_from_cfg()

    def setup_training_data(self, c):
        self._train_dl = _tts_loader(self, c, audio_only=True)

    def setup_validation_data(self, c):
        self._validation_dl = _tts_loader(self, c, audio_only=True)

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        audio, audio_len = batch[0], batch[1]
        with torch.no_grad():
            gen = self.forward(self.mel.mel(audio))
            n = min(gen.shape[-1], audio.shape[-1])
            return {"val_loss": self.mel(audio[..., :n], gen[..., :n], audio_len)}

    def forward(self, spec: torch.Tensor) -> torch.Tensor:
        lens = torch.full((spec.shape[0],), spec.shape[2], device=spec.device, dtype=torch.long)
        return self.generator(spec, lens)[0]

    def convert_spectrogram_to_audio(self, spec: torch.Tensor, **kwargs) -> torch.Tensor:
        return self.forward(spec)

    def configure_optimizers(self):
        lr = cfg_get(cfg_get(self._cfg, "optim", {}), "lr", 2e-4)
        self._optimizers = [torch.optim.AdamW(self.generator.parameters(), lr=lr, betas=(0.8, 0.99)),
                            torch.optim.AdamW(self.discriminator.parameters(), lr=lr, betas=(0.8, 0.99))]
        return self._optimizers

    def training_step(self, batch, batch_idx):
        audio, audio_len = batch[0], batch[1]
        with torch.no_grad():
            mel = self.mel.mel(audio)
        gen = self.forward(mel)
        n = min(gen.shape[-1], audio.shape[-1])
        audio, gen = audio[..., :n], gen[..., :n]
        opts = getattr(self, "_optimizers", None)
        if opts is not None:
            sr, sg, _, _ = self.discriminator(audio, gen.detach())
            d = discriminator_loss(sr, sg)
            gan_update(self, d, opts[1], standalone_step=True)
        sr, sg, fr, fg = self.discriminator(audio, gen)
        loss = self.l1_factor * self.mel(audio, gen, audio_len) + generator_adv_loss(sg) + 2.0 * feature_matching_loss(fr, fg)
        self.log_dict({"train_loss": loss.detach()})
        if opts is not None:
            gan_update(self, loss, opts[0], standalone_step=False)
        return {"loss": loss}


class AlignerModel(ModelPT):
    """Learns text ↔ mel alignments alone (used to extract durations for other models)."""

    def __init__(self, cfg: DictConfig, trainer=None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.tokenizer = tokenizer if tokenizer is not None else build_text_tokenizer(cfg_get(cfg, "text_tokenizer", None))
        d = cfg_get(cfg, "symbols_embedding_dim", 256)
        self.n_mel = cfg_get(cfg, "n_mel_channels", 80)
        self.embed = nn.Embedding(cfg_get(cfg, "n_symbols", None) or (self.tokenizer.vocab_size + 2 if self.tokenizer is not None else 128), d)
        self.alignment_encoder = ConvAttention(self.n_mel, d)
        self.forward_sum = ForwardSumLoss()
        self.mel = MelLoss(cfg_get(cfg, "sample_rate", 22050), self.n_mel, **dict(cfg_get(cfg, "mel", {}) or {}))
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "mel"):
            super()._setup_dataloaders_from_cfg()

    def setup_training_data(self, c):
        self._train_dl = _tts_loader(self, c)

    def setup_validation_data(self, c):
        self._validation_dl = None

    def forward(self, spec, spec_len, text, text_len, attn_prior=None):
        mask = torch.arange(text.shape[1], device=text.device)[None] >= text_len[:, None]
        soft, logp = self.alignment_encoder(spec, self.embed(text).transpose(1, 2), mask, attn_prior)
        return soft, logp

    def training_step(self, batch, batch_idx):
        text, text_len, audio, audio_len = batch[:4]
        with torch.no_grad():
            spec = self.mel.mel(audio)
            spec_len = torch.div(audio_len, self.mel.hop, rounding_mode="floor") + 1
        soft, logp = self.forward(spec, spec_len, text, text_len)
        loss = self.forward_sum(logp.squeeze(1), text_len, spec_len)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def durations(self, spec, spec_len, text, text_len) -> torch.Tensor:
        soft, _ = self.forward(spec, spec_len, text, text_len)
        return binarize_attention(soft.squeeze(1), text_len, spec_len).sum(1)


class SSLDisentangler(ModelPT):
    """Content / speaker disentanglement on a self-supervised speech encoder (features for voice conversion and zero-shot TTS).

    One Conformer encoder, two heads: the *content* head maps every frame to an embedding and to phoneme logits trained with CTC;
    the *speaker* head pools the frames (mean + standard deviation), maps to an embedding and classifies the speaker.  The
    content embedding is normalised per utterance (instance norm over time) so that speaker-dependent offsets do not leak into it.
    ``forward`` returns ``(content_logits, content_embedding [B, T, Dc], speaker_logits, speaker_embedding [B, Ds], lengths)``.
    Reference: ``tts/models/ssl_tts.py`` (``SSLDisentangler``: downstream heads, per-task losses, ``forward_for_export``).
    """

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        from ..core.instantiate import instantiate
        from ..modules.preprocessor import AudioToMelSpectrogramPreprocessor

        cfg = self._cfg
        self.preprocessor = AudioToMelSpectrogramPreprocessor(**{k: v for k, v in dict(cfg.preprocessor).items() if k != "_target_"})
        self.encoder = instantiate(cfg.encoder)
        d = int(cfg_get(cfg, "encoder_dim", getattr(self.encoder, "d_model", 256)))
        self.content_dim, self.speaker_dim = int(cfg_get(cfg, "content_emb_dim", 128)), int(cfg_get(cfg, "speaker_emb_dim", 128))
        self.num_phonemes, self.num_speakers = int(cfg_get(cfg, "num_phonemes", 64)), int(cfg_get(cfg, "num_speakers", 16))
        self.content_proj = nn.Linear(d, self.content_dim)
        self.content_out = nn.Linear(self.content_dim, self.num_phonemes + 1)           # + CTC blank (last index)
        self.speaker_proj = nn.Linear(2 * d, self.speaker_dim)
        self.speaker_out = nn.Linear(self.speaker_dim, self.num_speakers)
        self.content_weight, self.speaker_weight = float(cfg_get(cfg, "content_loss_weight", 1.0)), float(cfg_get(cfg, "speaker_loss_weight", 1.0))
        self._ssl_ready = True
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if getattr(self, "_ssl_ready", False):
            super()._setup_dataloaders_from_cfg()

    def _loader(self, c):
        """Manifest lines ``{"audio_filepath", "duration", "text" (space-separated content units, e.g. phonemes), "speaker"}``; unit and
        speaker inventories come from ``content_units`` / ``speakers`` of the data block (lists) or are collected from the manifest."""
        if c is None or (c.get("manifest_filepath", None) is None and c.get("synthetic", None) is None):
            return None
        from ..data.audio_to_text import load_audio, read_manifest

        sr = int(cfg_get(self._cfg, "sample_rate", 16000))
        if c.get("synthetic", None) is not None:
            syn = dict(c.synthetic)
            g = torch.Generator().manual_seed(int(syn.get("seed", 0)))
            items = [(0.1 * torch.randn(int(sr * 0.5), generator=g), torch.randint(0, self.num_phonemes, (4,), generator=g),
                      int(torch.randint(0, self.num_speakers, (1,), generator=g))) for _ in range(int(syn.get("num_samples", 8)))]
        else:
            rows = read_manifest(c.manifest_filepath, max_duration=c.get("max_duration", None))
            units = list(c.get("content_units", None) or sorted({u for r in rows for u in r["text"].split()}))
            spks = list(c.get("speakers", None) or sorted({str(r["speaker"]) for r in rows}))
            if len(units) > self.num_phonemes or len(spks) > self.num_speakers:
                raise ValueError(f"{len(units)} content units / {len(spks)} speakers exceed num_phonemes={self.num_phonemes} / num_speakers={self.num_speakers}")
            u2i, s2i = {u: i for i, u in enumerate(units)}, {s: i for i, s in enumerate(spks)}

            class _DS(torch.utils.data.Dataset):
                def __len__(self_inner):
                    return len(rows)

                def __getitem__(self_inner, i):
                    r = rows[i]
                    a = torch.as_tensor(load_audio(r["audio_filepath"], target_sr=sr, offset=float(r.get("offset", 0) or 0), duration=r.get("duration")), dtype=torch.float32)
                    return a, torch.tensor([u2i[u] for u in r["text"].split()], dtype=torch.long), s2i[str(r["speaker"])]
            items = _DS()

        def collate(batch):
            pad = torch.nn.utils.rnn.pad_sequence
            a, p, s = zip(*batch)
            return (pad(a, batch_first=True), torch.tensor([len(x) for x in a]), pad(p, batch_first=True), torch.tensor([len(x) for x in p]), torch.tensor(s))
        return torch.utils.data.DataLoader(items, batch_size=int(c.get("batch_size", 8)), shuffle=bool(c.get("shuffle", False)), collate_fn=collate,
                                           num_workers=int(c.get("num_workers", 0)))

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        with torch.no_grad():
            return {"val_loss": self.training_step(batch, batch_idx)["loss"]}

    def forward(self, input_signal, input_signal_length):
        feats, flen = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        enc, elen = self.encoder(audio_signal=feats, length=flen)                        # [B, D, T]
        h = enc.transpose(1, 2).float()
        mask = (torch.arange(h.shape[1], device=h.device)[None] < elen[:, None]).unsqueeze(-1)
        n = elen.clamp(min=1).view(-1, 1).float()
        mean = (h * mask).sum(1) / n
        std = (((h - mean.unsqueeze(1)) ** 2 * mask).sum(1) / n).clamp(min=1e-5).sqrt()
        spk_emb = F.normalize(self.speaker_proj(torch.cat([mean, std], dim=-1)), dim=-1)
        c = self.content_proj(h)
        cm = (c * mask).sum(1, keepdim=True) / n.unsqueeze(-1)
        cs = (((c - cm) ** 2 * mask).sum(1, keepdim=True) / n.unsqueeze(-1)).clamp(min=1e-5).sqrt()
        content = (c - cm) / cs * mask
        return self.content_out(content), content, self.speaker_out(spk_emb), spk_emb, elen

    def training_step(self, batch, batch_idx):
        """batch: audio [B, S], audio_len [B], phonemes [B, U], phoneme_len [B], speaker [B]."""
        audio, alen, ph, phl, spk = batch
        logits, _, spk_logits, _, elen = self(audio, alen)
        ctc = F.ctc_loss(logits.log_softmax(-1).transpose(0, 1), ph, elen, phl, blank=self.num_phonemes, zero_infinity=True)
        ce = F.cross_entropy(spk_logits, spk)
        loss = self.content_weight * ctc + self.speaker_weight * ce
        self.log_dict({"train_loss": loss.detach(), "content_loss": ctc.detach(), "speaker_loss": ce.detach(),
                       "speaker_acc": (spk_logits.argmax(-1) == spk).float().mean()})
        return {"loss": loss}

    @torch.no_grad()
    def forward_for_export(self, input_signal, input_signal_length):
        _, content, _, spk, elen = self(input_signal, input_signal_length)
        return content, spk, elen

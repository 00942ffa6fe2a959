"""FastPitch driven by self-supervised speech representations instead of text: the input is a sequence of *content* embeddings (from the content
head of ``SSLDisentangler``, optionally de-duplicated into segments with durations) plus one *speaker* embedding; the model predicts segment
durations and a pitch contour, expands the segments to frames and decodes a mel spectrogram.  Swapping the speaker embedding of one utterance for
another speaker's gives voice conversion; ``generate_wav`` runs the vocoder on the result.
Batch: ``content_embs [B, Dc, N]``, ``content_lens [B]``, ``speaker_emb [B, Ds]``, ``mel [B, n_mel, T]``, ``mel_lens [B]``, ``durations [B, N]`` (frames per
segment; ``None`` = one segment per frame) and ``pitch [B, T]`` (normalised contour, 0 where unvoiced).
Reference: ``tts/models/fastpitch_ssl.py`` (``FastPitchModel_SSL``), ``examples/tts/fastpitch_ssl.py``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from ..core.modelpt import ModelPT
from .classic import TemporalPredictor, regulate_len
from .transformer_2501 import Transformer


class FastPitchModel_SSL(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None, vocoder=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        d = int(cfg_get(cfg, "symbols_embedding_dim", 384))
        self.n_mel = int(cfg_get(cfg, "n_mel_channels", 80))
        self.content_dim, self.speaker_dim = int(cfg_get(cfg, "content_emb_indim", 128)), int(cfg_get(cfg, "speaker_emb_indim", 256))
        self.content_proj = nn.Linear(self.content_dim, d)
        self.speaker_proj = nn.Linear(self.speaker_dim, d)
        tf = dict(d_model=d, d_ffn=int(cfg_get(cfg, "d_inner", 1536)), sa_n_heads=int(cfg_get(cfg, "n_heads", 1)), kernel_size=3, p_dropout=float(cfg_get(cfg, "dropout", 0.1)),
                  is_causal=False, use_learnable_pos_emb=True, max_length_causal_mask=int(cfg_get(cfg, "max_frames", 4096)))
        self.encoder = Transformer(n_layers=int(cfg_get(cfg, "encoder_layers", 4)), **tf)
        self.decoder = Transformer(n_layers=int(cfg_get(cfg, "decoder_layers", 4)), **tf)
        self.use_duration_predictor = bool(cfg_get(cfg, "use_duration_predictor", True))
        self.duration_predictor = TemporalPredictor(d) if self.use_duration_predictor else None
        self.pitch_conditioning = bool(cfg_get(cfg, "pitch_conditioning", True))
        self.pitch_predictor = TemporalPredictor(d) if self.pitch_conditioning else None
        self.pitch_emb = nn.Conv1d(1, d, 3, padding=1) if self.pitch_conditioning else None
        self.proj = nn.Linear(d, self.n_mel)
        self.w = {"dur": float(cfg_get(cfg, "dur_loss_scale", 0.1)), "pitch": float(cfg_get(cfg, "pitch_loss_scale", 0.1))}
        self.vocoder = [vocoder] if vocoder is not None else None          # in a list: not a sub-module, not saved with the model
        if not self._is_model_being_restored and self._train_dl is None and hasattr(self, "proj"):
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "proj"):
            super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ data: pre-computed features (.pt dictionaries) or synthetic
    def _loader(self, c):
        if c is None:
            return None
        c = dict(c)
        syn = c.get("synthetic")
        if syn is None and c.get("manifest_filepath") is None:
            return None
        model = self

        class _DS(torch.utils.data.Dataset):
            def __init__(self):
                if syn is not None:
                    self.n, self.items = int(dict(syn).get("num_samples", 8)), None
                else:
                    from ..data.audio_to_text import read_manifest

                    self.items = read_manifest(c["manifest_filepath"])
                    self.n = len(self.items)

            def __len__(self):
                return self.n

            def __getitem__(self, i):
                if self.items is not None:                                # manifest entries point to a saved feature dictionary
                    d = torch.load(self.items[i]["feature_filepath"], map_location="cpu")
                    return d["content_embs"], d["speaker_emb"], d["mel"], d.get("durations"), d.get("pitch")
                g = torch.Generator().manual_seed(1000 + i)
                N = int(torch.randint(6, 12, (1,), generator=g))
                dur = torch.randint(1, 4, (N,), generator=g)
                T = int(dur.sum())
                return (torch.randn(model.content_dim, N, generator=g), torch.randn(model.speaker_dim, generator=g), torch.randn(model.n_mel, T, generator=g), dur,
                        torch.rand(T, generator=g))

        def collate(batch):
            B, N, T = len(batch), max(b[0].shape[1] for b in batch), max(b[2].shape[1] for b in batch)
            ce, mel = torch.zeros(B, self.content_dim, N), torch.zeros(B, self.n_mel, T)
            dur, pitch = torch.zeros(B, N), torch.zeros(B, T)
            cl, ml = torch.zeros(B, dtype=torch.long), torch.zeros(B, dtype=torch.long)
            for k, (c_, s_, m_, d_, p_) in enumerate(batch):
                n, t = c_.shape[1], m_.shape[1]
                ce[k, :, :n], mel[k, :, :t], cl[k], ml[k] = c_, m_, n, t
                dur[k, :n] = d_ if d_ is not None else torch.ones(n)
                if p_ is not None:
                    pitch[k, :t] = p_[:t]
            return ce, cl, torch.stack([b[1] for b in batch]), mel, ml, dur, pitch

        return torch.utils.data.DataLoader(_DS(), batch_size=int(c.get("batch_size", 4)), shuffle=bool(c.get("shuffle", False)), collate_fn=collate,
                                           num_workers=int(c.get("num_workers", 0)))

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    # ------------------------------------------------------------------ model
    def forward(self, content_embs, content_lens, speaker_emb, durations=None, pitch=None, pace: float = 1.0):
        mask = torch.arange(content_embs.shape[2], device=content_embs.device)[None] < content_lens[:, None]
        x = self.content_proj(content_embs.transpose(1, 2)) + self.speaker_proj(speaker_emb).unsqueeze(1)
        enc = self.encoder(x, mask)["output"].float()
        log_dur = self.duration_predictor(enc, mask) if self.duration_predictor is not None else None
        if durations is None:
            durations = (torch.clamp(torch.exp(log_dur) - 1, min=0) if log_dur is not None else torch.ones_like(mask, dtype=torch.float)) * mask
        pitch_pred = pitch_tok = None
        if self.pitch_conditioning:
            pitch_pred = self.pitch_predictor(enc, mask)
            if pitch is not None:                                       # frame-level contour → mean per segment
                ends = torch.cumsum(durations.long(), 1)
                csum = F.pad(torch.cumsum(pitch, 1), (1, 0))
                T = pitch.shape[1]
                seg = csum.gather(1, ends.clamp(max=T)) - csum.gather(1, (ends - durations.long()).clamp(max=T))
                pitch_tok = seg / durations.clamp(min=1)
            else:
                pitch_tok = pitch_pred
            enc = enc + self.pitch_emb(pitch_tok.unsqueeze(1)).transpose(1, 2)
        frames, flen = regulate_len(durations, enc, pace)
        fmask = torch.arange(frames.shape[1], device=frames.device)[None] < flen[:, None]
        dec = self.decoder(frames, fmask)["output"].float()
        return {"mel": self.proj(dec).transpose(1, 2) * fmask.unsqueeze(1), "mel_len": flen, "log_dur": log_dur, "pitch_pred": pitch_pred, "pitch_tok": pitch_tok,
                "mask": mask, "dur": durations}

    def _losses(self, batch):
        ce, cl, spk, mel, ml, dur, pitch = batch
        o = self.forward(ce, cl, spk, durations=dur, pitch=pitch if self.pitch_conditioning else None)
        T = min(o["mel"].shape[2], mel.shape[2])
        fm = (torch.arange(T, device=mel.device)[None] < ml[:, None]).unsqueeze(1)
        mel_loss = ((o["mel"][..., :T] - mel[..., :T]) ** 2 * fm).sum() / (fm.sum() * self.n_mel).clamp(min=1)
        m = o["mask"]
        loss, logs = mel_loss, {"mel_loss": mel_loss.detach()}
        if o["log_dur"] is not None:
            dl = ((o["log_dur"] - torch.log(dur + 1)) ** 2 * m).sum() / m.sum()
            loss, logs["dur_loss"] = loss + self.w["dur"] * dl, dl.detach()
        if self.pitch_conditioning:
            pl = ((o["pitch_pred"] - o["pitch_tok"].detach()) ** 2 * m).sum() / m.sum()
            loss, logs["pitch_loss"] = loss + self.w["pitch"] * pl, pl.detach()
        return loss, logs

    def training_step(self, batch, batch_idx):
        loss, logs = self._losses(batch)
        self.log_dict({"train_loss": loss.detach(), **logs})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        with torch.no_grad():
            return {"val_loss": self._losses(batch)[0]}

    @torch.no_grad()
    def synthesize_spectrogram(self, content_embs, speaker_emb, content_lens=None, durations=None, pitch=None, pace: float = 1.0):
        self.eval()
        if content_lens is None:
            content_lens = torch.full((content_embs.shape[0],), content_embs.shape[2], dtype=torch.long, device=content_embs.device)
        o = self.forward(content_embs, content_lens, speaker_emb, durations, pitch, pace)
        return o["mel"], o["mel_len"]

    @torch.no_grad()
    def generate_wav(self, content_embs, speaker_emb, content_lens=None, durations=None, pitch=None, pace: float = 1.0):
        """Mel from content + speaker, then the vocoder: a list of waveforms cut to their lengths."""
        if self.vocoder is None:
            raise RuntimeError("generate_wav needs a vocoder: pass vocoder= to the constructor")
        voc = self.vocoder[0]
        mel, mel_len = self.synthesize_spectrogram(content_embs, speaker_emb, content_lens, durations, pitch, pace)
        wav = voc.convert_spectrogram_to_audio(mel)
        hop = wav.shape[-1] // max(mel.shape[-1], 1)
        return [w[: int(n) * hop] for w, n in zip(wav, mel_len)]

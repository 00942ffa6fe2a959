"""Self-supervised speech pre-training models.

* ``SpeechEncDecSelfSupervisedModel`` — encoder + one or several (decoder, loss) heads listed in ``cfg.loss_list``
  (contrastive with optional quantised targets, masked-token prediction, CTC/RNNT on pseudo-labels); the masks come from
  the spectrogram augmentation (``models/ssl_models.py:40-600`` of the reference).
* ``EncDecMaskedTokenPredModel`` — NEST: a frozen random-projection quantiser turns clean features into target tokens,
  random block masking hides spans of the input, the encoder + ``MultiSoftmaxDecoder`` predict the tokens at masked steps
  (``ssl_models.py:600-900``; ``modules/ssl_modules/{quantizers,masking,multi_softmax_decoder}.py``).
* ``EncDecDenoiseMaskedTokenPredModel`` — same, the input is a noisy copy while the targets come from the clean audio.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.module import NeuralModule
from ..data import audio_to_text as _data
from ..losses.misc import ContrastiveLoss, MLMLoss, MultiMLMLoss
from .asr_model import ASRModel, ASRModuleMixin


class RandomProjectionVectorQuantizer(NeuralModule):
    """BEST-RQ quantiser: frozen random projection + nearest entry of a frozen random codebook, per codebook."""

    def __init__(self, feat_in: int, code_dim: int = 16, num_classes: int = 8192, num_books: int = 1, dist_fn: str = "l2",
                 freeze: bool = True, squeeze_single: bool = False, combine_time_steps: int = 1, time_ahead: bool = False):
        super().__init__()
        self.num_books, self.num_classes, self.combine, self.squeeze_single = num_books, num_classes, combine_time_steps, squeeze_single
        self.proj = nn.Linear(feat_in * combine_time_steps, num_books * code_dim, bias=False)
        nn.init.xavier_normal_(self.proj.weight)
        self.codebooks = nn.Parameter(F.normalize(torch.randn(num_books, num_classes, code_dim), dim=-1))
        self.dist_fn = dist_fn
        if freeze:
            for p in self.parameters():
                p.requires_grad_(False)

    @torch.no_grad()
    def forward(self, input_signal: torch.Tensor):
        """[B, D, T] → (quantised [B, T', code_dim*H], tokens [B, T', H])."""
        x = input_signal.transpose(1, 2).float()
        B, T, D = x.shape
        T2 = T // self.combine
        x = x[:, : T2 * self.combine].reshape(B, T2, D * self.combine)
        z = self.proj(x).view(B, T2, self.num_books, -1)
        z = F.normalize(z, dim=-1)
        sim = torch.einsum("bthd,hcd->bthc", z, self.codebooks)
        ids = sim.argmax(-1)
        q = torch.stack([self.codebooks[h][ids[..., h]] for h in range(self.num_books)], dim=2).reshape(B, T2, -1)
        if self.squeeze_single and self.num_books == 1:
            ids = ids.squeeze(-1)
        return q, ids


class RandomBlockMasking(NeuralModule):
    """Hide ``mask_prob`` of the frames in blocks of ``block_size`` by overwriting them with a learnt / noise embedding."""

    def __init__(self, feat_in: int, mask_prob: float = 0.5, block_size: int = 48, mask_value: Optional[float] = None,
                 freeze: bool = True, allow_overlap: bool = False, max_mask_ratio: float = 0.8):
        super().__init__()
        self.block_size, self.mask_prob, self.max_mask_ratio = block_size, mask_prob, max_mask_ratio
        self.mask_embedding = nn.Parameter(torch.full((feat_in,), float(mask_value)) if mask_value is not None
                                           else torch.randn(feat_in) * 0.1)
        if freeze:
            self.mask_embedding.requires_grad_(False)

    def forward(self, input_feats: torch.Tensor, input_lengths: torch.Tensor):
        B, D, T = input_feats.shape
        masks = torch.zeros((B, D, T), device=input_feats.device, dtype=input_feats.dtype)
        out = input_feats.clone()
        for b in range(B):
            n = int(input_lengths[b])
            n_blocks = max(1, int(n * self.mask_prob / self.block_size))
            n_blocks = min(n_blocks, max(1, int(n * self.max_mask_ratio / self.block_size)))
            hi = max(1, n - self.block_size)
            starts = torch.randint(0, hi, (n_blocks,))
            for s in starts.tolist():
                e = min(n, s + self.block_size)
                out[b, :, s:e] = self.mask_embedding.view(-1, 1).to(out.dtype)
                masks[b, :, s:e] = 1.0
        return out, masks


class MultiSoftmaxDecoder(NeuralModule):
    """One linear head per codebook; log-probs [B, T, V, H] (or [B, T, V] for a single squeezed head)."""

    def __init__(self, feat_in: int, num_classes: int, num_decoders: int = 1, squeeze_single: bool = False, use_bias: bool = False):
        super().__init__()
        self.num_classes, self.num_decoders, self.squeeze_single = num_classes, num_decoders, squeeze_single
        self.decoder_layers = nn.Conv1d(feat_in, num_classes * num_decoders, 1, bias=use_bias)

    def forward(self, encoder_output: torch.Tensor):
        lg = self.decoder_layers(encoder_output).transpose(1, 2)
        B, T, _ = lg.shape
        lg = lg.view(B, T, self.num_classes, self.num_decoders)
        lp = torch.log_softmax(lg.float(), dim=2)
        return lp.squeeze(-1) if self.squeeze_single and self.num_decoders == 1 else lp


class _SSLBase(ASRModel, ASRModuleMixin):
    def _setup_dataloader_from_config(self, config):
        if config is None:
            return None
        ds = _data.build_speech_dataset(config, tokenizer=None, labels=list(cfg_get(config, "labels", None) or [" ", "a"]))
        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        return _data.get_dataloader_from_config(config, ds, rank, ws)

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "encoder"):
            return
        super()._setup_dataloaders_from_cfg()


class SpeechEncDecSelfSupervisedModel(_SSLBase):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        self.dropout_features = nn.Dropout(cfg.get("dropout_features", 0.0))
        self.dropout_features_q = nn.Dropout(cfg.get("dropout_features_q", 0.0))
        self.feat_pen_weight = cfg.get("feature_penalty", 0.0)
        self.decoder_losses = nn.ModuleDict()
        self.loss_alphas: Dict[str, float] = {}
        self.start_step: Dict[str, int] = {}
        if cfg.get("loss_list") is not None:
            for name, lc in cfg.loss_list.items():
                if not lc.get("is_active", True):
                    continue
                self.decoder_losses[name] = nn.ModuleDict({"decoder": from_config_dict(lc.decoder), "loss": from_config_dict(lc.loss)})
                self.loss_alphas[name] = lc.get("loss_alpha", 1.0)
                self.start_step[name] = lc.get("start_step", 0)
        else:
            self.decoder_ssl = from_config_dict(cfg.decoder)
            self.loss = from_config_dict(cfg.loss)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def forward(self, input_signal, input_signal_length):
        feats, flen = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        clean = feats.detach().clone()
        pen = feats.float().pow(2).mean() if self.feat_pen_weight else None
        masked = self.dropout_features(feats)
        if self.spec_augmentation is not None:
            masked = self.spec_augmentation(input_spec=masked, length=flen)
        # masked cells are the ones the augmentation zeroed (``ssl_models.py`` builds the mask from |x| < 1e-5 as well)
        masks = ((masked < 1e-5) & (masked > -1e-5)).to(feats.dtype)
        for b in range(masks.shape[0]):
            masks[b, :, int(flen[b]):] = 0.0
        enc, enc_len = self.encoder(audio_signal=masked, length=flen)[:2]
        return clean, masks, enc, enc_len, pen

    def _head_loss(self, dec, loss, clean, masks, enc, enc_len, targets=None, target_lens=None):
        out = dec(encoder_output=enc)
        if isinstance(loss, ContrastiveLoss):
            return loss(spectrograms=clean, spec_masks=masks, decoder_outputs=out, decoder_lengths=enc_len)
        if isinstance(loss, (MLMLoss, MultiMLMLoss)):
            return loss(decoder_outputs=out, targets=targets, decoder_lengths=enc_len, target_lengths=target_lens, masks=masks)
        return loss(log_probs=out, targets=targets, input_lengths=enc_len, target_lengths=target_lens)

    def training_step(self, batch, batch_idx):
        signal, signal_len, targets, target_lens = batch[:4]
        clean, masks, enc, enc_len, pen = self.forward(signal, signal_len)
        logs = {}
        if len(self.decoder_losses):
            total = enc.new_zeros((), dtype=torch.float32)
            for name, mod in self.decoder_losses.items():
                if self.global_step < self.start_step[name]:
                    continue
                l = self._head_loss(mod["decoder"], mod["loss"], clean, masks, enc, enc_len, targets, target_lens)
                logs[f"train_{name}_loss"] = l.detach()
                total = total + self.loss_alphas[name] * l
        else:
            total = self._head_loss(self.decoder_ssl, self.loss, clean, masks, enc, enc_len, targets, target_lens)
        if pen is not None:
            total = total + self.feat_pen_weight * pen
        logs["train_loss"] = total.detach()
        self.log_dict(logs)
        return {"loss": total}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len, targets, target_lens = batch[:4]
        clean, masks, enc, enc_len, _ = self.forward(signal, signal_len)
        if len(self.decoder_losses):
            total = sum(self.loss_alphas[n] * self._head_loss(m["decoder"], m["loss"], clean, masks, enc, enc_len, targets, target_lens)
                        for n, m in self.decoder_losses.items())
        else:
            total = self._head_loss(self.decoder_ssl, self.loss, clean, masks, enc, enc_len, targets, target_lens)
        return {"val_loss": total}


class EncDecMaskedTokenPredModel(_SSLBase):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.quantizer = from_config_dict(cfg.quantizer)
        self.mask_processor = from_config_dict(cfg.masking)
        self.encoder = from_config_dict(cfg.encoder)
        self.decoder = from_config_dict(cfg.decoder)
        self.loss = from_config_dict(cfg.loss)
        self.pre_encoder_mask = cfg.get("mask_position", "pre_conv") == "post_conv"
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def forward(self, input_signal, input_signal_length, noisy_input_signal=None, noisy_input_signal_length=None,
                apply_mask: bool = True):
        feats, flen = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        _, tokens = self.quantizer(input_signal=feats)
        src = feats
        if noisy_input_signal is not None:
            src, flen = self.preprocessor(input_signal=noisy_input_signal, length=noisy_input_signal_length)
        if apply_mask:
            masked, masks = self.mask_processor(input_feats=src, input_lengths=flen)
        else:
            masked, masks = src, torch.zeros_like(src)
        enc, enc_len = self.encoder(audio_signal=masked, length=flen)[:2]
        log_probs = self.decoder(encoder_output=enc)
        return log_probs, enc_len, masks, tokens

    def _loss(self, batch, apply_mask=True):
        signal, signal_len = batch[0], batch[1]
        log_probs, enc_len, masks, tokens = self.forward(signal, signal_len, apply_mask=apply_mask)
        return self.loss(masks=masks, decoder_outputs=log_probs, targets=tokens, decoder_lengths=enc_len)

    def training_step(self, batch, batch_idx):
        loss = self._loss(batch)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        return {"val_loss": self._loss(batch)}


class EncDecDenoiseMaskedTokenPredModel(EncDecMaskedTokenPredModel):
    """Batches carry ``(clean, clean_len, noise, noise_len, noisy, noisy_len)``; plain 4-tuples get synthetic noise added."""

    def _loss(self, batch, apply_mask=True):
        if len(batch) >= 6:
            clean, clean_len, _, _, noisy, noisy_len = batch[:6]
        else:
            clean, clean_len = batch[0], batch[1]
            snr = cfg_get(self._cfg, "train_snr_db", 10.0)
            noise = torch.randn_like(clean) * clean.std(dim=1, keepdim=True) * (10 ** (-snr / 20.0))
            noisy, noisy_len = clean + noise, clean_len
        log_probs, enc_len, masks, tokens = self.forward(clean, clean_len, noisy, noisy_len, apply_mask=apply_mask)
        return self.loss(masks=masks, decoder_outputs=log_probs, targets=tokens, decoder_lengths=enc_len)

"""Hybrid transducer + CTC models: one encoder, an RNNT/TDT branch and an auxiliary CTC head.

``loss = (1 - w) * rnnt_loss + w * ctc_loss`` with ``w = aux_ctc.ctc_loss_weight``; ``cur_decoder`` selects which
branch ``transcribe`` / validation WER use (reference:
``nemo/collections/asr/models/hybrid_rnnt_ctc_models.py:37-520``, ``hybrid_rnnt_ctc_bpe_models.py``).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict, to_container
from ..core.instantiate import from_config_dict
from ..decoding.ctc_decoding import CTCBPEDecoding, CTCDecoding, CTCDecodingConfig
from ..losses.ctc import CTCLoss
from ..utils.metrics import WER
from .asr_model import ASRBPEMixin, InterCTCMixin
from .ctc_models import prepare_bpe_model_cfg
from .rnnt_models import EncDecRNNTModel
from ..decoding.rnnt_decoding import RNNTBPEDecoding


class EncDecHybridRNNTCTCModel(EncDecRNNTModel, InterCTCMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        if isinstance(cfg, dict):
            cfg = OmegaConf.create(cfg)
        if "aux_ctc" not in cfg:
            raise ValueError("The config need to have a section for the CTC decoder named as aux_ctc for Hybrid models.")
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        with open_dict(cfg):
            if "feat_in" not in cfg.aux_ctc.decoder or not cfg.aux_ctc.decoder.get("feat_in"):
                cfg.aux_ctc.decoder.feat_in = self.encoder._feat_out
            self._fill_ctc_vocab(cfg)
        self.ctc_decoder = from_config_dict(cfg.aux_ctc.decoder)
        self.ctc_loss_weight = cfg.aux_ctc.get("ctc_loss_weight", 0.5)
        self.ctc_loss = CTCLoss(num_classes=self.ctc_decoder.num_classes_with_blank - 1, zero_infinity=True,
                                reduction=cfg.aux_ctc.get("ctc_reduction", "mean_batch"))
        self._setup_ctc_decoding()
        self.ctc_wer = WER(decoding=self.ctc_decoding, use_cer=cfg.aux_ctc.get("use_cer", False),
                           log_prediction=cfg.get("log_prediction", False))
        self.cur_decoder = "rnnt"
        self.setup_interctc(decoder_name="ctc_decoder", loss_name="ctc_loss", wer_name="ctc_wer")
        if not self._is_model_being_restored and self._train_dl is None:
            self._hybrid_ready = True
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "ctc_decoder"):
            return
        super()._setup_dataloaders_from_cfg()

    def _fill_ctc_vocab(self, cfg):
        if cfg.aux_ctc.decoder.get("num_classes", -1) < 1 and cfg.get("labels") is not None:
            cfg.aux_ctc.decoder.vocabulary = list(cfg.labels)
            cfg.aux_ctc.decoder.num_classes = len(cfg.labels)

    def _setup_ctc_decoding(self):
        dcfg = self._cfg.aux_ctc.get("decoding", None)
        if dcfg is None:
            dcfg = OmegaConf.structured(CTCDecodingConfig)
            with open_dict(self._cfg):
                self._cfg.aux_ctc.decoding = dcfg
        self.ctc_decoding = CTCDecoding(dcfg, vocabulary=list(self.ctc_decoder.vocabulary))

    def change_decoding_strategy(self, decoding_cfg: DictConfig = None, decoder_type: str = None, verbose: bool = True):
        if decoder_type is None or decoder_type == "rnnt":
            self.cur_decoder = "rnnt"
            return super().change_decoding_strategy(decoding_cfg, verbose)
        if decoder_type != "ctc":
            raise ValueError(f"decoder_type={decoder_type} is not supported. Supported values: [ctc,rnnt]")
        if decoding_cfg is not None:
            with open_dict(self._cfg):
                self._cfg.aux_ctc.decoding = OmegaConf.merge(OmegaConf.structured(CTCDecodingConfig), decoding_cfg)
        self._setup_ctc_decoding()
        self.ctc_wer = WER(decoding=self.ctc_decoding, use_cer=self.ctc_wer.use_cer, log_prediction=self.ctc_wer.log_prediction)
        self.cur_decoder = "ctc"

    def training_step(self, batch, batch_idx):
        from ..core.module import AccessMixin

        if self.is_interctc_enabled():
            AccessMixin.set_access_enabled(True, self.model_guid)
        signal, signal_len, transcript, transcript_len = batch[:4]
        encoded, encoded_len, decoder, target_length = self._encode_and_predict(signal, signal_len, transcript, transcript_len)
        n = getattr(self._trainer, "log_every_n_steps", 1) if self._trainer is not None else 1
        compute_wer = cfg_get(self._cfg, "compute_train_wer", True) and (batch_idx + 1) % max(1, n) == 0
        logs: Dict[str, Any] = {}
        if not self.joint.fuse_loss_wer:
            joint = self.joint(encoder_outputs=encoded, decoder_outputs=decoder)
            loss_value = self.loss(log_probs=joint, targets=transcript, input_lengths=encoded_len, target_lengths=target_length)
            if compute_wer:
                self.wer.update(predictions=encoded, predictions_lengths=encoded_len, targets=transcript,
                                targets_lengths=transcript_len)
                logs["training_batch_wer"], _, _ = self.wer.compute()
                self.wer.reset()
        else:
            loss_value, wer, _, _ = self.joint(encoder_outputs=encoded, decoder_outputs=decoder, encoder_lengths=encoded_len,
                                               transcripts=transcript, transcript_lengths=transcript_len, compute_wer=compute_wer)
            if compute_wer:
                logs["training_batch_wer"] = wer
        loss_value = self.add_auxiliary_losses(loss_value)
        if self.ctc_loss_weight > 0:
            log_probs = self.ctc_decoder(encoder_output=encoded)
            ctc_loss = self.ctc_loss(log_probs=log_probs, targets=transcript, input_lengths=encoded_len,
                                     target_lengths=transcript_len)
            logs["train_rnnt_loss"] = loss_value.detach()
            logs["train_ctc_loss"] = ctc_loss.detach()
            loss_value = (1 - self.ctc_loss_weight) * loss_value + self.ctc_loss_weight * ctc_loss
            if compute_wer:
                self.ctc_wer.update(predictions=log_probs.detach(), targets=transcript, targets_lengths=transcript_len,
                                    predictions_lengths=encoded_len)
                logs["training_batch_wer_ctc"], _, _ = self.ctc_wer.compute()
                self.ctc_wer.reset()
        loss_value, extra = self.add_interctc_losses(loss_value, transcript, transcript_len)
        logs.update(extra)
        logs.update({"train_loss": loss_value.detach(), "global_step": float(self.global_step)})
        self.log_dict(logs)
        return {"loss": loss_value}

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len, transcript, transcript_len = batch[:4]
        out = super().validation_pass(batch, batch_idx, dataloader_idx)
        encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
        log_probs = self.ctc_decoder(encoder_output=encoded)
        if self.compute_eval_loss:
            ctc_loss = self.ctc_loss(log_probs=log_probs, targets=transcript, input_lengths=encoded_len,
                                     target_lengths=transcript_len)
            out["val_ctc_loss"] = ctc_loss
            if "val_loss" in out:
                out["val_rnnt_loss"] = out["val_loss"]
                out["val_loss"] = (1 - self.ctc_loss_weight) * out["val_loss"] + self.ctc_loss_weight * ctc_loss
        self.ctc_wer.update(predictions=log_probs, targets=transcript, targets_lengths=transcript_len,
                            predictions_lengths=encoded_len)
        w, n, d = self.ctc_wer.compute()
        self.ctc_wer.reset()
        out.update({"val_wer_num_ctc": n, "val_wer_denom_ctc": d, "val_wer_ctc": w})
        return out

    def _transcribe_forward_and_decode(self, audio, lens, cfg):
        if self.cur_decoder == "rnnt":
            return super()._transcribe_forward_and_decode(audio, lens, cfg)
        cdt = torch.bfloat16 if audio.is_cuda else None
        with ops.compute_dtype(cdt):
            encoded, encoded_len = self.forward(input_signal=audio, input_signal_length=lens)
            log_probs = self.ctc_decoder(encoder_output=encoded)
        return self.ctc_decoding.ctc_decoder_predictions_tensor(log_probs.float(), encoded_len, return_hypotheses=True)


class EncDecHybridRNNTCTCBPEModel(EncDecHybridRNNTCTCModel, ASRBPEMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        cfg = prepare_bpe_model_cfg(self, cfg)
        vocab_size = self.tokenizer.vocab_size
        with open_dict(cfg):
            cfg.labels = None
            cfg.decoder.vocab_size = vocab_size
            cfg.joint.num_classes = vocab_size
            cfg.joint.vocabulary = None
            cfg.aux_ctc.decoder.num_classes = vocab_size
            cfg.aux_ctc.decoder.vocabulary = None
        super().__init__(cfg=cfg, trainer=trainer)

    def _setup_decoding(self):
        self.decoding = RNNTBPEDecoding(self._decoding_cfg(), decoder=self.decoder, joint=self.joint, tokenizer=self.tokenizer)

    def _setup_ctc_decoding(self):
        dcfg = self._cfg.aux_ctc.get("decoding", None)
        if dcfg is None:
            dcfg = OmegaConf.structured(CTCDecodingConfig)
            with open_dict(self._cfg):
                self._cfg.aux_ctc.decoding = dcfg
        self.ctc_decoding = CTCBPEDecoding(dcfg, tokenizer=self.tokenizer)

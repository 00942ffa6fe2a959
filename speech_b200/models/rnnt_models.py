"""Transducer ASR models (RNNT, TDT, multi-blank).

``EncDecRNNTModel`` / ``EncDecRNNTBPEModel``: ``forward()`` runs preprocessor + SpecAugment + encoder only
(reference: ``nemo/collections/asr/models/rnnt_models.py:667-717``); ``training_step`` runs the prediction net
and the joint, fused with the loss when ``joint.fuse_loss_wer`` is set (``:720-816``).  A ``loss.loss_name`` of
``tdt`` adds ``len(durations)`` extra joint outputs and copies the durations into the decoding config
(``:230-238``).  On GPUs the prediction network runs on a side stream concurrently with the encoder — the two
are independent until the joint.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict, to_container
from ..core.instantiate import from_config_dict
from ..decoding.rnnt_decoding import RNNTBPEDecoding, RNNTDecoding, RNNTDecodingConfig
from ..losses.rnnt import RNNTLoss
from ..utils.metrics import WER
from .asr_model import ASRBPEMixin, ASRModel, ASRModuleMixin, TranscriptionMixin
from .ctc_models import prepare_bpe_model_cfg


class EncDecRNNTModel(ASRModel, ASRModuleMixin, TranscriptionMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        with open_dict(cfg):
            labels = cfg.get("labels", None)
            if labels is not None:
                cfg.decoder.vocab_size = len(labels)
                cfg.joint.num_classes = len(labels)
                cfg.joint.vocabulary = list(labels)
            cfg.joint.jointnet.encoder_hidden = cfg.get("model_defaults", {}).get("enc_hidden", None) or \
                cfg.joint.jointnet.get("encoder_hidden", None) or self.encoder._feat_out
            cfg.joint.jointnet.pred_hidden = cfg.get("model_defaults", {}).get("pred_hidden", None) or \
                cfg.joint.jointnet.get("pred_hidden", None) or cfg.decoder.prednet.pred_hidden
        loss_name, loss_kwargs = self.extract_rnnt_loss_cfg(cfg.get("loss", None))
        num_classes = cfg.joint.num_classes
        if loss_name == "tdt":
            with open_dict(cfg):
                cfg.joint.num_extra_outputs = len(loss_kwargs["durations"])
        elif loss_name == "multiblank_rnnt":
            with open_dict(cfg):
                cfg.joint.num_extra_outputs = len(loss_kwargs["big_blank_durations"])
        self.decoder = from_config_dict(cfg.decoder)
        self.joint = from_config_dict(cfg.joint)
        self.loss = RNNTLoss(num_classes=self.joint.num_classes_with_blank - 1 - self.joint.num_extra_outputs
                             if loss_name != "multiblank_rnnt" else self.joint.num_classes_with_blank - 1,
                             loss_name=loss_name, loss_kwargs=loss_kwargs, reduction=cfg.get("rnnt_reduction", "mean_batch"))
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        self.cfg_loss_name, self.cfg_loss_kwargs = loss_name, loss_kwargs
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, batch_dim_index=0, use_cer=cfg.get("use_cer", False),
                       log_prediction=cfg.get("log_prediction", False), dist_sync_on_step=True)
        if self.joint.fuse_loss_wer:
            self.joint.set_loss(self.loss)
            self.joint.set_wer(self.wer)
        self.compute_eval_loss = cfg.get("compute_eval_loss", True)
        self._side_stream = None
        for m in self.modules():
            if not hasattr(m, "model_guid"):
                try:
                    m.model_guid = self.model_guid
                except Exception:
                    pass
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "joint"):
            return
        super()._setup_dataloaders_from_cfg()

    @staticmethod
    def extract_rnnt_loss_cfg(cfg):
        if cfg is None:
            return "default", {}
        name = cfg.get("loss_name", "default")
        if name == "default":
            return name, {}
        kw = cfg.get(f"{name}_kwargs", None)
        return name, (to_container(kw, resolve=True) if isinstance(kw, DictConfig) else dict(kw or {}))

    def _decoding_cfg(self):
        dcfg = self._cfg.get("decoding", None)
        base = OmegaConf.structured(RNNTDecodingConfig)
        dcfg = OmegaConf.merge(base, dcfg) if dcfg is not None else base
        with open_dict(dcfg):
            if self.cfg_loss_name == "tdt":
                dcfg.durations = list(self.cfg_loss_kwargs["durations"])
                dcfg.model_type = "tdt"
            elif self.cfg_loss_name == "multiblank_rnnt":
                dcfg.big_blank_durations = list(self.cfg_loss_kwargs["big_blank_durations"])
                dcfg.model_type = "multiblank"
        with open_dict(self._cfg):
            self._cfg.decoding = dcfg
        return dcfg

    def _setup_decoding(self):
        self.decoding = RNNTDecoding(self._decoding_cfg(), decoder=self.decoder, joint=self.joint,
                                     vocabulary=list(self.joint.vocabulary))

    def change_decoding_strategy(self, decoding_cfg: DictConfig = None, verbose: bool = True):
        if decoding_cfg is not None:
            with open_dict(self._cfg):
                self._cfg.decoding = decoding_cfg
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, use_cer=self.wer.use_cer, log_prediction=self.wer.log_prediction)
        if self.joint.fuse_loss_wer:
            self.joint.set_loss(self.loss)
            self.joint.set_wer(self.wer)

    # ------------------------------------------------------------------ forward
    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None):
        has_in = input_signal is not None and input_signal_length is not None
        has_proc = processed_signal is not None and processed_signal_length is not None
        if not (has_in ^ has_proc):
            raise ValueError(f"{self} Arguments ``input_signal`` and ``input_signal_length`` are mutually exclusive "
                             " with ``processed_signal`` and ``processed_signal_len`` arguments.")
        if not has_proc:
            processed_signal, processed_signal_length = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.spec_augmentation is not None and self.training:
            processed_signal = self.spec_augmentation(input_spec=processed_signal, length=processed_signal_length)
        encoded, encoded_len = self.encoder(audio_signal=processed_signal, length=processed_signal_length)[:2]
        return encoded, encoded_len

    def _encode_and_predict(self, signal, signal_len, transcript, transcript_len):
        """Encoder and prediction network; on GPUs the (small, latency-bound) prediction network is issued on a
        side stream so that it overlaps the encoder."""
        if signal.is_cuda and not torch.cuda.is_current_stream_capturing() and not ops.eager_allowed():
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=signal.device)
            main = torch.cuda.current_stream(signal.device)
            self._side_stream.wait_stream(main)
            with torch.cuda.stream(self._side_stream):
                decoder, target_length, states = self.decoder(targets=transcript, target_length=transcript_len)
            encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
            main.wait_stream(self._side_stream)
            decoder.record_stream(main)
        else:
            encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
            decoder, target_length, states = self.decoder(targets=transcript, target_length=transcript_len)
        return encoded, encoded_len, decoder, target_length

    def training_step(self, batch, batch_idx):
        signal, signal_len, transcript, transcript_len = batch[:4]
        encoded, encoded_len, decoder, target_length = self._encode_and_predict(signal, signal_len, transcript, transcript_len)
        n = getattr(self._trainer, "log_every_n_steps", 1) if self._trainer is not None else 1
        compute_wer = cfg_get(self._cfg, "compute_train_wer", True) and (batch_idx + 1) % max(1, n) == 0
        logs: Dict[str, Any] = {}
        if not self.joint.fuse_loss_wer:
            joint = self.joint(encoder_outputs=encoded, decoder_outputs=decoder)
            loss_value = self.loss(log_probs=joint, targets=transcript, input_lengths=encoded_len, target_lengths=target_length)
            loss_value = self.add_auxiliary_losses(loss_value)
            if compute_wer:
                self.wer.update(predictions=encoded, predictions_lengths=encoded_len, targets=transcript,
                                targets_lengths=transcript_len)
                wer, _, _ = self.wer.compute()
                self.wer.reset()
                logs["training_batch_wer"] = wer
        else:
            loss_value, wer, _, _ = self.joint(encoder_outputs=encoded, decoder_outputs=decoder, encoder_lengths=encoded_len,
                                               transcripts=transcript, transcript_lengths=transcript_len,
                                               compute_wer=compute_wer)
            loss_value = self.add_auxiliary_losses(loss_value)
            if compute_wer:
                logs["training_batch_wer"] = wer
        logs.update({"train_loss": loss_value.detach(), "global_step": float(self.global_step)})
        self.log_dict(logs)
        return {"loss": loss_value}

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len, transcript, transcript_len = batch[:4]
        encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
        out = {}
        if not self.joint.fuse_loss_wer:
            if self.compute_eval_loss:
                decoder, target_length, _ = self.decoder(targets=transcript, target_length=transcript_len)
                joint = self.joint(encoder_outputs=encoded, decoder_outputs=decoder)
                out["val_loss"] = self.loss(log_probs=joint, targets=transcript, input_lengths=encoded_len,
                                            target_lengths=target_length)
            self.wer.update(predictions=encoded, predictions_lengths=encoded_len, targets=transcript,
                            targets_lengths=transcript_len)
            wer, num, den = self.wer.compute()
            self.wer.reset()
        else:
            decoder = None
            if self.compute_eval_loss:
                decoder, target_length, _ = self.decoder(targets=transcript, target_length=transcript_len)
            loss_value, wer, num, den = self.joint(encoder_outputs=encoded, decoder_outputs=decoder, encoder_lengths=encoded_len,
                                                   transcripts=transcript, transcript_lengths=transcript_len, compute_wer=True)
            if loss_value is not None:
                out["val_loss"] = loss_value
        out.update({"val_wer_num": num, "val_wer_denom": den, "val_wer": wer})
        return out

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx)

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        out = self.validation_pass(batch, batch_idx, dataloader_idx)
        return {k.replace("val_", "test_"): v for k, v in out.items()}

    def predict_step(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len = batch[0], batch[1]
        sample_id = batch[4] if len(batch) > 4 else torch.arange(signal.shape[0])
        encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
        hyps = self.decoding.rnnt_decoder_predictions_tensor(encoder_output=encoded, encoded_lengths=encoded_len)
        return list(zip(sample_id.cpu().tolist(), hyps))

    def _transcribe_forward_and_decode(self, audio, lens, cfg):
        cdt = torch.bfloat16 if audio.is_cuda else None
        with ops.compute_dtype(cdt):
            encoded, encoded_len = self.forward(input_signal=audio, input_signal_length=lens)
        return self.decoding.rnnt_decoder_predictions_tensor(encoder_output=encoded.float(), encoded_lengths=encoded_len,
                                                             return_hypotheses=True)

    def change_vocabulary(self, new_vocabulary: List[str], decoding_cfg: Optional[DictConfig] = None):
        if list(self.joint.vocabulary) == list(new_vocabulary):
            return
        if not new_vocabulary:
            raise ValueError(f"New vocabulary must be non-empty list of chars. But I got: {new_vocabulary}")
        dev = self.device
        jc = to_container(self._cfg.joint, resolve=True)
        jc["vocabulary"], jc["num_classes"] = list(new_vocabulary), len(new_vocabulary)
        dc = to_container(self._cfg.decoder, resolve=True)
        dc["vocab_size"] = len(new_vocabulary)
        self.joint = from_config_dict(jc).to(dev)
        self.decoder = from_config_dict(dc).to(dev)
        with open_dict(self._cfg):
            self._cfg.joint, self._cfg.decoder = OmegaConf.create(jc), OmegaConf.create(dc)
            self._cfg.labels = list(new_vocabulary)
        self.loss = RNNTLoss(num_classes=len(new_vocabulary), loss_name=self.cfg_loss_name, loss_kwargs=self.cfg_loss_kwargs)
        self.change_decoding_strategy(decoding_cfg)


class EncDecRNNTBPEModel(EncDecRNNTModel, ASRBPEMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        cfg = prepare_bpe_model_cfg(self, cfg)
        vocab_size = self.tokenizer.vocab_size
        with open_dict(cfg):
            cfg.labels = None
            cfg.decoder.vocab_size = vocab_size
            cfg.joint.num_classes = vocab_size
            cfg.joint.vocabulary = None
        super().__init__(cfg=cfg, trainer=trainer)

    def _setup_decoding(self):
        self.decoding = RNNTBPEDecoding(self._decoding_cfg(), decoder=self.decoder, joint=self.joint,
                                        tokenizer=self.tokenizer)

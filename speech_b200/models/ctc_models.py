"""CTC encoder-decoder ASR models.

``EncDecCTCModel`` (character vocabulary from ``cfg.decoder.vocabulary``) and ``EncDecCTCModelBPE`` (sub-word
tokenizer): preprocessor -> SpecAugment -> encoder -> ``ConvASRDecoder`` -> CTC loss, with inter-CTC and WER
logging (reference: ``nemo/collections/asr/models/ctc_models.py:49-604``, ``ctc_bpe_models.py``).
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict, to_container
from ..core.instantiate import from_config_dict
from ..core.neural_types import AudioSignal, LabelsType, LengthsType, LogprobsType, NeuralType, SpectrogramType
from ..decoding.ctc_decoding import CTCBPEDecoding, CTCDecoding, CTCDecodingConfig
from ..losses.ctc import CTCLoss
from ..utils.metrics import WER
from .asr_model import ASRBPEMixin, ASRModel, ASRModuleMixin, InterCTCMixin, TranscriptionMixin


class EncDecCTCModel(ASRModel, ASRModuleMixin, InterCTCMixin, TranscriptionMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        with open_dict(cfg):
            if "feat_in" not in cfg.decoder or (not cfg.decoder.feat_in and hasattr(self.encoder, "_feat_out")):
                cfg.decoder.feat_in = self.encoder._feat_out
            if not cfg.decoder.get("feat_in"):
                raise ValueError("param feat_in of the decoder's config is not set!")
            if cfg.decoder.get("num_classes", -1) < 1 and cfg.decoder.get("vocabulary") is not None:
                cfg.decoder["num_classes"] = len(cfg.decoder.vocabulary)
        self.decoder = from_config_dict(cfg.decoder)
        self.loss = CTCLoss(num_classes=self.decoder.num_classes_with_blank - 1, zero_infinity=True,
                            reduction=cfg.get("ctc_reduction", "mean_batch"))
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, use_cer=cfg.get("use_cer", False), dist_sync_on_step=True,
                       log_prediction=cfg.get("log_prediction", False))
        self.setup_interctc(decoder_name="decoder", loss_name="loss", wer_name="wer")
        for m in self.modules():
            if hasattr(m, "model_guid") is False:
                try:
                    m.model_guid = self.model_guid
                except Exception:
                    pass
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "decoder"):
            return  # called from the base constructor before modules exist; repeated at the end of __init__
        super()._setup_dataloaders_from_cfg()

    def _setup_decoding(self):
        dcfg = self._cfg.get("decoding", None)
        if dcfg is None:
            dcfg = OmegaConf.structured(CTCDecodingConfig)
            with open_dict(self._cfg):
                self._cfg.decoding = dcfg
        self.decoding = CTCDecoding(dcfg, vocabulary=list(self.decoder.vocabulary))

    def change_decoding_strategy(self, decoding_cfg: DictConfig = None, verbose: bool = True):
        if decoding_cfg is None:
            decoding_cfg = self._cfg.decoding
        merged = OmegaConf.merge(OmegaConf.structured(CTCDecodingConfig), decoding_cfg)
        with open_dict(self._cfg):
            self._cfg.decoding = merged
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, use_cer=self.wer.use_cer, log_prediction=self.wer.log_prediction)

    def change_vocabulary(self, new_vocabulary: List[str], decoding_cfg: Optional[DictConfig] = None):
        if self.decoder.vocabulary == list(new_vocabulary):
            return
        if not new_vocabulary:
            raise ValueError(f"New vocabulary must be non-empty list of chars. But I got: {new_vocabulary}")
        dc = copy.deepcopy(to_container(self._cfg.decoder, resolve=True))
        dc["vocabulary"], dc["num_classes"] = list(new_vocabulary), len(new_vocabulary)
        dev = self.device
        self.decoder = from_config_dict(dc).to(dev)
        self.loss = CTCLoss(num_classes=self.decoder.num_classes_with_blank - 1, zero_infinity=True,
                            reduction=self._cfg.get("ctc_reduction", "mean_batch"))
        with open_dict(self._cfg):
            self._cfg.decoder = OmegaConf.create(dc)
            if decoding_cfg is not None:
                self._cfg.decoding = decoding_cfg
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, use_cer=self.wer.use_cer, log_prediction=self.wer.log_prediction)

    @property
    def input_types(self):
        return {"input_signal": NeuralType(("B", "T"), AudioSignal(), optional=True),
                "input_signal_length": NeuralType(("B",), LengthsType(), optional=True),
                "processed_signal": NeuralType(("B", "D", "T"), SpectrogramType(), optional=True),
                "processed_signal_length": NeuralType(("B",), LengthsType(), optional=True)}

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
        log_probs = self.decoder(encoder_output=encoded)
        greedy = log_probs.argmax(dim=-1, keepdim=False)
        return log_probs, encoded_len, greedy

    def training_step(self, batch, batch_idx):
        if self.is_interctc_enabled():
            from ..core.module import AccessMixin

            AccessMixin.set_access_enabled(True, self.model_guid)
        signal, signal_len, transcript, transcript_len = batch[:4]
        log_probs, encoded_len, predictions = self.forward(input_signal=signal, input_signal_length=signal_len)
        loss = self.loss(log_probs=log_probs, targets=transcript, input_lengths=encoded_len, target_lengths=transcript_len)
        loss = self.add_auxiliary_losses(loss)
        loss, extra = self.add_interctc_losses(loss, transcript, transcript_len)
        logs = {"train_loss": loss.detach(), "global_step": float(self.global_step), **extra}
        n = getattr(self._trainer, "log_every_n_steps", 1) if self._trainer is not None else 1
        if cfg_get(self._cfg, "compute_train_wer", True) and (batch_idx + 1) % max(1, n) == 0:
            self.wer.update(predictions=log_probs.detach(), targets=transcript, targets_lengths=transcript_len,
                            predictions_lengths=encoded_len)
            wer, _, _ = self.wer.compute()
            self.wer.reset()
            logs["training_batch_wer"] = wer
        self.log_dict(logs)
        return {"loss": loss}

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len, transcript, transcript_len = batch[:4]
        log_probs, encoded_len, predictions = self.forward(input_signal=signal, input_signal_length=signal_len)
        loss = self.loss(log_probs=log_probs, targets=transcript, input_lengths=encoded_len, target_lengths=transcript_len)
        self.wer.update(predictions=log_probs, targets=transcript, targets_lengths=transcript_len,
                        predictions_lengths=encoded_len)
        wer, num, den = self.wer.compute()
        self.wer.reset()
        return {"val_loss": loss, "val_wer_num": num, "val_wer_denom": den, "val_wer": wer}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx)

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        out = self.validation_pass(batch, batch_idx, dataloader_idx)
        return {k.replace("val_", "test_"): v for k, v in out.items()}

    def predict_step(self, batch, batch_idx, dataloader_idx=0):
        signal, signal_len = batch[0], batch[1]
        sample_id = batch[4] if len(batch) > 4 else torch.arange(signal.shape[0])
        log_probs, encoded_len, _ = self.forward(input_signal=signal, input_signal_length=signal_len)
        hyps = self.decoding.ctc_decoder_predictions_tensor(log_probs, encoded_len)
        return list(zip(sample_id.cpu().tolist(), hyps))

    def _transcribe_forward_and_decode(self, audio, lens, cfg):
        from ..core.trainer import Trainer

        cdt = torch.bfloat16 if audio.is_cuda else None
        with ops.compute_dtype(cdt):
            log_probs, encoded_len, _ = self.forward(input_signal=audio, input_signal_length=lens)
        return self.decoding.ctc_decoder_predictions_tensor(log_probs.float(), encoded_len, return_hypotheses=True)


class EncDecCTCModelBPE(EncDecCTCModel, ASRBPEMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        cfg = prepare_bpe_model_cfg(self, cfg)
        vocab_size = self.tokenizer.vocab_size
        with open_dict(cfg):
            cfg.decoder["num_classes"] = vocab_size
            cfg.decoder["vocabulary"] = None
        super().__init__(cfg=cfg, trainer=trainer)

    def _setup_decoding(self):
        dcfg = self._cfg.get("decoding", None)
        if dcfg is None:
            dcfg = OmegaConf.structured(CTCDecodingConfig)
            with open_dict(self._cfg):
                self._cfg.decoding = dcfg
        self.decoding = CTCBPEDecoding(dcfg, tokenizer=self.tokenizer)


def prepare_bpe_model_cfg(model, cfg) -> DictConfig:
    """Tokenizer set-up has to precede module construction (the heads need the vocabulary size), so the pieces
    of ``ModelPT`` state that artifact registration touches are created here, before ``ModelPT.__init__`` runs."""
    cfg = OmegaConf.create(cfg) if isinstance(cfg, dict) else copy.deepcopy(cfg)
    OmegaConf.set_struct(cfg, False)
    if "tokenizer" not in cfg:
        raise ValueError("`cfg` must have `tokenizer` config to create a tokenizer !")
    object.__setattr__(model, "_cfg", cfg)
    object.__setattr__(model, "artifacts", {})
    from ..core.modelpt import ModelPT

    object.__setattr__(model, "_restore_folder", ModelPT._nemo_file_folder if ModelPT._is_model_being_restored else None)
    model._setup_tokenizer(cfg.tokenizer)
    return cfg

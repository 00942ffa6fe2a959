"""Speech classification models: utterance-level (commands, language id), frame-level (VAD with MarbleNet) and
regression, plus the speaker-label model (TitaNet / ECAPA / SpeakerNet) with embedding extraction and verification.

Reference: ``models/classification_models.py`` (``EncDecClassificationModel``, ``EncDecRegressionModel``,
``EncDecFrameClassificationModel``) and ``models/label_models.py`` (``EncDecSpeakerLabelModel``).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np
import torch
import torch.nn.functional as F

from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.modelpt import ModelPT
from ..data import audio_to_label as _ldata
from ..data.audio_to_text import get_dataloader_from_config, load_audio
from ..losses.cross_entropy import CrossEntropyLoss
from ..losses.misc import AngularSoftmaxLoss


def topk_accuracy(logits: torch.Tensor, labels: torch.Tensor, ks=(1,)) -> List[float]:
    maxk = min(max(ks), logits.shape[-1])
    pred = logits.topk(maxk, dim=-1).indices
    hit = pred == labels.view(-1, 1)
    return [float(hit[:, : min(k, maxk)].any(dim=1).float().mean()) for k in ks]


class _EncDecLabelBase(ModelPT):
    frame_level = False

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        with open_dict(cfg):
            if not cfg.decoder.get("feat_in"):
                cfg.decoder.feat_in = self.encoder._feat_out
            if cfg.get("labels") is not None and (cfg.decoder.get("num_classes", -1) or -1) < 1:
                cfg.decoder.num_classes = len(cfg.labels)
        self.decoder = from_config_dict(cfg.decoder)
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        self.crop_or_pad = from_config_dict(cfg.crop_or_pad_augment) if cfg.get("crop_or_pad_augment") is not None else None
        self.loss = self._make_loss()
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "decoder"):
            return
        super()._setup_dataloaders_from_cfg()

    def _make_loss(self):
        return CrossEntropyLoss()

    # ------------------------------------------------------------------ data
    def _loader(self, config):
        if config is None:
            return None
        ds = _ldata.build_label_dataset(config, frame_level=self.frame_level)
        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        return get_dataloader_from_config(config, ds, rank, ws)

    def setup_training_data(self, train_data_config):
        self._train_dl = self._loader(train_data_config)

    def setup_validation_data(self, val_data_config):
        self._validation_dl = self._loader(val_data_config)

    def setup_test_data(self, test_data_config):
        self._test_dl = self._loader(test_data_config)

    # ------------------------------------------------------------------ forward
    def encode(self, input_signal, input_signal_length):
        feats, flen = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.crop_or_pad is not None:
            feats, flen = self.crop_or_pad(input_signal=feats, length=flen)
        if self.spec_augmentation is not None and self.training:
            feats = self.spec_augmentation(input_spec=feats, length=flen)
        return self.encoder(audio_signal=feats, length=flen)[:2]

    def forward(self, input_signal, input_signal_length):
        enc, enc_len = self.encode(input_signal, input_signal_length)
        return self.decoder(encoder_output=enc, length=enc_len) if self._decoder_takes_length() else self.decoder(encoder_output=enc)

    def _decoder_takes_length(self) -> bool:
        import inspect

        return "length" in inspect.signature(self.decoder.forward).parameters

    def _loss_and_logits(self, batch):
        audio, alen, labels, llen = batch[:4]
        out = self.forward(input_signal=audio, input_signal_length=alen)
        logits = out[0] if isinstance(out, tuple) else out
        return self.loss(logits=logits, labels=labels), logits, labels

    def training_step(self, batch, batch_idx):
        loss, logits, labels = self._loss_and_logits(batch)
        acc = topk_accuracy(logits.detach().reshape(-1, logits.shape[-1]), labels.reshape(-1))[0]
        self.log_dict({"train_loss": loss.detach(), "training_batch_accuracy_top_1": acc})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        loss, logits, labels = self._loss_and_logits(batch)
        pred = logits.reshape(-1, logits.shape[-1]).argmax(-1)
        return {"val_loss": loss, "val_correct": (pred == labels.reshape(-1)).sum(), "val_total": torch.tensor(labels.numel())}

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        return {k.replace("val_", "test_"): v for k, v in self.validation_step(batch, batch_idx, dataloader_idx).items()}

    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0):
        if not outputs:
            return {}
        loss = torch.stack([o["val_loss"] for o in outputs]).mean()
        acc = sum(int(o["val_correct"]) for o in outputs) / max(1, sum(int(o["val_total"]) for o in outputs))
        return {"val_loss": loss, "log": {"val_loss": loss, "val_epoch_top@1": acc}}

    def multi_test_epoch_end(self, outputs, dataloader_idx: int = 0):
        if not outputs:
            return {}
        loss = torch.stack([o["test_loss"] for o in outputs]).mean()
        acc = sum(int(o["test_correct"]) for o in outputs) / max(1, sum(int(o["test_total"]) for o in outputs))
        return {"test_loss": loss, "log": {"test_loss": loss, "test_epoch_top@1": acc}}


class EncDecClassificationModel(_EncDecLabelBase):
    """Utterance-level classification (``classification_models.py`` ``EncDecClassificationModel``)."""

    @torch.no_grad()
    def transcribe(self, audio: Sequence[Union[str, np.ndarray, torch.Tensor]], batch_size: int = 4, logprobs: bool = False):
        self.eval()
        labels = list(cfg_get(self._cfg, "labels", None) or [])
        out = []
        sr = cfg_get(self._cfg, "sample_rate", 16000)
        for s in range(0, len(audio), batch_size):
            xs = [torch.as_tensor(load_audio(a, target_sr=sr) if isinstance(a, str) else a, dtype=torch.float32).reshape(-1)
                  for a in audio[s:s + batch_size]]
            lens = torch.tensor([x.numel() for x in xs])
            x = torch.nn.utils.rnn.pad_sequence(xs, batch_first=True).to(self.device)
            logits = self.forward(input_signal=x, input_signal_length=lens.to(self.device))
            if logprobs:
                out.extend(torch.log_softmax(logits.float(), -1).cpu())
            else:
                ids = logits.argmax(-1).cpu().tolist()
                out.extend(labels[i] if labels else i for i in ids)
        return out

    def change_labels(self, new_labels: List[str]):
        if not new_labels:
            raise ValueError("new_labels must be a non-empty list of labels")
        with open_dict(self._cfg):
            self._cfg.labels = list(new_labels)
            self._cfg.decoder.num_classes = len(new_labels)
        self.decoder = from_config_dict(self._cfg.decoder).to(self.device)


class EncDecRegressionModel(_EncDecLabelBase):
    def _make_loss(self):
        mse = torch.nn.MSELoss()
        return lambda logits, labels: mse(logits.view(-1).float(), labels.view(-1).float())

    def training_step(self, batch, batch_idx):
        loss, _, _ = self._loss_and_logits(batch)
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}


class EncDecFrameClassificationModel(_EncDecLabelBase):
    """Frame-level classification (VAD): the decoder emits one distribution per encoder frame; labels are resampled to
    the encoder's frame rate by nearest index (``classification_models.py`` ``EncDecFrameClassificationModel``)."""

    frame_level = True

    def forward(self, input_signal, input_signal_length):
        enc, enc_len = self.encode(input_signal, input_signal_length)
        logits = self.decoder(encoder_output=enc)       # [B, T, C] (ConvASRDecoder-style head without log-softmax reduce)
        return logits, enc_len

    def _loss_and_logits(self, batch):
        audio, alen, labels, llen = batch[:4]
        logits, enc_len = self.forward(input_signal=audio, input_signal_length=alen)
        B, T, C = logits.shape
        idx = (torch.arange(T, device=logits.device).float() * (labels.shape[1] / max(T, 1))).long().clamp(max=labels.shape[1] - 1)
        lab = labels.to(logits.device)[:, idx]
        mask = torch.arange(T, device=logits.device)[None] < enc_len[:, None]
        loss = F.cross_entropy(logits.float()[mask], lab[mask])
        return loss, logits[mask], lab[mask]


class EncDecSpeakerLabelModel(_EncDecLabelBase):
    """Speaker identification / verification model (``label_models.py:60-700``)."""

    def _make_loss(self):
        lcfg = cfg_get(self._cfg, "loss", None)
        if lcfg is not None and "_target_" in lcfg:
            return from_config_dict(lcfg)
        if cfg_get(self._cfg.decoder, "angular", False):
            return AngularSoftmaxLoss(scale=cfg_get(lcfg, "scale", 30.0) if lcfg else 30.0,
                                      margin=cfg_get(lcfg, "margin", 0.2) if lcfg else 0.2)
        return CrossEntropyLoss()

    def forward(self, input_signal, input_signal_length):
        enc, enc_len = self.encode(input_signal, input_signal_length)
        logits, embs = self.decoder(encoder_output=enc, length=enc_len)
        return logits, embs

    @torch.no_grad()
    def infer_segment(self, segment: Union[np.ndarray, torch.Tensor]):
        self.eval()
        x = torch.as_tensor(segment, dtype=torch.float32).reshape(1, -1).to(self.device)
        logits, emb = self.forward(input_signal=x, input_signal_length=torch.tensor([x.shape[1]], device=self.device))
        return emb, logits

    @torch.no_grad()
    def get_embedding(self, path_or_audio):
        x = load_audio(path_or_audio, target_sr=cfg_get(self._cfg, "sample_rate", 16000)) if isinstance(path_or_audio, str) \
            else path_or_audio
        return self.infer_segment(x)[0]

    @torch.no_grad()
    def get_label(self, path_or_audio):
        x = load_audio(path_or_audio, target_sr=cfg_get(self._cfg, "sample_rate", 16000)) if isinstance(path_or_audio, str) \
            else path_or_audio
        _, logits = self.infer_segment(x)
        i = int(logits.argmax(-1))
        labels = list(cfg_get(self._cfg, "labels", None) or [])
        return labels[i] if labels else i

    @torch.no_grad()
    def verify_speakers(self, a, b, threshold: float = 0.7) -> bool:
        ea, eb = self.get_embedding(a).squeeze(), self.get_embedding(b).squeeze()
        sim = float(F.cosine_similarity(ea, eb, dim=0))
        return (sim + 1) / 2 >= threshold

    @torch.no_grad()
    def batch_inference(self, audio: Sequence[Any], batch_size: int = 32):
        self.eval()
        embs, logits_all = [], []
        for s in range(0, len(audio), batch_size):
            xs = [torch.as_tensor(load_audio(a) if isinstance(a, str) else a, dtype=torch.float32).reshape(-1)
                  for a in audio[s:s + batch_size]]
            lens = torch.tensor([x.numel() for x in xs], device=self.device)
            x = torch.nn.utils.rnn.pad_sequence(xs, batch_first=True).to(self.device)
            lg, e = self.forward(input_signal=x, input_signal_length=lens)
            embs.append(e.cpu())
            logits_all.append(lg.cpu())
        return torch.cat(embs), torch.cat(logits_all)

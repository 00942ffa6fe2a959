"""Attention encoder-decoder multitask model (Canary).

FastConformer encoder -> optional ``encoder_decoder_proj`` -> optional extra transformer encoder ->
``transf_decoder`` (``TransformerDecoderNM``) -> ``log_softmax`` (``TokenClassifier``, weight tied to the decoder's
token embedding) -> label-smoothed cross-entropy with an optional prompt loss-mask.  The decoder vocabulary is padded
to a multiple of 8.  Sub-module names follow ``nemo/collections/asr/models/aed_multitask_models.py:133-200,802-825``.
Batches are ``PromptedAudioToTextMiniBatch``-like tuples
``(audio, audio_lens, prompted_transcript, prompted_transcript_lens, prompt, prompt_lens)``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict, to_container
from ..core.instantiate import from_config_dict
from ..decoding.rnnt_decoding import Hypothesis
from ..losses.cross_entropy import SmoothedCrossEntropyLoss
from ..modules.transformer_nm import (BeamSearchSequenceGenerator, GreedySequenceGenerator, TokenClassifier,
                                      TransformerDecoderNM, TransformerEncoderNM)
from ..utils.metrics import WER
from .asr_model import ASRBPEMixin, ASRModel, ASRModuleMixin, TranscriptionMixin
from .ctc_models import prepare_bpe_model_cfg


@dataclass
class MultiTaskDecodingConfig:
    strategy: str = "beam"
    compute_hypothesis_token_set: bool = False
    preserve_alignments: Optional[bool] = None
    compute_langs: bool = False
    beam_size: int = 1
    len_pen: float = 0.0
    max_generation_delta: int = 50
    temperature: Optional[float] = None


class MultiTaskDecoding:
    """Greedy / beam decoding front-end for AED models (reference: ``parts/submodules/multitask_decoding.py``)."""

    def __init__(self, decoding_cfg, transformer_decoder, log_softmax_module, tokenizer):
        cfg = decoding_cfg if decoding_cfg is not None else {}
        self.cfg = cfg
        self.tokenizer = tokenizer
        strategy = cfg_get(cfg, "strategy", "beam")
        beam = cfg_get(cfg, "beam", None) or {}
        greedy = cfg_get(cfg, "greedy", None) or {}
        beam_size = cfg_get(beam, "beam_size", cfg_get(cfg, "beam_size", 1))
        pad = getattr(tokenizer, "pad_id", 0) or 0
        bos = getattr(tokenizer, "bos_id", 1)
        eos = getattr(tokenizer, "eos_id", 2)
        kw = dict(pad=pad, bos=bos, eos=eos, max_sequence_length=transformer_decoder.max_sequence_length,
                  max_delta_length=cfg_get(beam, "max_generation_delta", cfg_get(greedy, "max_generation_delta", 50)))
        if strategy in ("greedy", "greedy_batch") or beam_size <= 1:
            self.generator = GreedySequenceGenerator(transformer_decoder.embedding, transformer_decoder.decoder, log_softmax_module,
                                                     temperature=cfg_get(greedy, "temperature", None), **kw)
        elif strategy == "beam":
            self.generator = BeamSearchSequenceGenerator(transformer_decoder.embedding, transformer_decoder.decoder, log_softmax_module,
                                                         beam_size=beam_size, len_pen=cfg_get(beam, "len_pen", 0.0), **kw)
        else:
            raise ValueError(f"unknown multitask decoding strategy '{strategy}'")
        self.eos, self.pad, self.bos = eos, pad, bos

    def decode_predictions_tensor(self, encoder_hidden_states, encoder_input_mask, decoder_input_ids=None,
                                  return_hypotheses: bool = False, partial_hypotheses=None) -> List[Hypothesis]:
        ids, scores = self.generator(decoder_input_ids=decoder_input_ids, encoder_hidden_states=encoder_hidden_states,
                                     encoder_input_mask=encoder_input_mask, return_beam_scores=True)
        prompt_len = decoder_input_ids.shape[1] if decoder_input_ids is not None else 1
        out = []
        for b in range(ids.shape[0]):
            seq = ids[b, prompt_len:].tolist()
            if self.eos in seq:
                seq = seq[: seq.index(self.eos)]
            seq = [t for t in seq if t != self.pad]
            out.append(Hypothesis(score=float(scores[b]), y_sequence=torch.tensor(seq, dtype=torch.long),
                                  text=self.decode_tokens_to_str(seq)))
        return out

    def decode_tokens_to_str(self, tokens: List[int]) -> str:
        special = set(getattr(self.tokenizer, "special_tokens", {}).values()) if hasattr(self.tokenizer, "special_tokens") else set()
        return self.tokenizer.ids_to_text([t for t in tokens if t not in special])

    def decode_ids_to_tokens(self, tokens):
        return self.tokenizer.ids_to_tokens(tokens)


def lens_to_mask(lens: torch.Tensor, max_length: int) -> torch.Tensor:
    return torch.arange(max_length, device=lens.device)[None, :] < lens[:, None]


class EncDecMultiTaskModel(ASRModel, ASRBPEMixin, ASRModuleMixin, TranscriptionMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        cfg = prepare_bpe_model_cfg(self, cfg)
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        from ..prompts import PromptFormatter

        self.prompt_format = cfg.get("prompt_format", "canary")
        self.prompt = PromptFormatter.resolve(self.prompt_format)(
            tokenizer=self.tokenizer, defaults=to_container(cfg.prompt_defaults) if cfg.get("prompt_defaults") else None)
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        md = cfg.get("model_defaults", {})
        enc_hidden = md.get("asr_enc_hidden", self.encoder._feat_out)
        lm_hidden = md.get("lm_dec_hidden", cfg.transf_decoder.config_dict.hidden_size)
        if enc_hidden != lm_hidden:
            self.encoder_decoder_proj = torch.nn.Linear(enc_hidden, lm_hidden)
        else:
            self.encoder_decoder_proj = torch.nn.Identity()
        self.use_transf_encoder = False
        te = cfg.get("transf_encoder", None)
        if te is not None and te.get("num_layers", 0) > 0:
            self.use_transf_encoder = True
            tcfg = to_container(te, resolve=True)
            tcfg.pop("_target_", None)
            self.transf_encoder = TransformerEncoderNM(vocab_size=8, **{k: v for k, v in tcfg.items() if k in (
                "hidden_size", "num_layers", "inner_size", "num_attention_heads", "ffn_dropout", "attn_score_dropout",
                "attn_layer_dropout", "hidden_act", "mask_future", "pre_ln", "pre_ln_final_layer_norm")})
            del self.transf_encoder.embedding
        vocab_size = 8 * math.ceil(self.tokenizer.vocab_size / 8)
        dcfg = to_container(cfg.transf_decoder, resolve=True)
        dconf = dict(dcfg.get("config_dict", dcfg))
        dconf["vocab_size"] = vocab_size
        dconf.pop("library", None), dconf.pop("model_name", None), dconf.pop("pretrained", None)
        self.transf_decoder = TransformerDecoderNM(pre_ln_final_layer_norm=dcfg.get("pre_ln_final_layer_norm", True), **dconf)
        with open_dict(cfg):
            if "config_dict" in cfg.transf_decoder:
                cfg.transf_decoder.config_dict.vocab_size = vocab_size
        hcfg = cfg.get("head", {})
        self.log_softmax = TokenClassifier(hidden_size=self.transf_decoder.hidden_size, num_classes=vocab_size,
                                           num_layers=hcfg.get("num_layers", 1), activation=hcfg.get("activation", "relu"),
                                           log_softmax=hcfg.get("log_softmax", True), dropout=hcfg.get("dropout", 0.0))
        self.log_softmax.mlp.layer0.weight = self.transf_decoder.embedding.token_embedding.weight  # weight tying
        std_init_range = 1 / self.transf_decoder.hidden_size ** 0.5
        self.transf_decoder.apply(lambda m: _transformer_weights_init(m, std_init_range))
        self.log_softmax.apply(lambda m: _transformer_weights_init(m, std_init_range))
        lcfg = cfg.get("loss", {})
        self.loss = SmoothedCrossEntropyLoss(pad_id=getattr(self.tokenizer, "pad_id", 0) or 0,
                                             label_smoothing=lcfg.get("label_smoothing", 0.0))
        self.use_loss_mask_for_prompt = cfg.get("use_loss_mask_for_prompt", False)
        self._setup_decoding()
        self.wer = WER(decoding=self.decoding, log_prediction=cfg.get("log_prediction", False))
        if self.__dict__.pop("_loaders_deferred", False):
            self._setup_dataloaders_from_cfg()

    def _setup_dataloader_from_config(self, config):
        """Manifests / cut sources go through the prompted dataset: every utterance becomes ``prompt tokens + transcript + end
        token`` under this model's prompt format, with the slot values (languages, task, punctuation ...) taken from the
        manifest fields (``data/cuts_datasets.py``).  Synthetic data keeps the plain token dataset."""
        if config is None:
            return None
        if cfg_get(config, "synthetic", None) is not None:
            return super()._setup_dataloader_from_config(config)
        if "prompt" not in self.__dict__:
            self._loaders_deferred = True          # called from the base constructor, before the prompt formatter exists
            return None
        import os
        from functools import partial

        from ..data.cuts import get_dataloader_from_cuts_config
        from ..data.cuts_datasets import PromptedAudioToTextCutsDataset

        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        defaults = cfg_get(config, "prompt_defaults", None)
        defaults = to_container(defaults, resolve=True) if isinstance(defaults, DictConfig) else (defaults if isinstance(defaults, dict) else None)
        ds_cls = partial(PromptedAudioToTextCutsDataset, prompt=self.prompt, prompt_defaults=defaults)
        return get_dataloader_from_cuts_config(config, rank, ws, tokenizer=self.tokenizer, dataset_cls=ds_cls)

    def _setup_decoding(self):
        dcfg = self._cfg.get("decoding", None) or OmegaConf.structured(MultiTaskDecodingConfig)
        with open_dict(self._cfg):
            self._cfg.decoding = dcfg
        self.decoding = MultiTaskDecoding(dcfg, self.transf_decoder, self.log_softmax, self.tokenizer)

    def change_decoding_strategy(self, decoding_cfg: DictConfig = None, verbose: bool = True):
        if decoding_cfg is not None:
            with open_dict(self._cfg):
                self._cfg.decoding = decoding_cfg
        self._setup_decoding()

    def change_prompt(self, prompt_format: Optional[str] = None, prompt_defaults: Optional[List[dict]] = None):
        from ..prompts import PromptFormatter

        if prompt_format is not None:
            self.prompt_format = prompt_format
        self.prompt = PromptFormatter.resolve(self.prompt_format)(tokenizer=self.tokenizer, defaults=prompt_defaults)
        with open_dict(self._cfg):
            self._cfg.prompt_format = self.prompt_format
            self._cfg.prompt_defaults = prompt_defaults

    # ------------------------------------------------------------------ forward
    def encode_audio(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None):
        if processed_signal is None:
            processed_signal, processed_signal_length = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.spec_augmentation is not None and self.training:
            processed_signal = self.spec_augmentation(input_spec=processed_signal, length=processed_signal_length)
        encoded, encoded_len = self.encoder(audio_signal=processed_signal, length=processed_signal_length)[:2]
        enc_states = encoded.transpose(1, 2)
        if isinstance(self.encoder_decoder_proj, torch.nn.Linear):
            enc_states = ops.linear(enc_states, self.encoder_decoder_proj.weight, self.encoder_decoder_proj.bias)
        enc_mask = lens_to_mask(encoded_len, enc_states.shape[1]).to(enc_states.dtype)
        if self.use_transf_encoder:
            enc_states = self.transf_encoder.encoder(enc_states, enc_mask)
        return enc_states, encoded_len, enc_mask

    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None,
                transcript=None, transcript_length=None):
        enc_states, encoded_len, enc_mask = self.encode_audio(input_signal, input_signal_length, processed_signal,
                                                              processed_signal_length)
        transf_log_probs = None
        if transcript is not None:
            dec_mask = lens_to_mask(transcript_length, transcript.shape[1]).to(enc_states.dtype)
            dec_states = self.transf_decoder(input_ids=transcript, decoder_mask=dec_mask, encoder_embeddings=enc_states,
                                             encoder_mask=enc_mask)
            transf_log_probs = self.log_softmax(hidden_states=dec_states)
        return transf_log_probs, encoded_len, enc_states, enc_mask

    def _loss_from_batch(self, batch):
        audio, audio_lens, tokens, token_lens = batch[:4]
        prompt_lens = batch[5] if len(batch) > 5 else None
        input_ids, labels = tokens[:, :-1], tokens[:, 1:]
        log_probs, encoded_len, _, _ = self.forward(input_signal=audio, input_signal_length=audio_lens, transcript=input_ids,
                                                    transcript_length=token_lens - 1)
        mask = lens_to_mask(token_lens - 1, labels.shape[1])
        if self.use_loss_mask_for_prompt and prompt_lens is not None:
            mask = mask & ~lens_to_mask(prompt_lens - 1, labels.shape[1])
        return self.loss(log_probs=log_probs, labels=labels, output_mask=mask), log_probs

    def training_step(self, batch, batch_idx):
        loss, _ = self._loss_from_batch(batch)
        self.log_dict({"train_loss": loss.detach(), "global_step": float(self.global_step)})
        return {"loss": loss}

    def validation_pass(self, batch, batch_idx, dataloader_idx=0, eval_mode="val"):
        loss, _ = self._loss_from_batch(batch)
        return {f"{eval_mode}_loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx)

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx, eval_mode="test")

    # ------------------------------------------------------------------ inference
    def _default_prompt_ids(self, B: int, device, **slots) -> torch.Tensor:
        defaults = {"source_lang": "en", "target_lang": "en", "task": "asr", "pnc": "yes", "decodercontext": "", "emotion": "undefined",
                    "itn": "no", "timestamp": "no", "diarize": "no"}
        defaults.update(slots)
        role = "user"
        need = self.prompt.get_slots(role)
        turn = {"role": role, "slots": {k: defaults[k] for k in need if k in defaults}}
        ids = self.prompt.encode_dialog([turn])["context_ids"]
        return ids.unsqueeze(0).expand(B, -1).to(device)

    def _transcribe_forward_and_decode(self, audio, lens, cfg):
        cdt = torch.bfloat16 if audio.is_cuda else None
        with ops.compute_dtype(cdt):
            enc_states, encoded_len, enc_mask = self.encode_audio(input_signal=audio, input_signal_length=lens)
            prompt_ids = self._default_prompt_ids(audio.shape[0], audio.device, **(getattr(cfg, "prompt", None) or {}))
            return self.decoding.decode_predictions_tensor(enc_states, enc_mask, decoder_input_ids=prompt_ids,
                                                           return_hypotheses=True)


def _transformer_weights_init(module, std_init_range=0.02, xavier=True):
    if isinstance(module, torch.nn.Linear):
        if xavier:
            torch.nn.init.xavier_uniform_(module.weight)
        else:
            torch.nn.init.normal_(module.weight, mean=0.0, std=std_init_range)
        if module.bias is not None:
            torch.nn.init.constant_(module.bias, 0.0)
    elif isinstance(module, torch.nn.Embedding):
        torch.nn.init.normal_(module.weight, mean=0.0, std=std_init_range)
    elif isinstance(module, torch.nn.LayerNorm):
        torch.nn.init.constant_(module.weight, 1.0)
        torch.nn.init.constant_(module.bias, 0.0)

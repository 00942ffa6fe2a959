"""Speech translation / recognition with a Transformer decoder: acoustic encoder -> (adapter) -> (Transformer encoder) ->
autoregressive Transformer decoder over BPE tokens, trained with label-smoothed cross entropy on ``<bos> text <eos>`` targets
and evaluated by beam search with corpus BLEU (reference ``asr/models/transformer_bpe_models.py:67-640``).

Config keys: ``tokenizer``, ``preprocessor``, ``encoder``, ``spec_augment``, ``transf_encoder`` (``num_layers`` 0 disables
it), ``transf_decoder`` (``hidden_size``, ``inner_size``, ``num_layers``, ``num_attention_heads``, dropouts, ``pre_ln``),
``head`` (``num_layers``, ``activation``, ``log_softmax``, ``dropout``), ``beam_search`` (``beam_size``, ``len_pen``,
``max_generation_delta``), ``label_smoothing``.  The tokenizer must define bos / eos / pad ids; datasets add the start and
end tokens (``use_start_end_token`` is forced on).
"""
from __future__ import annotations

import itertools
import math
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..core.config import DictConfig, open_dict, to_container
from ..core.instantiate import from_config_dict
from ..decoding.rnnt_decoding import Hypothesis
from ..losses.cross_entropy import SmoothedCrossEntropyLoss
from ..modules.transformer_nm import BeamSearchSequenceGenerator, TokenClassifier, TransformerDecoderNM, TransformerEncoderNM
from ..utils.logging import logging
from .aed_models import _transformer_weights_init, lens_to_mask
from .asr_model import ASRBPEMixin, ASRModel, ASRModuleMixin, TranscriptionMixin
from .ctc_models import prepare_bpe_model_cfg

_TRANSFORMER_KEYS = ("hidden_size", "num_layers", "inner_size", "num_attention_heads", "ffn_dropout", "attn_score_dropout",
                     "attn_layer_dropout", "hidden_act", "pre_ln", "pre_ln_final_layer_norm", "max_sequence_length",
                     "embedding_dropout", "learn_positional_encodings", "num_token_types")


def corpus_bleu(hyps: List[str], refs: List[str], max_n: int = 4, tokenize: str = "13a") -> float:
    """Corpus BLEU (single reference) with the ``13a`` tokenisation of the WMT scorer: punctuation split from words, except
    periods and commas between digits."""
    import re
    from collections import Counter

    def tok(s: str) -> List[str]:
        if tokenize != "13a":
            return s.split()
        s = re.sub(r"([\{-\~\[-\` -\&\(-\+\:-\@\/])", r" \1 ", s)
        s = re.sub(r"([^0-9])([\.,])", r"\1 \2 ", s)
        s = re.sub(r"([\.,])([^0-9])", r" \1 \2", s)
        s = re.sub(r"([0-9])(-)", r"\1 \2 ", s)
        return s.split()

    match, total, hl, rl = [0] * max_n, [0] * max_n, 0, 0
    for h, r in zip(hyps, refs):
        ht, rt = tok(h), tok(r)
        hl, rl = hl + len(ht), rl + len(rt)
        for n in range(1, max_n + 1):
            hc = Counter(tuple(ht[i:i + n]) for i in range(len(ht) - n + 1))
            rc = Counter(tuple(rt[i:i + n]) for i in range(len(rt) - n + 1))
            match[n - 1] += sum(min(c, rc[g]) for g, c in hc.items())
            total[n - 1] += max(0, len(ht) - n + 1)
    if hl == 0 or min(total) == 0 or match[0] == 0:
        return 0.0
    # higher orders without a match are floored the way the WMT scorer does ("floor" smoothing at 0.1 of a count would hide
    # real zeros; an exact zero BLEU is reported instead)
    if min(match) == 0:
        return 0.0
    logp = sum(math.log(m / t) for m, t in zip(match, total)) / max_n
    bp = 1.0 if hl > rl else math.exp(1 - rl / hl)
    return 100.0 * bp * math.exp(logp)


class EncDecTransfModelBPE(ASRModel, ASRBPEMixin, ASRModuleMixin, TranscriptionMixin):
    def __init__(self, cfg: DictConfig, trainer=None):
        cfg = prepare_bpe_model_cfg(self, cfg)
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        for name in ("bos_id", "eos_id", "pad_id"):
            if getattr(self.tokenizer, name, None) is None or getattr(self.tokenizer, name) < 0:
                raise ValueError(f"the tokenizer of a Transformer-decoder model must define {name}")
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.encoder = from_config_dict(cfg.encoder)
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        dcfg = to_container(cfg.transf_decoder, resolve=True)
        dcfg = dict(dcfg.get("config_dict", dcfg))
        d_enc = cfg.encoder.get("d_model", None) or self.encoder._feat_out
        self.adapter = torch.nn.Linear(d_enc, dcfg["hidden_size"]) if d_enc != dcfg["hidden_size"] else torch.nn.Identity()
        te = to_container(cfg.transf_encoder, resolve=True) if cfg.get("transf_encoder") is not None else {"num_layers": 0}
        self.use_transf_encoder = te.get("num_layers", 0) > 0
        if self.use_transf_encoder:
            full = TransformerEncoderNM(vocab_size=8, mask_future=False, **{k: v for k, v in te.items() if k in _TRANSFORMER_KEYS})
            self.transf_encoder = full.encoder                      # the layer stack only: its input is the acoustic encoding
            self.transf_encoder.apply(lambda m: _transformer_weights_init(m, 1 / te["hidden_size"] ** 0.5))
        vocab_size = 8 * math.ceil(self.tokenizer.vocab_size / 8)
        self.transf_decoder = TransformerDecoderNM(vocab_size=vocab_size, **{k: v for k, v in dcfg.items() if k in _TRANSFORMER_KEYS})
        h = cfg.get("head", {})
        self.log_softmax = TokenClassifier(hidden_size=self.transf_decoder.hidden_size, num_classes=vocab_size, num_layers=h.get("num_layers", 1),
                                           activation=h.get("activation", "relu"), log_softmax=h.get("log_softmax", True),
                                           dropout=h.get("dropout", 0.0))
        self.log_softmax.mlp.layer0.weight = self.transf_decoder.embedding.token_embedding.weight
        std = 1 / self.transf_decoder.hidden_size ** 0.5
        self.transf_decoder.apply(lambda m: _transformer_weights_init(m, std))
        self.log_softmax.apply(lambda m: _transformer_weights_init(m, std))
        bs = cfg.get("beam_search", {})
        self.beam_search = BeamSearchSequenceGenerator(
            self.transf_decoder.embedding, self.transf_decoder.decoder, self.log_softmax, beam_size=bs.get("beam_size", 4),
            len_pen=bs.get("len_pen", 0.0), pad=self.tokenizer.pad_id, bos=self.tokenizer.bos_id, eos=self.tokenizer.eos_id,
            max_sequence_length=self.transf_decoder.max_sequence_length, max_delta_length=bs.get("max_generation_delta", 50))
        self.transf_loss = SmoothedCrossEntropyLoss(pad_id=self.tokenizer.pad_id, label_smoothing=cfg.get("label_smoothing", 0.0))
        self._loss_sum, self._loss_n = 0.0, 0

    # ------------------------------------------------------------------ data
    def _setup_dataloader_from_config(self, config):
        if config is not None and not config.get("use_start_end_token", False):
            with open_dict(config):
                config["use_start_end_token"] = True           # targets are <bos> text <eos>
        return super()._setup_dataloader_from_config(config)

    # ------------------------------------------------------------------ forward
    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None,
                transcript=None, transcript_length=None):
        if (input_signal is None) == (processed_signal is None):
            raise ValueError("pass either input_signal (+ length) or processed_signal (+ length)")
        if processed_signal is None:
            processed_signal, processed_signal_length = self.preprocessor(input_signal=input_signal, length=input_signal_length)
        if self.spec_augmentation is not None and self.training:
            processed_signal = self.spec_augmentation(input_spec=processed_signal, length=processed_signal_length)
        encoded, encoded_len = self.encoder(audio_signal=processed_signal, length=processed_signal_length)[:2]
        enc_states = encoded.transpose(1, 2)
        if isinstance(self.adapter, torch.nn.Linear):
            enc_states = ops.linear(enc_states, self.adapter.weight, self.adapter.bias)
        enc_mask = lens_to_mask(encoded_len, enc_states.shape[1]).to(enc_states.dtype)
        if self.use_transf_encoder:
            enc_states = self.transf_encoder(enc_states, enc_mask)
        log_probs = None
        if transcript is not None:
            dec_mask = lens_to_mask(transcript_length, transcript.shape[1]).to(enc_states.dtype)
            dec = self.transf_decoder(input_ids=transcript, decoder_mask=dec_mask, encoder_embeddings=enc_states, encoder_mask=enc_mask)
            log_probs = self.log_softmax(hidden_states=dec)
        return log_probs, encoded_len, enc_states, enc_mask

    def compute_audio_loss(self, batch):
        signal, signal_len, transcript, transcript_len = batch[:4]
        input_ids, labels = transcript[:, :-1], transcript[:, 1:]
        log_probs, _, enc_states, enc_mask = self.forward(input_signal=signal, input_signal_length=signal_len, transcript=input_ids,
                                                          transcript_length=transcript_len - 1)
        mask = lens_to_mask(transcript_len - 1, labels.shape[1])
        return self.transf_loss(log_probs=log_probs, labels=labels, output_mask=mask), log_probs, enc_states, enc_mask

    def training_step(self, batch, batch_idx):
        loss = self.compute_audio_loss(batch)[0]
        self.log_dict({"train_loss": loss.detach(), "global_step": float(self.global_step)})
        return {"loss": loss}

    def _strip(self, ids: List[int]) -> List[int]:
        t = self.tokenizer
        out = []
        for i in ids:
            if i == t.eos_id:
                break
            if i not in (t.bos_id, t.pad_id):
                out.append(i)
        return out

    def validation_pass(self, batch, batch_idx, dataloader_idx=0, eval_mode="val"):
        loss, log_probs, enc_states, enc_mask = self.compute_audio_loss(batch)
        hyp = self.beam_search(encoder_hidden_states=enc_states, encoder_input_mask=enc_mask)
        translations = [self.tokenizer.ids_to_text(self._strip(s)) for s in hyp.cpu().tolist()]
        truths = [self.tokenizer.ids_to_text(self._strip(s)) for s in batch[2].cpu().tolist()]
        n = log_probs.shape[0] * log_probs.shape[1]
        return {f"{eval_mode}_loss": loss, "loss_weight": n, "translations": translations, "ground_truths": truths}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx)

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_pass(batch, batch_idx, dataloader_idx, eval_mode="test")

    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0, eval_mode: str = "val"):
        """Loss averaged with the number of scored positions as weight; BLEU over the translations of all ranks."""
        if not outputs:
            return {}
        pairs = [(t, g) for o in outputs for t, g in zip(o["translations"], o["ground_truths"]) if g.strip()]
        sums = torch.tensor([sum(float(o[f"{eval_mode}_loss"]) * o["loss_weight"] for o in outputs),
                             float(sum(o["loss_weight"] for o in outputs))], dtype=torch.float64, device=self.device)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sums)
            gathered = [None] * dist.get_world_size()
            dist.all_gather_object(gathered, pairs)
            pairs = list(itertools.chain(*gathered))
        score = corpus_bleu([t for t, _ in pairs], [g for _, g in pairs])
        loss = float(sums[0] / sums[1].clamp(min=1))
        name = self.get_validation_dataloader_prefix(dataloader_idx) if eval_mode == "val" else self.get_test_dataloader_prefix(dataloader_idx)
        logging.info(f"{eval_mode} set {dataloader_idx}: loss {loss:.4f}  BLEU {score:.2f} on {len(pairs)} sentences")
        logs = {f"{name}{eval_mode}_loss": torch.tensor(loss), f"{name}{eval_mode}_sacreBLEU": torch.tensor(score)}
        return {f"{eval_mode}_loss": torch.tensor(loss), "log": logs}

    def multi_test_epoch_end(self, outputs, dataloader_idx: int = 0):
        return self.multi_validation_epoch_end(outputs, dataloader_idx, eval_mode="test")

    # ------------------------------------------------------------------ inference
    @torch.no_grad()
    def _transcribe_forward_and_decode(self, audio, lens, cfg):
        cdt = torch.bfloat16 if audio.is_cuda else None
        with ops.compute_dtype(cdt):
            _, _, enc_states, enc_mask = self.forward(input_signal=audio, input_signal_length=lens)
            hyp = self.beam_search(encoder_hidden_states=enc_states, encoder_input_mask=enc_mask)
        out = []
        for b, s in enumerate(hyp.cpu().tolist()):
            ids = self._strip(s)
            out.append(Hypothesis(score=0.0, y_sequence=torch.tensor(ids, dtype=torch.long), text=self.tokenizer.ids_to_text(ids)))
        return out


"""Shared machinery of the ASR models: base class, tokenizer mix-in, transcription and streaming mix-ins.

* ``ASRModel`` — multi-validation aggregation, auxiliary losses from the tensor registry, NaN/Inf gradient
  containment with one MIN all-reduce, CUDA-graph decoder toggles around train / validation epochs
  (reference: ``nemo/collections/asr/models/asr_model.py:33-254``).
* ``ASRBPEMixin`` — ``tokenizer: {dir, type: bpe|wpe|agg}`` set-up with artifact registration
  (``parts/mixins/mixins.py:41-360``).
* ``TranscriptionMixin`` — ``transcribe(audio=[paths|arrays|tensors], batch_size, return_hypotheses,
  timestamps, ...)`` with dither / pad_to switched off for inference (``parts/mixins/transcription.py:199-640``).
* ``ASRModuleMixin`` — ``change_attention_model``, ``conformer_stream_step`` for cache-aware streaming
  (``parts/mixins/mixins.py:624-763``).
* ``InterCTCMixin`` — intermediate-layer CTC losses (``parts/mixins/interctc_mixin.py:214-294``).
"""
from __future__ import annotations

import copy
import json
import os
import tempfile
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict, to_container
from ..core.modelpt import ModelPT
from ..core.module import AccessMixin
from ..data import audio_to_text as _data
from ..decoding.rnnt_decoding import Hypothesis
from ..utils.logging import logging


@dataclass
class TranscribeConfig:
    batch_size: int = 4
    return_hypotheses: bool = False
    num_workers: Optional[int] = None
    channel_selector: Any = None
    augmentor: Optional[DictConfig] = None
    timestamps: Optional[bool] = None
    verbose: bool = True
    partial_hypothesis: Optional[List[Any]] = None
    chunk_duration_seconds: Optional[float] = None      # recordings longer than this are cut into chunks of this length and merged


class ASRModel(ModelPT):
    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0):
        if not outputs:
            return {}
        # validation data is sharded over ranks: numerators and denominators are summed over all of them first
        losses = [x["val_loss"] for x in outputs if "val_loss" in x]
        loss_sum = float(torch.stack([l.detach().float() for l in losses]).sum()) if losses else 0.0
        num = sum(float(x["val_wer_num"]) for x in outputs if "val_wer_num" in x)
        den = sum(float(x["val_wer_denom"]) for x in outputs if "val_wer_denom" in x)
        loss_sum, loss_cnt, num, den = self.reduce_sums([loss_sum, float(len(losses)), num, den], self.device)
        val_loss_mean = torch.tensor(loss_sum / loss_cnt) if loss_cnt > 0 else None
        log = {}
        if val_loss_mean is not None:
            log["val_loss"] = val_loss_mean
        if den > 0:
            log["val_wer"] = torch.tensor(num / den)
        return {**({"val_loss": val_loss_mean} if val_loss_mean is not None else {}), "log": log}

    def multi_test_epoch_end(self, outputs, dataloader_idx: int = 0):
        out = self.multi_validation_epoch_end(
            [{k.replace("test_", "val_"): v for k, v in o.items()} for o in outputs], dataloader_idx)
        log = {k.replace("val_", "test_"): v for k, v in out.get("log", {}).items()}
        return {"log": log}

    def add_auxiliary_losses(self, loss: torch.Tensor, reset_registry: bool = False) -> torch.Tensor:
        """Add losses that sub-modules published under the ``loss`` registry key."""
        if not self.training:
            return loss
        if AccessMixin.is_access_enabled(self.model_guid):
            for _, reg in AccessMixin.get_module_registry(self).items():
                if "loss" in reg:
                    loss = loss + sum(reg["loss"])
        if reset_registry:
            AccessMixin.reset_registry(self)
        return loss

    def on_after_backward(self):
        """``skip_nan_grad``: if any rank has a non-finite gradient every rank zeroes its gradients."""
        if not cfg_get(self._cfg, "skip_nan_grad", False):
            return
        dev = self.device
        valid = torch.ones(1, device=dev, dtype=torch.float32)
        arena = next((getattr(p, "_arena", None) for p in self.parameters() if getattr(p, "_arena", None) is not None), None)
        if arena is not None:
            valid = torch.isfinite(arena.grad).all().float().view(1)
        else:
            for p in self.parameters():
                if p.grad is not None and not torch.isfinite(p.grad).all():
                    valid = valid * 0
                    break
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            v = valid if dist.get_backend() == "nccl" else valid.cpu()
            dist.all_reduce(v, op=dist.ReduceOp.MIN)
            valid = v.to(dev)
        if valid.item() < 1:
            logging.warning("detected inf or nan values in gradients! Setting gradients to zero.")
            if arena is not None:
                arena.grad.zero_()
            else:
                self.zero_grad()

    # CUDA-graph decoders are kept off while training (shapes / memory change) and on for evaluation
    def _toggle_graph_decoder(self, enable: bool):
        for attr in ("decoding", "ctc_decoding"):
            dec = getattr(self, attr, None)
            inner = getattr(dec, "decoding", None)
            if inner is not None and hasattr(inner, "maybe_enable_cuda_graphs"):
                (inner.maybe_enable_cuda_graphs if enable else inner.disable_cuda_graphs)()

    def on_train_epoch_start(self):
        self._toggle_graph_decoder(False)

    def on_train_epoch_end(self):
        self._toggle_graph_decoder(True)

    def on_validation_epoch_start(self):
        self._toggle_graph_decoder(True)

    def on_test_epoch_start(self):
        self._toggle_graph_decoder(True)

    @property
    def oomptimizer_schema(self) -> dict:
        return {"cls": tuple, "inputs": [{"name": "audio_signal", "type": "NeuralType(('B','T'), AudioSignal())", "seq_length": "input"},
                                         {"name": "audio_signal_length", "type": "lengths", "seq_length": "input"},
                                         {"name": "transcripts", "type": "labels", "seq_length": "output",
                                          "vocab_size": getattr(getattr(self, "tokenizer", None), "vocab_size", None)},
                                         {"name": "transcript_length", "type": "lengths", "seq_length": "output"}]}

    # ------------------------------------------------------------------ data plumbing shared by CTC / RNNT models
    def _setup_dataloader_from_config(self, config):
        if config is None:
            return None
        tok = getattr(self, "tokenizer", None)
        labels = None
        if tok is None:
            labels = cfg_get(config, "labels", None) or cfg_get(self._cfg, "labels", None)
            if labels is None and hasattr(self, "decoder") and getattr(self.decoder, "vocabulary", None):
                labels = self.decoder.vocabulary
        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        if cfg_get(config, "synthetic", None) is None and (cfg_get(config, "use_lhotse", False) or
                                                           cfg_get(config, "input_cfg", None) is not None):
            from ..data.cuts import get_dataloader_from_cuts_config

            return get_dataloader_from_cuts_config(config, rank, ws, tokenizer=tok, labels=list(labels) if labels is not None else None)
        ds = _data.build_speech_dataset(config, tokenizer=tok, labels=list(labels) if labels is not None else None)
        if ds is None:
            return None
        return _data.get_dataloader_from_config(config, ds, rank, ws)

    def setup_training_data(self, train_data_config):
        self._train_dl = self._setup_dataloader_from_config(train_data_config)

    def setup_validation_data(self, val_data_config):
        if val_data_config is not None and "shuffle" not in val_data_config:
            with open_dict(val_data_config):
                val_data_config["shuffle"] = False
        self._validation_dl = self._setup_dataloader_from_config(val_data_config)

    def setup_test_data(self, test_data_config):
        self._test_dl = self._setup_dataloader_from_config(test_data_config)


class ASRBPEMixin:
    def _setup_tokenizer(self, tokenizer_cfg):
        from .. import tokenizers as T

        if tokenizer_cfg is None:
            raise ValueError("`cfg` must have `tokenizer` config to create a tokenizer !")
        tcfg = to_container(tokenizer_cfg, resolve=True) if isinstance(tokenizer_cfg, DictConfig) else dict(tokenizer_cfg)
        ttype = (tcfg.get("type") or "bpe").lower()
        self.tokenizer_cfg = tcfg
        self.tokenizer_type = ttype
        if ttype == "synthetic":
            self.tokenizer = T.SyntheticTokenizer(int(tcfg["vocab_size"]))
        elif ttype == "agg":
            self.tokenizer = self._make_aggregate(tcfg, "tokenizer")
        else:
            self.tokenizer = self._make_monolingual(tcfg, "tokenizer")
        logging.info(f"Tokenizer {type(self.tokenizer).__name__} initialized with {self.tokenizer.vocab_size} tokens")

    def _make_monolingual(self, tcfg: dict, cfg_prefix: str):
        from .. import tokenizers as T

        ttype = (tcfg.get("type") or "bpe").lower()
        tdir = tcfg.get("dir")
        if ttype == "bpe":
            model_path = tcfg.get("model_path") or (os.path.join(tdir, "tokenizer.model") if tdir else None)
            model_path = self.register_artifact(f"{cfg_prefix}.model_path", model_path)
            with open_dict(self._cfg):
                OmegaConf.update(self._cfg, f"{cfg_prefix}.model_path", tcfg.get("model_path") or model_path)
            for key, fname in (("vocab_path", "vocab.txt"), ("spe_tokenizer_vocab", "tokenizer.vocab")):
                p = tcfg.get(key) or (os.path.join(tdir, fname) if tdir else None)
                if p and (os.path.exists(p) or str(p).startswith("nemo:")):
                    self.register_artifact(f"{cfg_prefix}.{key}", p, verify_src_exists=False)
            return T.SentencePieceTokenizer(model_path=model_path)
        if ttype == "wpe":
            vocab_path = tcfg.get("vocab_path") or os.path.join(tdir, "vocab.txt")
            vocab_path = self.register_artifact(f"{cfg_prefix}.vocab_path", vocab_path)
            return T.WordPieceVocabTokenizer(vocab_path)
        if ttype == "char":
            return T.CharTokenizer(tcfg.get("vocab") or tcfg.get("vocab_path"))
        if ttype in ("spl", "special"):
            p = tcfg.get("vocab_path") or os.path.join(tdir, "tokenizer.vocab")
            p = self.register_artifact(f"{cfg_prefix}.vocab_path", p)
            return T.SpecialTokenTable(p)
        raise ValueError(f"`tokenizer.type` must be one of bpe|wpe|agg|char|synthetic, got {ttype}")

    def _make_aggregate(self, tcfg: dict, cfg_prefix: str):
        from .. import tokenizers as T

        toks = {}
        for lang, sub in tcfg["langs"].items():
            toks[lang] = self._make_monolingual(dict(sub), f"{cfg_prefix}.langs.{lang}")
        if tcfg.get("custom_tokenizer", {}) and "canary" in str(tcfg["custom_tokenizer"].get("_target_", "")).lower() or \
                T.CANARY_SPECIAL_TOKENIZER in toks:
            return T.CanaryTokenizer(toks)
        return T.AggregateTokenizer(toks)


class InterCTCMixin:
    """``interctc: {loss_weights: [...], apply_at_layers: [...]}`` — extra CTC losses on intermediate encoder layers."""

    def setup_interctc(self, decoder_name: str, loss_name: str, wer_name: str):
        ic = cfg_get(self._cfg, "interctc", None)
        self._interctc = {"enabled": False}
        if ic is None:
            return
        w = list(cfg_get(ic, "loss_weights", []) or [])
        layers = list(cfg_get(ic, "apply_at_layers", []) or [])
        if len(w) != len(layers):
            raise ValueError("Length of interctc.apply_at_layers has to match interctc.loss_weights")
        if not w:
            return
        main = 1.0 - sum(w)
        if main <= 0:
            raise ValueError("Make sure that sum of intermediate loss weights is < 1.0.")
        self._interctc = {"enabled": True, "weights": w, "layers": layers, "main": main, "decoder": decoder_name,
                          "loss": loss_name}
        AccessMixin.update_access_cfg({"interctc": {"capture_layers": layers}}, self.model_guid)

    def is_interctc_enabled(self) -> bool:
        return getattr(self, "_interctc", {}).get("enabled", False)

    def set_interctc_enabled(self, enabled: bool):
        if getattr(self, "_interctc", {}).get("weights"):
            self._interctc["enabled"] = enabled
            AccessMixin.set_access_enabled(enabled, self.model_guid)

    def add_interctc_losses(self, loss_value, transcript, transcript_len, compute_wer=False, log_prefix="train_"):
        if not self.is_interctc_enabled() or not AccessMixin.is_access_enabled(self.model_guid):
            return loss_value, {}
        ic = self._interctc
        metrics = {f"{log_prefix}final_loss": loss_value.detach()}
        total = ic["main"] * loss_value
        captured = {}
        for _, reg in AccessMixin.get_module_registry(self.encoder).items():
            captured.update(reg)
        dec, lossf = getattr(self, ic["decoder"]), getattr(self, ic["loss"])
        for layer, w in zip(ic["layers"], ic["weights"]):
            outs = captured.get(f"interctc/layer_output_{layer}")
            lens = captured.get(f"interctc/layer_length_{layer}")
            if not outs:
                raise RuntimeError(f"Intermediate layer {layer} was not captured; is the access registry enabled?")
            lp = dec(encoder_output=outs[-1])
            li = lossf(log_probs=lp, targets=transcript, input_lengths=lens[-1], target_lengths=transcript_len)
            metrics[f"{log_prefix}inter_ctc_loss_l{layer}"] = li.detach()
            total = total + w * li
        AccessMixin.reset_registry(self.encoder)
        metrics[f"{log_prefix}loss"] = total.detach()
        return total, metrics


from ..core.adapters import ASRAdapterModelMixin  # noqa: E402


class ASRModuleMixin(ASRAdapterModelMixin):
    def change_attention_model(self, self_attention_model: str = None, att_context_size: List[int] = None,
                               update_config: bool = True):
        if not hasattr(self, "encoder") or not hasattr(self.encoder, "change_attention_model"):
            logging.info("Model does not have an encoder with a switchable attention model; nothing changed")
            return
        self.encoder.change_attention_model(self_attention_model, att_context_size, update_config, self.device)
        if update_config:
            with open_dict(self._cfg):
                self._cfg.encoder.self_attention_model = self.encoder.self_attention_model
                self._cfg.encoder.att_context_size = list(self.encoder.att_context_size)

    def change_subsampling_conv_chunking_factor(self, subsampling_conv_chunking_factor: int, update_config: bool = True):
        self.encoder.subsampling_conv_chunking_factor = subsampling_conv_chunking_factor
        if update_config:
            with open_dict(self._cfg):
                self._cfg.encoder.subsampling_conv_chunking_factor = subsampling_conv_chunking_factor

    @torch.no_grad()
    def conformer_stream_step(self, processed_signal: torch.Tensor, processed_signal_length: torch.Tensor = None,
                              cache_last_channel=None, cache_last_time=None, cache_last_channel_len=None,
                              keep_all_outputs: bool = True, previous_hypotheses: List[Hypothesis] = None,
                              previous_pred_out=None, drop_extra_pre_encoded: int = None,
                              return_transcription: bool = True, return_log_probs: bool = False,
                              bypass_pre_encode: bool = False):
        """One cache-aware streaming step: encoder chunk with caches, then greedy decode continuing from the
        previous hypotheses.  Returns ``(greedy_predictions, all_hyp_or_transcribed_texts, cache_last_channel_next,
        cache_last_time_next, cache_last_channel_next_len, best_hyp[, encoded])``."""
        from .ctc_models import EncDecCTCModel
        from .rnnt_models import EncDecRNNTModel

        if not isinstance(self, (EncDecRNNTModel, EncDecCTCModel)):
            raise NotImplementedError(f"{type(self)} is not supported for streaming")
        decoder_type = getattr(self, "cur_decoder", None) or ("ctc" if isinstance(self, EncDecCTCModel) else "rnnt")
        with ops.compute_dtype(ops.get_compute_dtype()):
            (encoded, encoded_len, clc_next, clt_next, clcl_next) = self.encoder.cache_aware_stream_step(
                processed_signal=processed_signal, processed_signal_length=processed_signal_length,
                cache_last_channel=cache_last_channel, cache_last_time=cache_last_time,
                cache_last_channel_len=cache_last_channel_len, keep_all_outputs=keep_all_outputs,
                drop_extra_pre_encoded=drop_extra_pre_encoded, bypass_pre_encode=bypass_pre_encode)
        if decoder_type == "ctc":
            dec = self.ctc_decoder if hasattr(self, "ctc_decoder") else self.decoder
            decoding = self.ctc_decoding if hasattr(self, "ctc_decoding") else self.decoding
            log_probs = dec(encoder_output=encoded)
            preds = log_probs.argmax(dim=-1)
            greedy_predictions = []
            all_hyp = []
            for b in range(preds.shape[0]):
                cur = preds[b, : int(encoded_len[b])]
                prev = previous_pred_out[b] if previous_pred_out is not None else cur.new_zeros(0)
                full = torch.cat([prev, cur])
                greedy_predictions.append(full)
            lens = torch.tensor([len(g) for g in greedy_predictions], device=preds.device)
            padded = torch.nn.utils.rnn.pad_sequence(greedy_predictions, batch_first=True, padding_value=decoding.blank_id)
            all_hyp = decoding.ctc_decoder_predictions_tensor(padded, lens) if return_transcription else None
            best_hyp = all_hyp
            result = [greedy_predictions, all_hyp, clc_next, clt_next, clcl_next, best_hyp]
        else:
            best_hyp = self.decoding.rnnt_decoder_predictions_tensor(
                encoder_output=encoded, encoded_lengths=encoded_len, return_hypotheses=True,
                partial_hypotheses=previous_hypotheses)
            greedy_predictions = [h.y_sequence for h in best_hyp]
            result = [greedy_predictions, best_hyp, clc_next, clt_next, clcl_next, best_hyp]
        if return_log_probs:
            result.append(encoded)
            result.append(encoded_len)
        return tuple(result)


class TranscriptionMixin:
    @torch.no_grad()
    def transcribe(self, audio: Union[str, List[str], np.ndarray, torch.Tensor, List[np.ndarray], List[torch.Tensor]],
                   batch_size: int = 4, return_hypotheses: bool = False, num_workers: int = 0,
                   channel_selector=None, augmentor=None, verbose: bool = False, timestamps: Optional[bool] = None,
                   override_config: Optional[TranscribeConfig] = None, chunk_duration_seconds: Optional[float] = None, **kw):
        """Transcribe files / arrays.  Returns texts, or ``Hypothesis`` objects when ``return_hypotheses`` (or
        ``timestamps``) is set.  ``chunk_duration_seconds``: very long recordings are cut into non-overlapping chunks of that
        length, the chunks are transcribed as a batch and merged back (tokens concatenated, frame indices shifted)."""
        cfg = override_config or TranscribeConfig(batch_size=batch_size, return_hypotheses=return_hypotheses,
                                                  num_workers=num_workers, channel_selector=channel_selector,
                                                  timestamps=timestamps, verbose=verbose, chunk_duration_seconds=chunk_duration_seconds)
        if isinstance(audio, (str, np.ndarray)) or torch.is_tensor(audio) and audio.dim() == 1:
            audio = [audio]
        elif torch.is_tensor(audio):
            audio = list(audio)
        results: List[Any] = []
        for out in self.transcribe_generator(audio, cfg):
            results.extend(out)
        return results

    def _transcribe_chunked(self, audio, cfg: TranscribeConfig, sr: int):
        """Every recording -> its chunks -> one flat list through the ordinary path -> merged per recording."""
        import dataclasses

        from ..utils.asr_eval_utils import merge_parallel_chunks

        n = int(cfg.chunk_duration_seconds * sr)
        flat, owner = [], []
        for i, a in enumerate(audio):
            w = torch.from_numpy(_data.load_audio(a, sr, channel_selector=cfg.channel_selector)) if isinstance(a, str) else torch.as_tensor(a, dtype=torch.float32).flatten()
            pieces = list(w.split(n)) if w.numel() > n else [w]
            if len(pieces) > 1 and pieces[-1].numel() < sr // 10:          # a sliver at the end joins the chunk before it
                pieces[-2] = torch.cat([pieces[-2], pieces[-1]])
                pieces.pop()
            flat += pieces
            owner += [i] * len(pieces)
        inner = dataclasses.replace(cfg, chunk_duration_seconds=None, return_hypotheses=True)
        hyps = [h for out in self.transcribe_generator(flat, inner) for h in out]
        feat = getattr(getattr(self, "preprocessor", None), "featurizer", None)
        hop = int(getattr(feat, "hop_length", 160))
        sub = int(getattr(getattr(self, "encoder", None), "subsampling_factor", 1))
        dec = getattr(self, "decoding", None) or getattr(self, "ctc_decoding", None)
        to_text = getattr(dec, "decode_tokens_to_str", None)
        merged = []
        for i in range(len(audio)):
            idx = [k for k, o in enumerate(owner) if o == i]
            frames = [int(hyps[k].length) if int(hyps[k].length or 0) > 0 else -(-flat[k].numel() // (hop * sub)) for k in idx]
            m = merge_parallel_chunks([hyps[k] for k in idx], frames, to_text) if len(idx) > 1 else hyps[idx[0]]
            merged.append(m)
        return merged

    def transcribe_generator(self, audio, cfg: TranscribeConfig):
        sr = cfg_get(cfg_get(self._cfg, "preprocessor", {}), "sample_rate", 16000)
        if getattr(cfg, "chunk_duration_seconds", None):
            hyps = self._transcribe_chunked(audio, cfg, int(sr))
            yield hyps if (cfg.return_hypotheses or cfg.timestamps) else [h.text for h in hyps]
            return
        state = self._transcribe_on_begin(cfg)
        try:
            sr = cfg_get(cfg_get(self._cfg, "preprocessor", {}), "sample_rate", 16000)
            for s in range(0, len(audio), cfg.batch_size):
                chunk = audio[s:s + cfg.batch_size]
                waves = []
                for a in chunk:
                    if isinstance(a, str):
                        waves.append(torch.from_numpy(_data.load_audio(a, sr, channel_selector=cfg.channel_selector)))
                    else:
                        waves.append(torch.as_tensor(a, dtype=torch.float32).flatten())
                lens = torch.tensor([len(w) for w in waves], dtype=torch.long)
                x = torch.nn.utils.rnn.pad_sequence(waves, batch_first=True)
                dev = self.device
                hyps = self._transcribe_forward_and_decode(x.to(dev), lens.to(dev), cfg)
                if cfg.return_hypotheses or cfg.timestamps:
                    yield hyps
                else:
                    yield [h.text for h in hyps]
        finally:
            self._transcribe_on_end(state)

    def _transcribe_on_begin(self, cfg: TranscribeConfig):
        st = {"training": self.training}
        feat = getattr(getattr(self, "preprocessor", None), "featurizer", None)
        if feat is not None:
            st["dither"], st["pad_to"] = feat.dither, feat.pad_to
            feat.dither, feat.pad_to = 0.0, 0
        self.eval()
        st["ts"] = []
        if cfg.timestamps:
            for attr in ("decoding", "ctc_decoding"):
                d = getattr(self, attr, None)
                if d is not None:
                    st["ts"].append((d, d.compute_timestamps))
                    d.compute_timestamps = True
        return st

    def _transcribe_on_end(self, st):
        feat = getattr(getattr(self, "preprocessor", None), "featurizer", None)
        if feat is not None and "dither" in st:
            feat.dither, feat.pad_to = st["dither"], st["pad_to"]
        for d, prev in st.get("ts", []):
            d.compute_timestamps = prev
        self.train(st["training"])

    def _transcribe_forward_and_decode(self, audio, lens, cfg) -> List[Hypothesis]:
        raise NotImplementedError

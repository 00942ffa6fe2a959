"""Full-duplex speech models on a decoder-only LLM, and SALM variants.

* ``DuplexSTTModel`` — frame-synchronous speech-to-text: at every perception frame the LLM reads ``user audio embedding +
  embedding of the agent's previous text token`` and predicts the agent's next text token (PAD while listening, BOS ... EOS while
  answering).
* ``DuplexS2SModel`` — adds the agent's speech channel: the input also carries the embeddings of the previous frame's audio-codec
  codes (one table per codebook) and an audio head predicts the next codes of all codebooks; generated codes are turned into a
  waveform by the codec.  Codebook vocabulary = codec size + 3 control codes (speech BOS / EOS / delay).
* ``SALMWithAsrDecoder`` — SALM plus an auxiliary CTC head on the perception output (loss = LLM loss + ``asr_weight`` · CTC).

Reference: ``speechlm2/models/duplex_s2s_model.py:48-400`` (channels, control codes, ``forward`` with ``text_logits`` /
``audio_logits``, ``offline_inference``), ``duplex_stt_model.py``, ``salm_asr_decoder.py``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get, open_dict
from ..core.modelpt import ModelPT
from .llm import CausalLM
from .perception import AudioPerceptionModule
from .salm import SALM


class _IdTokenizer:
    """Stand-in when no tokenizer is attached (synthetic data): every character is its code point modulo a small range."""
    pad_id, bos_id, eos_id = 0, 1, 2

    def text_to_ids(self, text):
        return [3 + (ord(c) % 29) for c in text if not c.isspace()]

    def ids_to_text(self, ids):
        return " ".join(str(i) for i in ids)


class DuplexSTTModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None, llm: Optional[CausalLM] = None, tokenizer=None, perception: Optional[nn.Module] = None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.tokenizer = tokenizer
        self.llm = llm if llm is not None else CausalLM.from_config(dict(cfg.llm))
        self.embed_tokens = self.llm.model.embed_tokens
        self.llm.model.embed_tokens = None
        if perception is not None:
            self.perception = perception
        else:
            pcfg = cfg.perception
            with open_dict(pcfg):
                pcfg.output_dim = self.llm.config.hidden_size
            self.perception = AudioPerceptionModule(pcfg)
        self.text_pad_id = int(cfg_get(cfg, "text_pad_id", getattr(tokenizer, "pad_id", 0) or 0))
        self.text_bos_id = int(cfg_get(cfg, "text_bos_id", getattr(tokenizer, "bos_id", 1) or 1))
        self.text_eos_id = int(cfg_get(cfg, "text_eos_id", getattr(tokenizer, "eos_id", 2) or 2))
        self.text_loss_weight = float(cfg_get(cfg, "text_loss_weight", 1.0))
        # optional second output channel: the recognised text of the user, frame aligned like the agent channel
        self.predict_user_text = bool(cfg_get(cfg, "predict_user_text", False))
        if self.predict_user_text and type(self) is DuplexSTTModel:
            H, V = self.llm.config.hidden_size, self.llm.config.vocab_size
            self.embed_asr_tokens = nn.Embedding(V, H)
            self.asr_head = nn.Linear(H, V, bias=False)
            self.asr_loss_weight = float(cfg_get(cfg, "asr_loss_weight", 1.0))
        else:
            self.predict_user_text = False
        self._duplex_ready = True
        if not self._is_model_being_restored and any(cfg_get(cfg, k, None) for k in ("pretrained_s2s_model", "pretrained_perception_from_s2s", "init_from_checkpoint")):
            from .pretrained import maybe_load_pretrained_models

            if type(self) is DuplexSTTModel:                          # subclasses call it after they have added their own layers
                maybe_load_pretrained_models(self)
        if type(self) is DuplexSTTModel and not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if getattr(self, "_duplex_ready", False):                    # the base constructor calls this before the layers exist
            super()._setup_dataloaders_from_cfg()

    @property
    def streaming_inference(self):
        """The frame-synchronous engine (prompts, forced turn taking, chunk-by-chunk feeding)."""
        from .duplex_streaming import DuplexSTTStreamingInference

        return DuplexSTTStreamingInference(self)

    def _loader(self, c):
        from .duplex_data import build_duplex_dataloader

        rank = self.global_rank if self._trainer is not None else 0
        ws = self.world_size if self._trainer is not None else 1
        return build_duplex_dataloader(c, self.tokenizer if self.tokenizer is not None else _IdTokenizer(), float(self.perception.token_equivalent_duration),
                                       self.text_bos_id, self.text_eos_id, self.text_pad_id, num_codebooks=int(getattr(self, "_num_codebooks", 0) or 0),
                                       codebook_size=int(getattr(self, "_codebook_size", 16) or 16), rank=rank, world_size=ws)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        with torch.no_grad():
            l = self._losses(batch)
        return {"val_loss": l["loss"].detach()}

    # ------------------------------------------------------------------ channels
    def _frame_inputs(self, source_emb: torch.Tensor, prev_text: torch.Tensor, prev_codes: Optional[torch.Tensor] = None,
                      prev_asr: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = source_emb + self.embed_tokens(prev_text).to(source_emb.dtype)
        if self.predict_user_text and prev_asr is not None:
            x = x + self.embed_asr_tokens(prev_asr).to(source_emb.dtype)
        return x

    def _heads(self, hidden: torch.Tensor) -> Dict[str, torch.Tensor]:
        out = {"text_logits": self.llm.lm_head(hidden)}
        if self.predict_user_text:
            out["asr_logits"] = self.asr_head(hidden)
        return out

    def forward(self, input_embeds: torch.Tensor, cache=None) -> Dict[str, Any]:
        out = self.llm(inputs_embeds=input_embeds, cache=cache, return_hidden=True)
        ans = self._heads(out["hidden_states"])
        if cache is not None:
            ans["cache"] = out["cache"]
        return ans

    def prepare_inputs(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """batch: ``source_audio`` [B, S], ``source_audio_lens`` [B], ``target_tokens`` [B, T] frame-aligned text channel
        (``target_codes`` [B, T, K] in the speech-to-speech model).  Inputs at frame t carry the targets of frame t-1."""
        emb, emb_len = self.perception(input_signal=batch["source_audio"], input_signal_length=batch["source_audio_lens"])
        T = min(emb.shape[1], batch["target_tokens"].shape[1])
        emb, tgt = emb[:, :T], batch["target_tokens"][:, :T].long()
        prev = torch.cat([torch.full_like(tgt[:, :1], self.text_pad_id), tgt[:, :-1]], dim=1)
        mask = torch.arange(T, device=emb.device)[None, :] < emb_len.clamp(max=T)[:, None]
        out = {"emb": emb, "prev_text": prev, "text_labels": tgt, "mask": mask, "T": T}
        if self.predict_user_text and "source_tokens" in batch:
            src = batch["source_tokens"][:, :T].long()
            out["asr_labels"] = src
            out["prev_asr"] = torch.cat([torch.full_like(src[:, :1], self.text_pad_id), src[:, :-1]], dim=1)
        return out

    def _losses(self, batch) -> Dict[str, torch.Tensor]:
        inp = self.prepare_inputs(batch)
        if self.predict_user_text:
            out = self(self._frame_inputs(inp["emb"], inp["prev_text"], inp.get("prev_codes"), inp.get("prev_asr")))
        else:
            out = self(self._frame_inputs(inp["emb"], inp["prev_text"], inp.get("prev_codes")))
        m = inp["mask"]
        text = F.cross_entropy(out["text_logits"][m].float(), inp["text_labels"][m])
        res = {"text_loss": text, "loss": self.text_loss_weight * text, "_out": out, "_inp": inp}
        if self.predict_user_text and "asr_labels" in inp:
            asr = F.cross_entropy(out["asr_logits"][m].float(), inp["asr_labels"][m])
            res["asr_loss"] = asr
            res["loss"] = res["loss"] + self.asr_loss_weight * asr
        return res

    def training_step(self, batch, batch_idx):
        l = self._losses(batch)
        self.log_dict({"train_loss": l["loss"].detach(), "text_loss": l["text_loss"].detach()})
        return {"loss": l["loss"]}

    @torch.no_grad()
    def offline_inference(self, source_audio: torch.Tensor, source_audio_lens: torch.Tensor) -> Dict[str, Any]:
        """Frame-by-frame greedy decoding with a KV cache: the agent's text channel for every input frame."""
        self.eval()
        emb, emb_len = self.perception(input_signal=source_audio, input_signal_length=source_audio_lens)
        B, T, _ = emb.shape
        cache = [dict() for _ in self.llm.model.layers]
        prev = torch.full((B, 1), self.text_pad_id, dtype=torch.long, device=emb.device)
        prev_codes = self._initial_codes(B, emb.device)
        tokens, codes = [], []
        for t in range(T):
            out = self(self._frame_inputs(emb[:, t:t + 1], prev, prev_codes), cache=cache)
            prev = out["text_logits"][:, -1].argmax(-1, keepdim=True)
            tokens.append(prev)
            if "audio_logits" in out:
                prev_codes = out["audio_logits"][:, -1:].argmax(-1)
                codes.append(prev_codes)
        tokens = torch.cat(tokens, dim=1)
        res = {"tokens": tokens, "lengths": emb_len, "text": self._tokens_to_text(tokens, emb_len)}
        if codes:
            res["codes"] = torch.cat(codes, dim=1)
        return res

    def _initial_codes(self, B, device):
        return None

    def _tokens_to_text(self, tokens: torch.Tensor, lens: torch.Tensor) -> List[str]:
        out = []
        for b in range(tokens.shape[0]):
            ids = [t for t in tokens[b, : int(lens[b])].tolist() if t not in (self.text_pad_id, self.text_bos_id, self.text_eos_id)]
            out.append(self.tokenizer.ids_to_text(ids) if self.tokenizer is not None else " ".join(map(str, ids)))
        return out


class DuplexS2SModel(DuplexSTTModel):
    def __init__(self, cfg: DictConfig, trainer=None, llm=None, tokenizer=None, perception=None, audio_codec=None):
        super().__init__(cfg, trainer, llm, tokenizer, perception)
        cfg = self._cfg
        if audio_codec is None and cfg_get(cfg, "audio_codec", None) is not None:
            from ..tts.audio_codec import AudioCodecModel

            audio_codec = AudioCodecModel(cfg.audio_codec)
        self.audio_codec = audio_codec
        if audio_codec is not None:
            for p in audio_codec.parameters():
                p.requires_grad_(False)
            q = audio_codec.vector_quantizer
            self._codebook_size = int(cfg_get(cfg, "codebook_size", getattr(q, "codebook_size_per_group", None) or q.codebook_size))
            self._num_codebooks = int(cfg_get(cfg, "num_codebooks", getattr(q, "num_groups", 1)))
        else:
            self._codebook_size, self._num_codebooks = int(cfg.codebook_size), int(cfg.num_codebooks)
        H = self.llm.config.hidden_size
        self.embed_audio_tokens = nn.ModuleList([nn.Embedding(self.speech_vocab_size, H) for _ in range(self._num_codebooks)])
        self.audio_head = nn.Linear(H, self.speech_vocab_size * self._num_codebooks)
        self.audio_loss_weight = float(cfg_get(cfg, "audio_loss_weight", 1.0))
        if not self._is_model_being_restored and any(cfg_get(cfg, k, None) for k in ("pretrained_s2s_model", "pretrained_perception_from_s2s", "init_from_checkpoint")):
            from .pretrained import maybe_load_pretrained_models

            maybe_load_pretrained_models(self)
        if type(self) is DuplexS2SModel and not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    speech_vocab_size = property(lambda self: self._codebook_size + 3)
    speech_bos_id = property(lambda self: self._codebook_size)
    speech_eos_id = property(lambda self: self._codebook_size + 1)
    speech_delay_id = property(lambda self: self._codebook_size + 2)

    def _frame_inputs(self, source_emb, prev_text, prev_codes=None):
        x = super()._frame_inputs(source_emb, prev_text)
        if prev_codes is not None:
            for k, table in enumerate(self.embed_audio_tokens):
                x = x + table(prev_codes[..., k]).to(x.dtype)
        return x

    def _heads(self, hidden):
        B, T, _ = hidden.shape
        return {"text_logits": self.llm.lm_head(hidden), "audio_logits": self.audio_head(hidden).view(B, T, self._num_codebooks, self.speech_vocab_size)}

    def _initial_codes(self, B, device):
        return torch.full((B, 1, self._num_codebooks), self.speech_delay_id, dtype=torch.long, device=device)

    def prepare_inputs(self, batch):
        inp = super().prepare_inputs(batch)
        T = inp["T"]
        if "target_codes" in batch:
            codes = batch["target_codes"][:, :T].long()
        else:
            with torch.no_grad():
                c, _ = self.audio_codec.encode(batch["target_audio"], batch["target_audio_lens"])      # [B, K, T_codec]
            codes = c.transpose(1, 2)[:, :T]
            if codes.shape[1] < T:
                codes = F.pad(codes, (0, 0, 0, T - codes.shape[1]), value=self.speech_eos_id)
        inp["prev_codes"] = torch.cat([self._initial_codes(codes.shape[0], codes.device), codes[:, :-1]], dim=1)
        inp["code_labels"] = codes
        return inp

    def _losses(self, batch):
        l = super()._losses(batch)
        out, inp = l["_out"], l["_inp"]
        m = inp["mask"]
        audio = F.cross_entropy(out["audio_logits"][m].float().reshape(-1, self.speech_vocab_size), inp["code_labels"][m].reshape(-1))
        l["audio_loss"] = audio
        l["loss"] = l["loss"] + self.audio_loss_weight * audio
        return l

    def training_step(self, batch, batch_idx):
        l = self._losses(batch)
        self.log_dict({"train_loss": l["loss"].detach(), "text_loss": l["text_loss"].detach(), "audio_loss": l["audio_loss"].detach()})
        return {"loss": l["loss"]}

    @torch.no_grad()
    def offline_inference(self, source_audio, source_audio_lens, decode_audio: bool = True):
        res = super().offline_inference(source_audio, source_audio_lens)
        if decode_audio and self.audio_codec is not None and "codes" in res:
            codes = res["codes"].clamp(max=self._codebook_size - 1).transpose(1, 2)                        # control codes -> valid indices
            audio, audio_len = self.audio_codec.decode(codes, res["lengths"].clamp(max=codes.shape[2]))
            res["audio"], res["audio_len"] = audio, audio_len
        return res


class SALMWithAsrDecoder(SALM):
    """SALM that also reads the hypothesis of an ASR decoder.  With ``perception._target_`` =
    ``AudioTranscriptionPerceptionModule`` (a complete ASR model inside the perception module) every audio placeholder is replaced
    by ``audio embeddings + embeddings of ">> <hypothesis> <<"`` tokenised with the LLM's tokenizer, so the LLM can copy, correct
    or ignore the recogniser's words; ``asr_transcript_drop_prob`` blanks the hypothesis of a training example now and then so the
    model keeps listening (reference ``speechlm2/models/salm_asr_decoder.py:169-215``).  Independently of that, ``asr_weight`` > 0
    with ``asr_tokens`` in the batch trains an auxiliary CTC head on the perception embeddings."""

    def __init__(self, cfg: DictConfig, trainer=None, llm=None, tokenizer=None):
        super().__init__(cfg, trainer=trainer, llm=llm, tokenizer=tokenizer)
        self.asr_weight = float(cfg_get(self._cfg, "asr_weight", 0.3))
        self.asr_vocab = int(cfg_get(self._cfg, "asr_vocab_size", self.embed_tokens.num_embeddings))
        self.asr_head = nn.Linear(self.llm.config.hidden_size, self.asr_vocab + 1)
        self.asr_transcript_drop_prob = float(cfg_get(self._cfg, "asr_transcript_drop_prob", 0.0))
        self.transcript_template = str(cfg_get(self._cfg, "asr_transcript_template", ">> {} <<"))

    @property
    def reads_asr_hypotheses(self) -> bool:
        return hasattr(self.perception, "transcribe_encoded")

    def transcript_embeddings(self, encoded: torch.Tensor, encoded_len: torch.Tensor) -> Tuple[List[torch.Tensor], List[str]]:
        import random

        hyps = self.perception.transcribe_encoded(encoded, encoded_len)
        texts = []
        for h in hyps:
            t = (h.text if hasattr(h, "text") else str(h)) or ""
            if self.training and self.asr_transcript_drop_prob > 0 and random.random() < self.asr_transcript_drop_prob:
                t = ""
            texts.append(t)
        ids = [torch.as_tensor(self.tokenizer.text_to_ids(self.transcript_template.format(t) if t else self.transcript_template.format("").replace("  ", " ")),
                               dtype=torch.long, device=encoded.device) for t in texts]
        embs = [self.embed_tokens(i) for i in ids]
        return embs, texts

    def prepare_inputs(self, batch):
        if not self.reads_asr_hypotheses:
            return super().prepare_inputs(batch)
        from .. import ops
        from .salm import IGNORE_INDEX, replace_placeholders_and_build_targets

        encoded, encoded_len = self.perception.forward_encoder(batch["audios"], batch["audio_lens"])
        t_embs, texts = self.transcript_embeddings(encoded, encoded_len)
        audio_embs, audio_lens = self.perception(encoded=encoded, encoded_len=encoded_len)
        repl = [torch.cat([e[: int(n)], t.to(e.dtype)], dim=0) for e, n, t in zip(audio_embs, audio_lens, t_embs)]
        ids = batch["input_ids"]
        text = self.embed_tokens(torch.where(ids == self.audio_locator_tag_id, torch.zeros_like(ids), ids))
        cdt = ops.get_compute_dtype()
        if cdt is not None:
            text = text.to(cdt)
        repl = [r.to(text.dtype) for r in repl]
        tgt = torch.where(batch["loss_mask"].bool(), ids, torch.full_like(ids, IGNORE_INDEX))
        emb, tgt, mask = replace_placeholders_and_build_targets(ids, text, self.text_pad_id, self.audio_locator_tag_id, repl, tgt)
        self.last_asr_hypotheses = texts
        return {"input_embeds": emb[:, :-1], "attention_mask": mask[:, :-1], "target_ids": tgt[:, 1:]}

    def asr_loss(self, audio_emb: torch.Tensor, audio_emb_lens: torch.Tensor, transcripts: torch.Tensor, transcript_lens: torch.Tensor) -> torch.Tensor:
        lp = F.log_softmax(self.asr_head(audio_emb.float()), dim=-1).transpose(0, 1)
        return F.ctc_loss(lp, transcripts, audio_emb_lens, transcript_lens, blank=self.asr_vocab, zero_infinity=True)

    def training_step(self, batch, batch_idx):
        out = super().training_step(batch, batch_idx)
        if "asr_tokens" in batch and self.asr_weight > 0:
            emb, emb_len = self.perception(input_signal=batch["audios"], input_signal_length=batch["audio_lens"])
            aux = self.asr_loss(emb, emb_len, batch["asr_tokens"], batch["asr_token_lens"])
            out["loss"] = out["loss"] + self.asr_weight * aux
            self.log_dict({"asr_loss": aux.detach()})
        return out

    @torch.no_grad()
    def transcribe_with_asr_head(self, audios: torch.Tensor, audio_lens: torch.Tensor) -> List[List[int]]:
        emb, emb_len = self.perception(input_signal=audios, input_signal_length=audio_lens)
        best = self.asr_head(emb.float()).argmax(-1)
        out = []
        for b in range(best.shape[0]):
            seq, prev = [], -1
            for t in best[b, : int(emb_len[b])].tolist():
                if t != prev and t != self.asr_vocab:
                    seq.append(t)
                prev = t
            out.append(seq)
        return out



"""SALM: speech-augmented language model (audio perception + decoder-only LLM).

Behaviour follows ``speechlm2/models/salm.py`` of the reference: the token embedding table lives on the model, outside the
LLM (``:77-80``); every ``audio_locator_tag`` placeholder in the token stream is replaced by the audio embeddings of the
corresponding recording and the batch is re-padded on the left (``replace_placeholders_and_build_targets`` ``:570-703``);
training minimises next-token cross entropy over assistant tokens only (``:221-230``); generation feeds the spliced
embeddings to the LLM's KV-cache decoder (``:438-443``); ``configure_model`` applies tensor / sequence parallelism and
parameter sharding (``:449-543``) — here through ``speech_b200.parallel``.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.modelpt import ModelPT
from ..prompts import PromptFormatter
from .llm import CausalLM, LLMConfig
from .lora import apply_lora, freeze_and_subset
from .perception import AudioPerceptionModule

IGNORE_INDEX = -100


def replace_placeholders_and_build_targets(input_ids: torch.Tensor, embeds: torch.Tensor, padding_id: int, placeholder_id: int,
                                           replacements: Sequence[torch.Tensor], target_ids: Optional[torch.Tensor] = None,
                                           left_pad: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """Splice ``replacements[k]`` ([T_k, H]) over the k-th placeholder token (row-major order over the batch).

    Returns ``(embeds [B, L', H], targets [B, L'] or None, attention_mask [B, L'])``; positions covered by audio and padding
    get ``IGNORE_INDEX`` targets; padding tokens of the input are dropped before re-padding."""
    B = input_ids.shape[0]
    rows_e, rows_t = [], []
    k = 0
    for b in range(B):
        ids = input_ids[b]
        keep = ids != padding_id
        pos = (ids == placeholder_id).nonzero().squeeze(-1).tolist()
        segs_e, segs_t = [], []
        start = 0
        for p in pos:
            if p > start:
                m = keep[start:p]
                segs_e.append(embeds[b, start:p][m])
                if target_ids is not None:
                    segs_t.append(target_ids[b, start:p][m])
            if k >= len(replacements):
                raise ValueError("more audio placeholders than audio recordings in the batch")
            r = replacements[k]
            k += 1
            segs_e.append(r.to(embeds.dtype))
            if target_ids is not None:
                segs_t.append(torch.full((r.shape[0],), IGNORE_INDEX, dtype=torch.long, device=ids.device))
            start = p + 1
        m = keep[start:]
        segs_e.append(embeds[b, start:][m])
        if target_ids is not None:
            segs_t.append(target_ids[b, start:][m])
        rows_e.append(torch.cat(segs_e, dim=0))
        rows_t.append(torch.cat(segs_t, dim=0) if target_ids is not None else None)
    if k != len(replacements):
        raise ValueError(f"{len(replacements)} audio recordings but only {k} placeholders in the batch")
    L = max(r.shape[0] for r in rows_e)
    H = embeds.shape[-1]
    out_e = embeds.new_zeros((B, L, H))
    out_m = torch.zeros((B, L), dtype=torch.bool, device=embeds.device)
    out_t = torch.full((B, L), IGNORE_INDEX, dtype=torch.long, device=embeds.device) if target_ids is not None else None
    for b, r in enumerate(rows_e):
        n = r.shape[0]
        sl = slice(L - n, L) if left_pad else slice(0, n)
        out_e[b, sl] = r
        out_m[b, sl] = True
        if out_t is not None:
            out_t[b, sl] = rows_t[b]
    return out_e, out_t, out_m


class SALM(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None, llm: Optional[CausalLM] = None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.audio_locator_tag = cfg_get(cfg, "audio_locator_tag", "<|audioplaceholder|>")
        # ---- tokenizer
        if tokenizer is not None:
            self.tokenizer = tokenizer
        else:
            from ..tokenizers import AutoTokenizer, build_tokenizer

            tcfg = cfg_get(cfg, "tokenizer", None)
            self.tokenizer = build_tokenizer(tcfg) if tcfg is not None else AutoTokenizer(cfg.pretrained_llm, use_fast=True)
        if hasattr(self.tokenizer, "add_special_tokens"):
            self.tokenizer.add_special_tokens({"additional_special_tokens": [self.audio_locator_tag]}
                                              if "AutoTokenizer" in type(self.tokenizer).__name__ else [self.audio_locator_tag])
        # ---- LLM
        if llm is not None:
            self.llm = llm
        elif cfg_get(cfg, "llm", None) is not None:
            self.llm = CausalLM.from_config(dict(cfg.llm))
        else:
            self.llm = CausalLM.from_pretrained(cfg.pretrained_llm, load_weights=cfg_get(cfg, "pretrained_weights", True))
        vocab = max(self.llm.config.vocab_size, int(getattr(self.tokenizer, "vocab_size", 0)))
        # the embedding table is owned by the model so that sharding / parallel plans of the LLM blocks never see it
        emb = self.llm.model.embed_tokens
        if vocab > emb.num_embeddings:
            new = nn.Embedding(vocab, emb.embedding_dim)
            with torch.no_grad():
                new.weight[: emb.num_embeddings] = emb.weight
                new.weight[emb.num_embeddings:] = emb.weight.mean(0, keepdim=True)
            tied = self.llm.lm_head.weight is emb.weight
            emb = new
            if tied:
                self.llm.lm_head.weight = emb.weight
            else:
                head = nn.Linear(emb.embedding_dim, vocab, bias=False)
                with torch.no_grad():
                    head.weight[: self.llm.lm_head.weight.shape[0]] = self.llm.lm_head.weight
                self.llm.lm_head.weight = head.weight
            self.llm.config.vocab_size = vocab
        self.embed_tokens = emb
        self.llm.model.embed_tokens = None
        # ---- perception
        pcfg = cfg.perception
        with open_dict(pcfg):
            pcfg.output_dim = self.llm.config.hidden_size
        if cfg_get(cfg, "pretrained_asr", None) and cfg_get(pcfg, "encoder", None) is None:
            from ..models.asr_model import ASRModel

            asr = ASRModel.restore_from(cfg.pretrained_asr)
            self.perception = AudioPerceptionModule(pcfg, preprocessor=asr.preprocessor, encoder=asr.encoder)
        elif cfg_get(pcfg, "asr", None) is not None or "Transcription" in str(cfg_get(pcfg, "_target_", "")):
            from .perception import AudioTranscriptionPerceptionModule

            # a complete ASR model inside the perception module: its decoder's hypotheses can be read by the LLM
            self.perception = AudioTranscriptionPerceptionModule(pcfg, asr=cfg_get(pcfg, "asr", None) or cfg_get(cfg, "pretrained_asr", None))
        else:
            self.perception = AudioPerceptionModule(pcfg)
        if cfg_get(cfg, "lora", None) is not None:
            apply_lora(self.llm, **{k: v for k, v in dict(cfg.lora).items() if k != "task_type"})
            for n, p in self.llm.named_parameters():       # with adapters the backbone itself stays frozen
                if ".lora_" not in n:
                    p.requires_grad_(False)
        freeze_and_subset(self.named_parameters(), cfg_get(cfg, "freeze_params", None), cfg_get(cfg, "prevent_freeze_params", None))
        self._prompt = None
        if type(self).__name__ == "SALM" and not self._is_model_being_restored and any(
                cfg_get(cfg, k, None) for k in ("pretrained_s2s_model", "pretrained_perception_from_s2s", "init_from_checkpoint")):
            from .pretrained import maybe_load_pretrained_models

            maybe_load_pretrained_models(self)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "perception"):
            return
        super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ ids
    @property
    def audio_locator_tag_id(self) -> int:
        return int(self.tokenizer.token_to_id(self.audio_locator_tag))

    @property
    def text_pad_id(self) -> int:
        pad = getattr(self.tokenizer, "pad_id", None)
        pad = pad() if callable(pad) else pad
        if pad is None or pad < 0:
            pad = getattr(self.tokenizer, "unk_id", 0)
            pad = pad() if callable(pad) else pad
        return int(pad if pad is not None else 0)

    @property
    def text_eos_id(self) -> int:
        e = getattr(self.tokenizer, "eos_id", None)
        e = e() if callable(e) else e
        return int(e) if e is not None else -1

    def prompt_formatter(self) -> PromptFormatter:
        if self._prompt is None:
            self._prompt = PromptFormatter.resolve(cfg_get(self._cfg, "prompt_format", "plain"))(self.tokenizer)
        return self._prompt

    # ------------------------------------------------------------------ data
    def _loader(self, config):
        if config is None:
            return None
        from .data import build_salm_dataloader

        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        return build_salm_dataloader(config, self.tokenizer, self.prompt_formatter(), self.audio_locator_tag, self.text_pad_id,
                                     rank, ws)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def setup_test_data(self, c):
        self._test_dl = self._loader(c)

    # ------------------------------------------------------------------ forward
    def forward(self, input_embeds: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, cache=None) -> Dict[str, Any]:
        return self.llm(inputs_embeds=input_embeds, attention_mask=attention_mask, cache=cache)

    def prepare_inputs(self, batch: Dict[str, torch.Tensor]):
        """Audio → embeddings, splice over placeholders, shift for next-token prediction."""
        audio_embs, audio_lens = self.perception(input_signal=batch["audios"], input_signal_length=batch["audio_lens"])
        repl = [e[: int(n)] for e, n in zip(audio_embs, audio_lens)]
        ids = batch["input_ids"]
        text = self.embed_tokens(torch.where(ids == self.audio_locator_tag_id, torch.zeros_like(ids), ids))
        cdt = ops.get_compute_dtype()
        if cdt is not None:
            text = text.to(cdt)
        tgt = torch.where(batch["loss_mask"].bool(), ids, torch.full_like(ids, IGNORE_INDEX))
        emb, tgt, mask = replace_placeholders_and_build_targets(ids, text, self.text_pad_id, self.audio_locator_tag_id, repl, tgt)
        return {"input_embeds": emb[:, :-1], "attention_mask": mask[:, :-1], "target_ids": tgt[:, 1:]}

    def _loss(self, batch):
        inp = self.prepare_inputs(batch)
        out = self.forward(inp["input_embeds"], inp["attention_mask"])
        logits = out["logits"].float()
        tgt = inp["target_ids"]
        n = (tgt != IGNORE_INDEX).sum().clamp(min=1)
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1), ignore_index=IGNORE_INDEX, reduction="sum") / n
        return loss, n, inp

    def training_step(self, batch, batch_idx):
        loss, n, inp = self._loss(batch)
        B, T = inp["input_embeds"].shape[:2]
        self.log_dict({"train_loss": loss.detach(), "learning_rate": 0.0, "batch_size": float(B), "sequence_length": float(T),
                       "num_frames": float(n), "padding_ratio": float(1 - inp["attention_mask"].float().mean())})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        loss, n, _ = self._loss(batch)
        return {"val_loss": loss}

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: Any, audios: Optional[torch.Tensor] = None, audio_lens: Optional[torch.Tensor] = None,
                 max_new_tokens: int = 64, **gen_kw) -> torch.Tensor:
        """``prompts``: token ids [B, L] containing placeholders, or a list of dialogs (lists of ``{"role", "content"}``
        turns; ``content`` may contain the audio locator tag).  Returns generated ids [B, <= max_new_tokens]."""
        if not torch.is_tensor(prompts):
            fm = self.prompt_formatter()
            enc = [fm.encode_dialog([{"role": t["role"], "slots": {"message": t["content"]}} for t in d])["input_ids"] for d in prompts]
            L = max(e.numel() for e in enc)
            prompts = torch.full((len(enc), L), self.text_pad_id, dtype=torch.long)
            for i, e in enumerate(enc):
                prompts[i, L - e.numel():] = e
        ids = prompts.to(self.device)
        text = self.embed_tokens(torch.where(ids == self.audio_locator_tag_id, torch.zeros_like(ids), ids))
        repl = []
        if audios is not None:
            embs, lens = self.perception(input_signal=audios.to(self.device), input_signal_length=audio_lens.to(self.device))
            repl = [e[: int(n)] for e, n in zip(embs, lens)]
            text = text.to(embs.dtype)
        emb, _, mask = replace_placeholders_and_build_targets(ids, text, self.text_pad_id, self.audio_locator_tag_id, repl, None)
        return self.llm.generate(inputs_embeds=emb, attention_mask=mask.long(), max_new_tokens=max_new_tokens,
                                 eos_token_id=gen_kw.pop("eos_token_id", self.text_eos_id if self.text_eos_id >= 0 else None),
                                 pad_token_id=self.text_pad_id, embed_fn=self.embed_tokens, **gen_kw)

    # ------------------------------------------------------------------ parallelism
    def configure_model(self, device_mesh=None) -> None:
        """Apply tensor parallelism to the LLM blocks and shard parameters over the data-parallel group
        (reference ``salm.py:449-543``); ``device_mesh`` is a ``speech_b200.parallel.mesh.DeviceMesh``."""
        if device_mesh is None:
            return
        from ..parallel.tp import apply_tensor_parallel_llm

        if device_mesh.size("tp") > 1:
            apply_tensor_parallel_llm(self.llm, device_mesh.group("tp"))
        self._device_mesh = device_mesh

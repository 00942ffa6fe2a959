"""MagpieTTS: text → audio-codec tokens with an encoder-decoder transformer, decoded to a waveform by a frozen codec.

Structure (reference ``tts/models/magpietts.py``): text embedding + non-causal text encoder; causal decoder with
cross-attention over the text (optionally with a beta-binomial alignment prior and a CTC forward-sum alignment loss on
selected cross-attention heads); audio frames enter as the sum of one embedding per codebook (times ``frame_stacking_factor``
stacked frames) and leave through ``final_proj: d_model → codebooks · stack · tokens`` (``:524-530``); an optional *local
transformer* refines the codebooks of one step autoregressively (``:532-570``); classifier-free guidance by dropping the
text condition during training and mixing conditional / unconditional logits at inference; KV-cache autoregressive
``infer_batch`` (``:2856``) and ``do_tts`` (``:3711``).  Voice context (``model_type``: extra cross-attention memory through a
context encoder, or a decoder prefix), an attention prior that keeps inference monotonic, and chunked long-form synthesis with
state carried between chunks (``:4380``) are part of the model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict
from ..core.modelpt import ModelPT
from .audio_codec import AudioCodecModel
from .transformer_2501 import Transformer


def beta_binomial_prior(text_len: int, audio_len: int, scaling: float = 1.0) -> torch.Tensor:
    """[audio_len, text_len]: row ``t`` is BetaBinomial(n = text_len - 1, a = s·(t+1), b = s·(audio_len - t))."""
    k = torch.arange(text_len, dtype=torch.float64)
    n = float(text_len - 1)
    out = []
    for t in range(1, audio_len + 1):
        a, b = scaling * t, scaling * (audio_len + 1 - t)
        logp = (torch.lgamma(torch.tensor(n + 1)) - torch.lgamma(k + 1) - torch.lgamma(n - k + 1)
                + torch.lgamma(k + a) + torch.lgamma(n - k + b) - torch.lgamma(torch.tensor(n + a + b))
                - (torch.lgamma(torch.tensor(a)) + torch.lgamma(torch.tensor(b)) - torch.lgamma(torch.tensor(a + b))))
        out.append(logp.exp())
    return torch.stack(out).float()


class ForwardSumLoss(nn.Module):
    """CTC over attention: the text positions are the labels 1..T_text, a constant blank column is prepended."""

    def __init__(self, blank_logprob: float = -1.0):
        super().__init__()
        self.blank_logprob = blank_logprob

    def forward(self, attn_logprob: torch.Tensor, in_lens: torch.Tensor, out_lens: torch.Tensor) -> torch.Tensor:
        """attn_logprob [B, T_audio, T_text] (log-probabilities); in_lens = text lengths, out_lens = audio lengths."""
        B = attn_logprob.shape[0]
        x = F.pad(attn_logprob.float(), (1, 0), value=self.blank_logprob)
        total = attn_logprob.new_zeros((), dtype=torch.float32)
        for b in range(B):
            Tt, Ta = int(in_lens[b]), int(out_lens[b])
            lp = torch.log_softmax(x[b, :Ta, : Tt + 1], dim=-1).unsqueeze(1)
            tgt = torch.arange(1, Tt + 1).unsqueeze(0)
            total = total + F.ctc_loss(lp, tgt, torch.tensor([Ta]), torch.tensor([Tt]), blank=0, zero_infinity=True)
        return total / B


@dataclass
class LongFormState:
    """What a long-form synthesis run carries from one text chunk to the next."""

    context_codes: Optional[torch.Tensor] = None          # stacked codes of the voice context [1, C·S, Tc]
    context_len: Optional[torch.Tensor] = None
    chunks_done: int = 0
    text_history: List[str] = field(default_factory=list)


def split_text_for_tts(transcript: str, max_chars: int = 200) -> List[str]:
    """Sentences are kept whole where possible and merged up to ``max_chars``; a single sentence longer than that is split at
    commas / semicolons, then at spaces."""
    import re

    def pieces(s: str) -> List[str]:
        if len(s) <= max_chars:
            return [s]
        parts = [p.strip() for p in re.split(r"(?<=[,;:])\s+", s) if p.strip()]
        if len(parts) == 1:
            words, cur, out = s.split(), "", []
            for w in words:
                if cur and len(cur) + len(w) + 1 > max_chars:
                    out.append(cur)
                    cur = w
                else:
                    cur = (cur + " " + w).strip()
            return out + ([cur] if cur else [])
        return [q for p in parts for q in pieces(p)]

    sents = [q for s in re.split(r"(?<=[.!?])\s+", transcript) if s.strip() for q in pieces(s.strip())]
    chunks, cur = [], ""
    for s in sents:
        if cur and len(cur) + len(s) + 1 > max_chars:
            chunks.append(cur)
            cur = s
        else:
            cur = (cur + " " + s).strip()
    return chunks + ([cur] if cur else [])


class MagpieTTSModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None, codec: Optional[AudioCodecModel] = None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        # ---- codec (frozen)
        if codec is None:
            if cfg_get(cfg, "codecmodel_path", None):
                codec = AudioCodecModel.restore_from(cfg.codecmodel_path)
            else:
                codec = AudioCodecModel(cfg.codec)
        object.__setattr__(self, "_codec", codec)                    # not a sub-module: never trained or check-pointed here
        codec.eval()
        for p in codec.parameters():
            p.requires_grad_(False)
        self.num_audio_codebooks = codec.num_codebooks
        self.codebook_size = codec.codebook_size
        self.audio_bos_id, self.audio_eos_id = self.codebook_size, self.codebook_size + 1
        self.num_all_tokens_per_codebook = self.codebook_size + cfg_get(cfg, "num_special_audio_tokens", 8)
        self.frame_stacking_factor = cfg_get(cfg, "frame_stacking_factor", 1)
        # ---- text
        if tokenizer is None:
            from ..tokenizers import build_tokenizer

            tokenizer = build_tokenizer(cfg.text_tokenizer)
        self.tokenizer = tokenizer
        n_text = int(tokenizer.vocab_size) + 2
        self.text_bos_id, self.text_eos_id = n_text - 2, n_text - 1
        d = cfg_get(cfg, "embedding_dim", 256)
        self.d_model = d
        self.text_embedding = nn.Embedding(n_text, d)
        self.encoder = Transformer(**dict(cfg.encoder))
        self.decoder = Transformer(**dict(cfg.decoder))
        C = self.num_audio_codebooks * self.frame_stacking_factor
        self.audio_embeddings = nn.ModuleList([nn.Embedding(self.num_all_tokens_per_codebook, d) for _ in range(C)])
        self.final_proj = nn.Linear(d, C * self.num_all_tokens_per_codebook)
        # ---- conditioning on a context recording (voice cloning).  ``model_type``:
        #   "text_only"                 no context;
        #   "multi_encoder_context_tts" context codes -> context encoder -> extra cross-attention memory next to the text;
        #   "decoder_context_tts"       context code embeddings are a prefix of the decoder input;
        #   "decoder_ce"                as above, but the prefix first goes through the context encoder.
        # (reference ``tts/models/magpietts.py``: ``prepare_context_tensors`` and the ``model_type`` switch)
        self.model_type = str(cfg_get(cfg, "model_type", "text_only"))
        if self.model_type not in ("text_only", "multi_encoder_context_tts", "decoder_context_tts", "decoder_ce"):
            raise ValueError(f"unknown model_type '{self.model_type}'")
        if self.model_type in ("multi_encoder_context_tts", "decoder_ce"):
            self.context_encoder = Transformer(**dict(cfg.context_encoder))
        self.context_duration_min = float(cfg_get(cfg, "context_duration_min", 3.0))
        self.context_duration_max = float(cfg_get(cfg, "context_duration_max", 10.0))
        # ---- optional local transformer over the codebooks of one step
        self.local_transformer_type = str(cfg_get(cfg, "local_transformer_type", "none")).lower()
        if self.local_transformer_type != "none":
            dl = cfg_get(cfg, "local_transformer_hidden_dim", d)
            self.local_transformer_in_projection = nn.Linear(d, dl)
            self.local_transformer = Transformer(n_layers=cfg_get(cfg, "local_transformer_n_layers", 1), d_model=dl, d_ffn=dl * 4,
                                                 sa_n_heads=cfg_get(cfg, "local_transformer_n_heads", 1), kernel_size=1,
                                                 is_causal=self.local_transformer_type == "autoregressive",
                                                 max_length_causal_mask=C + 2, use_learnable_pos_emb=True)
            self.local_transformer_audio_embeddings = nn.ModuleList([nn.Embedding(self.num_all_tokens_per_codebook, dl) for _ in range(C)])
            self.local_transformer_out_projections = nn.ModuleList([nn.Linear(dl, self.num_all_tokens_per_codebook) for _ in range(C)])
        # ---- losses / regularisers
        self.alignment_loss_scale = cfg_get(cfg, "alignment_loss_scale", 0.0)
        self.alignment_layers = list(cfg_get(cfg, "alignment_decoder_loss_layers", cfg_get(cfg, "prior_layers", [])) or [])
        self.prior_scaling_factor = cfg_get(cfg, "prior_scaling_factor", None)
        self.prior_end_step = cfg_get(cfg, "prior_end_step", 0)
        self.cfg_unconditional_prob = cfg_get(cfg, "cfg_unconditional_prob", 0.0)
        self.alignment_loss = ForwardSumLoss()
        self.moe_loss_scale = cfg_get(cfg, "moe_load_balancing_loss_scale", 0.01)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "final_proj"):
            return
        super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ data: (text ids, text len, audio, audio len)
    def _loader(self, config):
        if config is None:
            return None
        from .data import build_tts_dataloader

        return build_tts_dataloader(config, self.tokenizer, sample_rate=self._codec.sample_rate)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    # ------------------------------------------------------------------ token plumbing
    @torch.no_grad()
    def audio_to_codes(self, audio, audio_len):
        """→ codes [B, C, T+2] with BOS / EOS added, lengths."""
        self._codec.to(audio.device)
        codes, lens = self._codec.encode(audio, audio_len)
        B, C, T = codes.shape
        out = torch.full((B, C, T + 2), self.audio_eos_id, dtype=torch.long, device=codes.device)
        out[:, :, 0] = self.audio_bos_id
        out[:, :, 1:T + 1] = codes
        for b in range(B):
            out[b, :, int(lens[b]) + 1] = self.audio_eos_id
            out[b, :, int(lens[b]) + 2:] = 0
        return out, lens + 2

    @torch.no_grad()
    def codes_to_audio(self, codes, codes_len):
        self._codec.to(codes.device)
        codes = codes.clamp(max=self.codebook_size - 1)
        return self._codec.decode(codes, codes_len)

    def stack_codes(self, codes, lens):
        S = self.frame_stacking_factor
        if S == 1:
            return codes, lens
        B, C, T = codes.shape
        pad = (-T) % S
        codes = F.pad(codes, (0, pad), value=self.audio_eos_id)
        codes = codes.view(B, C, -1, S).permute(0, 1, 3, 2).reshape(B, C * S, -1)
        return codes, torch.div(lens + S - 1, S, rounding_mode="floor")

    def unstack_codes(self, codes, lens):
        S = self.frame_stacking_factor
        if S == 1:
            return codes, lens
        B, CS, T = codes.shape
        C = CS // S
        return codes.view(B, C, S, T).permute(0, 1, 3, 2).reshape(B, C, T * S), lens * S

    def embed_audio_tokens(self, codes):
        """codes [B, C·S, T] → [B, T, d]: mean of the per-codebook embeddings."""
        x = 0.0
        for c, emb in enumerate(self.audio_embeddings):
            x = x + emb(codes[:, c])
        return x / len(self.audio_embeddings)

    def encode_text(self, text, text_len):
        mask = torch.arange(text.shape[1], device=text.device)[None] < text_len[:, None]
        out = self.encoder(self.text_embedding(text), mask)["output"]
        return out, mask

    # ------------------------------------------------------------------ teacher-forced forward
    def _priors(self, text_len, audio_len, Ta, Tt, device):
        if self.prior_scaling_factor is None or (self.prior_end_step and self.global_step >= self.prior_end_step):
            return None
        pri = torch.zeros((len(text_len), Ta, Tt), device=device)
        for b in range(len(text_len)):
            tl, al = int(text_len[b]), int(audio_len[b])
            pri[b, :al, :tl] = beta_binomial_prior(tl, al, self.prior_scaling_factor).to(device)
        return pri

    def prepare_context(self, context_codes: Optional[torch.Tensor], context_codes_len: Optional[torch.Tensor]):
        """Context codes ``[B, C·S, Tc]`` (stacked like the targets) -> ``(embeddings [B, Tc, d], mask [B, Tc])`` after the
        context encoder where the model has one; ``(None, None)`` for text-only models or when no context is given."""
        if self.model_type == "text_only" or context_codes is None:
            return None, None
        emb = self.embed_audio_tokens(context_codes)
        mask = torch.arange(emb.shape[1], device=emb.device)[None] < context_codes_len[:, None]
        if hasattr(self, "context_encoder"):
            emb = self.context_encoder(emb, mask)["output"]
        return emb, mask

    def forward(self, text, text_len, codes, codes_len, drop_condition: bool = False, context_codes=None, context_codes_len=None):
        """Teacher forcing.  codes [B, C·S, T] (stacked, with BOS / EOS).  Returns logits [B, T-1, C·S, N] and the
        cross-attention probabilities of the decoder layers (over the text positions only)."""
        cond, cond_mask = self.encode_text(text, text_len)
        ctx, ctx_mask = self.prepare_context(context_codes, context_codes_len)
        if drop_condition:
            cond = torch.zeros_like(cond)
            ctx = torch.zeros_like(ctx) if ctx is not None else None
        inp, tgt_len = codes[:, :, :-1], codes_len - 1
        x = self.embed_audio_tokens(inp)
        xmask = torch.arange(x.shape[1], device=x.device)[None] < tgt_len[:, None]
        prior = self._priors(text_len, tgt_len, x.shape[1], cond.shape[1], x.device) if self.training else None
        n_prefix = n_mem = 0
        if ctx is not None and self.model_type == "multi_encoder_context_tts":
            n_mem = ctx.shape[1]
            cond, cond_mask = torch.cat([ctx.to(cond.dtype), cond], 1), torch.cat([ctx_mask, cond_mask], 1)
            if prior is not None:                                   # the prior constrains text positions only
                prior = torch.cat([torch.ones(prior.shape[0], prior.shape[1], n_mem, device=prior.device), prior], 2)
        elif ctx is not None:
            n_prefix = ctx.shape[1]
            x, xmask = torch.cat([ctx.to(x.dtype), x], 1), torch.cat([ctx_mask, xmask], 1)
            if prior is not None:
                prior = torch.cat([torch.ones(prior.shape[0], n_prefix, prior.shape[2], device=prior.device), prior], 1)
        priors = [prior if i in self.alignment_layers else None for i in range(len(self.decoder.layers))] if prior is not None else None
        out = self.decoder(x, xmask, cond=cond, cond_mask=cond_mask, attn_prior=priors)
        h = out["output"][:, n_prefix:]
        xmask = xmask[:, n_prefix:]
        out["attn_probabilities"] = [None if a is None else a[:, :, n_prefix:, n_mem:] for a in out["attn_probabilities"]]
        B, T, _ = h.shape
        logits = ops.linear(h, self.final_proj.weight, self.final_proj.bias).float().view(B, T, len(self.audio_embeddings), -1)
        return logits, out["attn_probabilities"], h, xmask

    def local_transformer_logits(self, h: torch.Tensor, target_codes: torch.Tensor) -> torch.Tensor:
        """Teacher-forced local transformer: h [N, d] decoder states, target_codes [N, C] → logits [N, C, V]."""
        x0 = self.local_transformer_in_projection(h).unsqueeze(1)
        embs = [self.local_transformer_audio_embeddings[c](target_codes[:, c]).unsqueeze(1) for c in range(target_codes.shape[1] - 1)]
        seq = torch.cat([x0] + embs, dim=1)
        mask = torch.ones(seq.shape[:2], dtype=torch.bool, device=seq.device)
        out = self.local_transformer(seq, mask)["output"]
        return torch.stack([self.local_transformer_out_projections[c](out[:, c]) for c in range(target_codes.shape[1])], dim=1).float()

    @property
    def local_mask_id(self) -> int:
        """Token that stands for "not decided yet" in the MaskGit local transformer (the last special audio token)."""
        return self.num_all_tokens_per_codebook - 1

    def local_transformer_maskgit_logits(self, h: torch.Tensor, target_codes: torch.Tensor, masked: torch.Tensor) -> torch.Tensor:
        """Bidirectional local transformer: position 0 = decoder state, position 1+c = embedding of codebook c's token, or of
        the mask token where ``masked[:, c]``; logits [N, C, V] for every codebook (reference: ``magpietts.py:532-570``)."""
        C = target_codes.shape[1]
        x0 = self.local_transformer_in_projection(h).unsqueeze(1)
        inp = torch.where(masked, torch.full_like(target_codes, self.local_mask_id), target_codes)
        embs = [self.local_transformer_audio_embeddings[c](inp[:, c]).unsqueeze(1) for c in range(C)]
        seq = torch.cat([x0] + embs, dim=1)
        mask = torch.ones(seq.shape[:2], dtype=torch.bool, device=seq.device)
        out = self.local_transformer(seq, mask)["output"]
        return torch.stack([self.local_transformer_out_projections[c](out[:, 1 + c]) for c in range(C)], dim=1).float()

    def _maskgit_loss(self, h: torch.Tensor, target_codes: torch.Tensor) -> torch.Tensor:
        """Mask a cosine-scheduled random share of every frame's codebooks (at least one) and predict the masked ones."""
        N, C = target_codes.shape
        ratio = torch.cos(torch.rand(N, device=h.device) * math.pi / 2)                     # in (0, 1], more often high
        n_mask = (ratio * C).ceil().clamp(1, C).long()
        order = torch.rand(N, C, device=h.device).argsort(dim=1).argsort(dim=1)
        masked = order < n_mask[:, None]
        lg = self.local_transformer_maskgit_logits(h, target_codes, masked)
        return F.cross_entropy(lg[masked], target_codes[masked])

    @torch.no_grad()
    def _local_maskgit(self, h, temperature, topk, n_steps: int = 3, uncond=None, cfg_scale: float = 1.0):
        """Iterative parallel decoding of one frame: predict all undecided codebooks, keep the most confident ones, repeat."""
        CS = len(self.audio_embeddings)
        N = h.shape[0]
        codes = torch.full((N, CS), self.local_mask_id, dtype=torch.long, device=h.device)
        masked = torch.ones(N, CS, dtype=torch.bool, device=h.device)
        for it in range(n_steps):
            lg = self.local_transformer_maskgit_logits(h, codes, masked)
            if uncond is not None:
                ul = self.local_transformer_maskgit_logits(uncond, codes, masked)
                lg = ul + cfg_scale * (lg - ul)
            lg[..., self.audio_bos_id] = float("-inf")
            lg[..., self.audio_eos_id + 1:] = float("-inf")
            tok = self._sample(lg, temperature, topk)
            conf = torch.softmax(lg, -1).gather(-1, tok.unsqueeze(-1)).squeeze(-1).masked_fill(~masked, float("inf"))
            # number of codebooks still undecided after this round follows the cosine schedule; the last round decides all
            keep_masked = 0 if it == n_steps - 1 else int(math.floor(CS * math.cos(math.pi / 2 * (it + 1) / n_steps)))
            codes = torch.where(masked, tok, codes)
            if keep_masked > 0:
                redo = conf.argsort(dim=1)[:, :keep_masked]                                 # least confident stay undecided
                newmask = torch.zeros_like(masked).scatter(1, redo, True) & masked
            else:
                newmask = torch.zeros_like(masked)
            codes = torch.where(newmask, torch.full_like(codes, self.local_mask_id), codes)
            masked = newmask
        return codes

    def _loss(self, batch):
        text, text_len, audio, audio_len = batch[:4]
        codes, codes_len = self.audio_to_codes(audio, audio_len)
        codes, codes_len = self.stack_codes(codes, codes_len)
        drop = self.training and self.cfg_unconditional_prob > 0 and float(torch.rand(())) < self.cfg_unconditional_prob
        ctx_codes = ctx_len = None
        if self.model_type != "text_only" and len(batch) >= 6 and batch[4] is not None:
            ctx_codes, ctx_len = self.audio_to_codes(batch[4], batch[5])           # (context_audio, context_audio_len)
            ctx_codes, ctx_len = self.stack_codes(ctx_codes, ctx_len)
        logits, attn, h, xmask = self.forward(text, text_len, codes, codes_len, drop_condition=drop, context_codes=ctx_codes,
                                              context_codes_len=ctx_len)
        tgt = codes[:, :, 1:].permute(0, 2, 1)                         # [B, T-1, C·S]
        ce = F.cross_entropy(logits[xmask].reshape(-1, logits.shape[-1]), tgt[xmask].reshape(-1))
        logs = {"codebook_loss": ce.detach()}
        loss = ce
        if self.local_transformer_type != "none":
            if self.local_transformer_type == "maskgit":
                lt_loss = self._maskgit_loss(h[xmask].float(), tgt[xmask])
            else:
                lt = self.local_transformer_logits(h[xmask].float(), tgt[xmask])
                lt_loss = F.cross_entropy(lt.reshape(-1, lt.shape[-1]), tgt[xmask].reshape(-1))
            loss = loss + lt_loss
            logs["local_transformer_loss"] = lt_loss.detach()
        if self.alignment_loss_scale > 0 and not drop and self.alignment_layers:
            al = 0.0
            for i in self.alignment_layers:
                p = attn[i]
                if p is None:
                    continue
                al = al + self.alignment_loss(torch.log(p.float().mean(1) + 1e-8), text_len, codes_len - 1)
            loss = loss + self.alignment_loss_scale * al / max(1, len(self.alignment_layers))
            logs["alignment_loss"] = torch.as_tensor(al).detach()
        for k, v in self.decoder.moe_aux_losses().items():
            if k == "load_balancing_loss":
                loss = loss + self.moe_loss_scale * v
                logs["moe_load_balancing_loss"] = v.detach()
        return loss, logs

    def training_step(self, batch, batch_idx):
        loss, logs = self._loss(batch)
        self.log_dict({"train_loss": loss.detach(), **{f"train_{k}": v for k, v in logs.items()}})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        loss, logs = self._loss(batch)
        return {"val_loss": loss}

    # ------------------------------------------------------------------ inference
    @staticmethod
    def _sample(logits: torch.Tensor, temperature: float, topk: int) -> torch.Tensor:
        if temperature <= 0:
            return logits.argmax(-1)
        lg = logits / temperature
        if topk and topk < lg.shape[-1]:
            kth = lg.topk(topk, dim=-1).values[..., -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        return torch.multinomial(torch.softmax(lg, -1).view(-1, lg.shape[-1]), 1).view(lg.shape[:-1])

    @torch.no_grad()
    def infer_batch(self, text, text_len, max_decoder_steps: int = 500, temperature: float = 0.7, topk: int = 80,
                    use_cfg: bool = False, cfg_scale: float = 2.5, min_generated_frames: int = 4, context_codes=None,
                    context_codes_len=None, attention_prior_strength: float = 0.0, attention_prior_window: int = 4,
                    return_attention: bool = False):
        """Autoregressive decoding with KV caches.  Returns (audio [B, n], audio_len, codes [B, C, T], codes_len).

        ``context_codes`` [B, C·S, Tc] condition the voice (see ``model_type``).  For decoder-prefix models the contexts of a batch
        are cut to the shortest one so that the prefix is dense in the cache.  ``attention_prior_strength`` > 0 keeps the
        cross-attention monotonic at inference: at every step text positions further than ``attention_prior_window`` from the
        position attended at the previous step are down-weighted by that factor (in log space), which prevents skipped or
        repeated words on long inputs; generation of a row also ends once its attention has sat on the last text token for
        ``2 * attention_prior_window`` steps without an end token."""
        self.eval()
        B, dev = text.shape[0], text.device
        cond, cond_mask = self.encode_text(text, text_len)
        n_mem = 0
        prefix = None
        if context_codes is not None and self.model_type != "text_only":
            if self.model_type != "multi_encoder_context_tts":
                keep = int(context_codes_len.min())
                context_codes, context_codes_len = context_codes[:, :, :keep], context_codes_len.clamp(max=keep)
            ctx, ctx_mask = self.prepare_context(context_codes, context_codes_len)
            if self.model_type == "multi_encoder_context_tts":
                n_mem = ctx.shape[1]
                cond, cond_mask = torch.cat([ctx.to(cond.dtype), cond], 1), torch.cat([ctx_mask, cond_mask], 1)
            else:
                prefix = ctx
        if use_cfg:
            cond = torch.cat([cond, torch.zeros_like(cond)], 0)
            cond_mask = torch.cat([cond_mask, cond_mask], 0)
        CS = len(self.audio_embeddings)
        cur = torch.full((B, CS, 1), self.audio_bos_id, dtype=torch.long, device=dev)
        cache = self.decoder.new_cache()
        offset = 0
        if prefix is not None:
            px = torch.cat([prefix, torch.zeros_like(prefix)], 0) if use_cfg else prefix
            self.decoder(px, torch.ones(px.shape[:2], dtype=torch.bool, device=dev), cond=cond, cond_mask=cond_mask, cache=cache)
            offset = prefix.shape[1]
        attended = torch.zeros(B, dtype=torch.long, device=dev)          # text position the alignment currently sits on
        at_end = torch.zeros(B, dtype=torch.long, device=dev)
        attn_trace = []
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        end_step = torch.full((B,), max_decoder_steps, dtype=torch.long, device=dev)
        frames = []
        for step in range(max_decoder_steps):
            x = self.embed_audio_tokens(cur)
            if use_cfg:
                x = torch.cat([x, x], 0)
            xmask = torch.ones(x.shape[:2], dtype=torch.bool, device=dev)
            prior = None
            if attention_prior_strength > 0:
                pos = torch.arange(cond.shape[1] - n_mem, device=dev)[None, :]
                near = (pos >= attended[:, None] - 1) & (pos <= attended[:, None] + attention_prior_window)
                pr = torch.where(near, torch.ones((), device=dev), torch.full((), math.exp(-attention_prior_strength), device=dev))
                pr = torch.cat([torch.ones(B, n_mem, device=dev), pr], 1).unsqueeze(1)          # [B, 1, T_cond]
                prior = torch.cat([pr, torch.ones_like(pr)], 0) if use_cfg else pr
                prior = [prior if (not self.alignment_layers or i in self.alignment_layers) else None for i in range(len(self.decoder.layers))]
            dec = self.decoder(x, xmask, cond=cond, cond_mask=cond_mask, cache=cache, position_offset=offset + step, attn_prior=prior)
            h = dec["output"][:, -1]
            probs = [a for i, a in enumerate(dec["attn_probabilities"]) if a is not None and (not self.alignment_layers or i in self.alignment_layers)]
            if probs:
                a = torch.stack([p[:B, :, -1, n_mem:].float().mean(1) for p in probs]).mean(0)   # [B, T_text]
                a = a.masked_fill(~cond_mask[:B, n_mem:], 0.0)
                peak = a.argmax(-1)
                attended = torch.where(peak > attended, torch.minimum(peak, attended + attention_prior_window), attended) \
                    if attention_prior_strength > 0 else peak
                at_end = torch.where(attended >= text_len.to(dev) - 1, at_end + 1, torch.zeros_like(at_end))
                if return_attention:
                    attn_trace.append(a)
            logits = ops.linear(h, self.final_proj.weight, self.final_proj.bias).float().view(h.shape[0], CS, -1)
            if use_cfg:
                logits = logits[B:] + cfg_scale * (logits[:B] - logits[B:])
            if self.local_transformer_type == "autoregressive":
                nxt = self._local_ar(h[:B].float(), temperature, topk, uncond=h[B:].float() if use_cfg else None, cfg_scale=cfg_scale)
            elif self.local_transformer_type == "maskgit":
                nxt = self._local_maskgit(h[:B].float(), temperature, topk, uncond=h[B:].float() if use_cfg else None, cfg_scale=cfg_scale)
                if step < min_generated_frames:
                    nxt = torch.where(nxt == self.audio_eos_id, torch.zeros_like(nxt), nxt)
            else:
                logits[..., self.audio_bos_id] = float("-inf")
                logits[..., self.audio_eos_id + 1:] = float("-inf")
                if step < min_generated_frames:
                    logits[..., self.audio_eos_id] = float("-inf")
                nxt = self._sample(logits, temperature, topk)
            is_eos = (nxt == self.audio_eos_id).any(dim=1)
            if attention_prior_strength > 0:
                is_eos = is_eos | ((at_end >= 2 * attention_prior_window) & (step >= min_generated_frames))
            newly = is_eos & ~done
            end_step = torch.where(newly, torch.full_like(end_step, step), end_step)
            done = done | is_eos
            frames.append(nxt)
            cur = nxt.unsqueeze(-1)
            if bool(done.all()):
                break
        codes = torch.stack(frames, dim=-1)                               # [B, C·S, T]
        lens = end_step.clamp(max=codes.shape[-1])
        codes, lens = self.unstack_codes(codes, lens)
        lens = lens.clamp(min=1)
        audio, audio_len = self.codes_to_audio(codes, lens)
        if return_attention:
            return audio, audio_len, codes, lens, (torch.stack(attn_trace, 1) if attn_trace else None)
        return audio, audio_len, codes, lens

    def _local_ar(self, h, temperature, topk, uncond=None, cfg_scale=1.0):
        CS = len(self.audio_embeddings)
        seq = self.local_transformer_in_projection(h).unsqueeze(1)
        useq = self.local_transformer_in_projection(uncond).unsqueeze(1) if uncond is not None else None
        out = []
        for c in range(CS):
            m = torch.ones(seq.shape[:2], dtype=torch.bool, device=seq.device)
            lg = self.local_transformer_out_projections[c](self.local_transformer(seq, m)["output"][:, -1]).float()
            if useq is not None:
                ul = self.local_transformer_out_projections[c](self.local_transformer(useq, m)["output"][:, -1]).float()
                lg = ul + cfg_scale * (lg - ul)
            lg[..., self.audio_bos_id] = float("-inf")
            lg[..., self.audio_eos_id + 1:] = float("-inf")
            tok = self._sample(lg, temperature, topk)
            out.append(tok)
            e = self.local_transformer_audio_embeddings[c](tok).unsqueeze(1)
            seq = torch.cat([seq, e], 1)
            if useq is not None:
                useq = torch.cat([useq, e], 1)
        return torch.stack(out, dim=1)

    def _generate_speech_with_state(self, transcript, max_chars_per_chunk, context_audio, carry_voice, crossfade_ms, **kw):
        state = LongFormState()
        if context_audio is not None:
            a = context_audio.view(1, -1).to(self.device)
            codes, n = self.audio_to_codes(a, torch.tensor([a.shape[1]], device=self.device))
            state.context_codes, state.context_len = self.stack_codes(codes, n)
        sr = int(getattr(self._codec, "sample_rate", 22050))
        fade = int(sr * crossfade_ms / 1000)
        out = torch.zeros(0, device=self.device)
        for chunk in split_text_for_tts(transcript, max_chars_per_chunk):
            ids = self.tokenize(chunk).unsqueeze(0).to(self.device)
            audio, alen, codes, clen = self.infer_batch(ids, torch.tensor([ids.shape[1]], device=self.device),
                                                        context_codes=state.context_codes, context_codes_len=state.context_len, **kw)
            piece = audio[0, : int(alen[0])]
            if state.context_codes is None and carry_voice:
                # the first chunk fixes the voice of the rest (bounded by the longest context the model was trained with)
                max_frames = max(1, int(self.context_duration_max * sr / max(1, getattr(self._codec, "samples_per_frame", 1024))))
                st, sl = self.stack_codes(codes[:, :, :max_frames], clen.clamp(max=max_frames))
                state.context_codes, state.context_len = st, sl
            state.chunks_done += 1
            state.text_history.append(chunk)
            if out.numel() and fade > 0 and piece.numel() > fade and out.numel() > fade:
                ramp = torch.linspace(0, 1, fade, device=piece.device)
                out = torch.cat([out[:-fade], out[-fade:] * (1 - ramp) + piece[:fade] * ramp, piece[fade:]])
            else:
                out = torch.cat([out, piece])
        self.last_long_form_state = state
        return out

    def tokenize(self, transcript: str) -> torch.Tensor:
        ids = [self.text_bos_id] + list(self.tokenizer.text_to_ids(transcript)) + [self.text_eos_id]
        return torch.tensor(ids, dtype=torch.long)

    @torch.no_grad()
    def do_tts(self, transcript: str, **kw) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = self.tokenize(transcript).unsqueeze(0).to(self.device)
        audio, alen, _, _ = self.infer_batch(ids, torch.tensor([ids.shape[1]], device=self.device), **kw)
        return audio, alen

    @torch.no_grad()
    def generate_speech(self, transcript: str, max_chars_per_chunk: int = 200, context_audio: Optional[torch.Tensor] = None,
                        carry_voice: bool = True, crossfade_ms: float = 20.0, **kw) -> torch.Tensor:
        """Long-form synthesis: the text is split at sentence boundaries into chunks that the decoder handles comfortably and
        synthesised chunk by chunk; the state that crosses chunks (:class:`LongFormState`) is the voice context: the caller's
        ``context_audio`` where given, otherwise (``carry_voice``) the codes of the first generated chunk, so that every chunk
        is spoken by the same voice.  Chunks are joined with a short cross-fade."""
        import re

        if self.model_type != "text_only":
            return self._generate_speech_with_state(transcript, max_chars_per_chunk, context_audio, carry_voice, crossfade_ms, **kw)

        sents = [s.strip() for s in re.split(r"(?<=[.!?])\s+", transcript) if s.strip()]
        chunks, cur = [], ""
        for s in sents:
            if cur and len(cur) + len(s) + 1 > max_chars_per_chunk:
                chunks.append(cur)
                cur = s
            else:
                cur = (cur + " " + s).strip()
        if cur:
            chunks.append(cur)
        outs = []
        for c in chunks:
            a, n = self.do_tts(c, **kw)
            outs.append(a[0, : int(n[0])])
        return torch.cat(outs) if outs else torch.zeros(0)

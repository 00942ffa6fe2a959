"""Streaming text-to-speech on continuous codec latents (EAR-TTS), and the duplex models built on it.

* ``ResidualVQ`` — residual vector quantiser: ``K`` codebooks of ``N`` entries over a ``latent``-dimensional space; the embedding
  of a code tuple is the sum of its codebook entries ("depth sum"), and ``encode`` quantises a continuous latent greedily, one
  codebook after the other, on the residual.
* ``MoGHead`` — mixture-of-Gaussians output head: an MLP stack, then mixture logits, per-component means (low-rank: a shared
  full-rank mean plus ``low_mat[k] @ z_k``) and one shared log standard deviation.  ``nll`` is the training loss of a target
  latent; ``infer`` samples a component (top-k / top-p, temperature) and, optionally, noise around its mean.
* ``GatedProjectedSumRMSNorm`` — fuses the audio-frame embedding and the text embedding of a frame with a learned sigmoid gate.
* ``EARTTSModel`` — causal transformer backbone over frames.  Input at frame ``t`` = embedding of the latent of frame ``t-1``
  (depth sum of its codes, with random codebook-depth masking during training) fused with the embedding of the text token
  scheduled at frame ``t``; output = MoG over the latent of frame ``t``, which is re-quantised by the RVQ to give the codes fed
  back at ``t+1``.  Classifier-free guidance: the text channel is replaced by a learned null embedding with probability
  ``cfg_dropout`` in training, and ``generate`` mixes conditional and unconditional means with ``guidance_scale``.
* ``DuplexEARTTS`` — the trainable model around it (frame-aligned text channel + target codes -> MoG loss), with
  ``offline_inference`` that speaks a frame-aligned token stream.
* ``DuplexS2SSpeechDecoderModel`` — duplex speech-to-speech in which the LLM predicts only the text channel and a separate
  causal speech decoder (a small transformer over LLM hidden states + previous codes) predicts the audio codes.
* ``NemotronVoiceChat`` — full-duplex voice chat: a ``DuplexSTTModel`` listens and writes the agent's text channel frame by
  frame; ``DuplexEARTTS`` speaks it with one frame of delay; both run incrementally with their own caches.

Reference: ``speechlm2/modules/ear_tts_model.py`` (``MoGHead`` ``:397-573``, ``GatedProjectedSumRMSNorm`` ``:888-925``,
``RVQEARTTSModel`` ``:927-1577``, ``depthsum_encoding_step`` ``:375``), ``models/duplex_ear_tts.py``,
``models/duplex_s2s_speech_decoder_model.py``, ``models/nemotron_voicechat.py``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from ..core.modelpt import ModelPT
from .llm import CausalLM, RMSNorm


class ResidualVQ(nn.Module):
    def __init__(self, num_quantizers: int, codebook_size: int, latent_size: int):
        super().__init__()
        self.K, self.N, self.D = int(num_quantizers), int(codebook_size), int(latent_size)
        scale = torch.tensor([0.5 ** k for k in range(self.K)]).view(self.K, 1, 1)          # residual stages shrink
        self.codebooks = nn.Parameter(torch.randn(self.K, self.N, self.D) * scale)

    def embed(self, codes: torch.Tensor, depth: Optional[torch.Tensor] = None) -> torch.Tensor:
        """codes [..., K] -> latent [..., D]; ``depth`` [...] keeps only the first ``depth`` codebooks of each position."""
        parts = torch.stack([self.codebooks[k][codes[..., k]] for k in range(self.K)], dim=-2)   # [..., K, D]
        if depth is not None:
            keep = torch.arange(self.K, device=codes.device) < depth.unsqueeze(-1)
            parts = parts * keep.unsqueeze(-1).to(parts.dtype)
        return parts.sum(dim=-2)

    @torch.no_grad()
    def encode(self, latent: torch.Tensor) -> torch.Tensor:
        """Greedy residual quantisation: latent [..., D] -> codes [..., K]."""
        res = latent.float()
        out = []
        for k in range(self.K):
            cb = self.codebooks[k].float()
            d = (res.unsqueeze(-2) - cb).pow(2).sum(-1)                                      # [..., N]
            idx = d.argmin(-1)
            out.append(idx)
            res = res - cb[idx]
        return torch.stack(out, dim=-1)


class _MLPLayer(nn.Module):
    def __init__(self, hidden: int, inter: int, eps: float = 1e-6):
        super().__init__()
        self.norm = RMSNorm(hidden, eps)
        self.up, self.gate, self.down = nn.Linear(hidden, inter, bias=False), nn.Linear(hidden, inter, bias=False), nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        h = self.norm(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class MoGHead(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, out_size: int, num_layers: int = 2, num_predictions: int = 8,
                 low_rank: Optional[int] = 16, min_log_std: float = -4.0, eps: float = 1e-6):
        super().__init__()
        self.out_size, self.P, self.low_rank, self.min_log_std = out_size, num_predictions, low_rank, min_log_std
        self.mlp_stack = nn.Sequential(*[_MLPLayer(hidden_size, intermediate_size, eps) for _ in range(num_layers)], RMSNorm(hidden_size, eps))
        self.proj_logits = nn.Linear(hidden_size, num_predictions, bias=False)
        self.proj_logs = nn.Linear(hidden_size, 1, bias=False)
        if low_rank is None:
            self.proj_mus = nn.Linear(hidden_size, num_predictions * out_size, bias=False)
        else:
            if low_rank >= out_size:
                raise ValueError("low_rank must be smaller than out_size")
            self.proj_mus = nn.Linear(hidden_size, num_predictions * low_rank, bias=False)
            self.proj_else = nn.Linear(hidden_size, out_size, bias=False)
            self.low_mat = nn.Parameter(torch.randn(num_predictions, out_size, low_rank) * low_rank ** -0.5)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [..., H] -> (logits [..., P], mus [..., P, D], log_std [..., 1])."""
        h = self.mlp_stack(x)
        logits = self.proj_logits(h)
        logs = self.proj_logs(h).clamp(min=self.min_log_std)
        if self.low_rank is None:
            mus = self.proj_mus(h).view(*h.shape[:-1], self.P, self.out_size)
        else:
            z = self.proj_mus(h).view(*h.shape[:-1], self.P, self.low_rank)
            mus = torch.einsum("pdr,...pr->...pd", self.low_mat.to(z.dtype), z) + self.proj_else(h).unsqueeze(-2)
        return logits, mus, logs

    def nll(self, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Negative log-likelihood of ``target`` [..., D] under the isotropic mixture, per position."""
        logits, mus, logs = self(x)
        D = self.out_size
        sq = (target.unsqueeze(-2).float() - mus.float()).pow(2).sum(-1)                     # [..., P]
        logs = logs.float()
        comp = -0.5 * sq * torch.exp(-2.0 * logs) - D * logs - 0.5 * D * math.log(2 * math.pi)
        return -torch.logsumexp(F.log_softmax(logits.float(), dim=-1) + comp, dim=-1)

    @torch.no_grad()
    def infer(self, x: torch.Tensor, uncond: Optional[torch.Tensor] = None, guidance_scale: float = 0.0, top_p_or_k=1.0,
              temperature: float = 1.0, noise_scale: float = 0.0, generator=None) -> torch.Tensor:
        """Sample a latent [..., D].  With ``uncond`` hidden states the mixture logits and means are extrapolated away from the
        unconditional prediction by ``guidance_scale``."""
        logits, mus, logs = self(x)
        if uncond is not None and guidance_scale:
            ul, um, _ = self(uncond)
            logits = logits + guidance_scale * (logits - ul)
            mus = mus + guidance_scale * (mus - um)
        logits = logits.float() / max(temperature, 1e-5)
        if isinstance(top_p_or_k, int) and not isinstance(top_p_or_k, bool) and top_p_or_k >= 1:
            k = min(int(top_p_or_k), self.P)
            kth = logits.topk(k, dim=-1).values[..., -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        elif isinstance(top_p_or_k, float) and top_p_or_k < 1.0:
            srt, idx = logits.sort(dim=-1, descending=True)
            cum = srt.softmax(-1).cumsum(-1)
            drop = cum - srt.softmax(-1) >= top_p_or_k
            logits = logits.masked_fill(torch.zeros_like(drop).scatter(-1, idx, drop), float("-inf"))
        flat = logits.reshape(-1, self.P).softmax(-1)
        pick = torch.multinomial(flat, 1, generator=generator).view(*logits.shape[:-1])
        mu = mus.gather(-2, pick[..., None, None].expand(*pick.shape, 1, self.out_size)).squeeze(-2)
        if noise_scale:
            mu = mu + noise_scale * torch.exp(logs.float()).to(mu.dtype) * torch.randn(mu.shape, device=mu.device, dtype=mu.dtype, generator=generator)
        return mu


class GatedProjectedSumRMSNorm(nn.Module):
    def __init__(self, audio_dim: int, text_dim: int, hidden_dim: int, final_norm: bool = True, init_residual_scale: float = 0.5):
        super().__init__()
        self.audio_proj, self.text_proj = nn.Linear(audio_dim, hidden_dim, bias=False), nn.Linear(text_dim, hidden_dim, bias=False)
        self.gate = nn.Linear(2 * hidden_dim, hidden_dim)
        nn.init.zeros_(self.gate.weight)
        nn.init.constant_(self.gate.bias, math.log(init_residual_scale / (1 - init_residual_scale)))
        self.norm = RMSNorm(hidden_dim) if final_norm else nn.Identity()

    def forward(self, audio_emb, text_emb):
        a, t = self.audio_proj(audio_emb), self.text_proj(text_emb)
        g = torch.sigmoid(self.gate(torch.cat([a, t], dim=-1)))
        return self.norm(a + g * t)


class EARTTSModel(nn.Module):
    def __init__(self, cfg: Any):
        super().__init__()
        g = lambda k, d=None: cfg_get(cfg, k, d)  # noqa: E731
        self.K, self.N, self.D = int(g("num_quantizers", 4)), int(g("codebook_size", 64)), int(g("latent_size", 32))
        self.backbone = CausalLM.from_config(dict(g("backbone")))
        self.hidden = self.backbone.config.hidden_size
        self.text_vocab = int(self.backbone.config.vocab_size)
        self.embed_text = self.backbone.model.embed_tokens
        self.backbone.model.embed_tokens = None
        self.backbone.lm_head = None
        self.rvq = ResidualVQ(self.K, self.N, self.D)
        self.embed_code = nn.Linear(self.D, self.hidden, bias=False)
        self.bos_emb = nn.Parameter(torch.randn(self.D) * 0.02)
        self.null_emb = nn.Parameter(torch.randn(self.hidden) * 0.02)
        self.fuse = GatedProjectedSumRMSNorm(self.hidden, self.hidden, self.hidden)
        self.head = MoGHead(self.hidden, int(g("head_intermediate_size", 2 * self.hidden)), self.D, int(g("head_layers", 2)),
                            int(g("num_predictions", 8)), g("low_rank", min(16, self.D - 1)), float(g("min_log_std", -4.0)))
        self.cfg_dropout = float(g("cfg_dropout", 0.1))
        self.random_target_masking = bool(g("random_target_masking", True))
        self.freeze_rvq = bool(g("freeze_rvq", True))
        if self.freeze_rvq:
            self.rvq.codebooks.requires_grad_(False)

    def set_rvq_embs(self, codebooks: torch.Tensor) -> None:
        """Adopt the codebooks of a trained codec ([K, N, D])."""
        with torch.no_grad():
            self.rvq.codebooks.copy_(codebooks.to(self.rvq.codebooks))

    def _inputs(self, prev_latent: torch.Tensor, text_tokens: torch.Tensor, drop_text: Optional[torch.Tensor] = None) -> torch.Tensor:
        t = self.embed_text(text_tokens)
        if drop_text is not None:
            t = torch.where(drop_text.view(-1, 1, 1), self.null_emb.to(t.dtype).expand_as(t), t)
        return self.fuse(self.embed_code(prev_latent.to(t.dtype)), t)

    def forward(self, codes: torch.Tensor, text_tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """codes [B, T, K] target codes, text_tokens [B, T] frame-aligned text channel, mask [B, T] valid frames -> loss."""
        B, T, _ = codes.shape
        target = self.rvq.embed(codes)                                                     # full-depth latents
        depth = None
        if self.training and self.random_target_masking:
            depth = torch.randint(1, self.K + 1, (B, T), device=codes.device)              # feed coarser history at random
        hist = self.rvq.embed(codes, depth)
        prev = torch.cat([self.bos_emb.to(hist.dtype).expand(B, 1, -1), hist[:, :-1]], dim=1)
        drop = (torch.rand(B, device=codes.device) < self.cfg_dropout) if self.training and self.cfg_dropout > 0 else None
        out = self.backbone(inputs_embeds=self._inputs(prev, text_tokens, drop), return_hidden=True)
        nll = self.head.nll(out["hidden_states"], target.detach() if self.freeze_rvq else target)
        if mask is None:
            mask = torch.ones(B, T, dtype=torch.bool, device=codes.device)
        loss = (nll * mask).sum() / mask.sum().clamp(min=1)
        return {"loss": loss, "nll": nll}

    @torch.no_grad()
    def generate_step(self, prev_latent: torch.Tensor, text_token: torch.Tensor, cache: List[dict], uncond_cache: Optional[List[dict]] = None,
                      guidance_scale: float = 0.0, top_p_or_k=1.0, temperature: float = 1.0, noise_scale: float = 0.0, generator=None):
        """One frame: prev_latent [B, D], text_token [B] -> (codes [B, K], latent [B, D])."""
        x = self._inputs(prev_latent[:, None], text_token[:, None])
        h = self.backbone(inputs_embeds=x, cache=cache, return_hidden=True)["hidden_states"][:, -1]
        hu = None
        if uncond_cache is not None and guidance_scale:
            xu = self._inputs(prev_latent[:, None], text_token[:, None], torch.ones(x.shape[0], dtype=torch.bool, device=x.device))
            hu = self.backbone(inputs_embeds=xu, cache=uncond_cache, return_hidden=True)["hidden_states"][:, -1]
        latent = self.head.infer(h, hu, guidance_scale, top_p_or_k, temperature, noise_scale, generator)
        codes = self.rvq.encode(latent)
        return codes, self.rvq.embed(codes)

    @torch.no_grad()
    def generate(self, text_tokens: torch.Tensor, guidance_scale: float = 0.0, **sampling) -> torch.Tensor:
        """Speak a frame-aligned token stream [B, T]: codes [B, T, K]."""
        B, T = text_tokens.shape
        cache = [dict() for _ in self.backbone.model.layers]
        ucache = [dict() for _ in self.backbone.model.layers] if guidance_scale else None
        prev = self.bos_emb.expand(B, -1).to(self.embed_code.weight.dtype)
        out = []
        for t in range(T):
            codes, prev = self.generate_step(prev, text_tokens[:, t], cache, ucache, guidance_scale, **sampling)
            out.append(codes)
        return torch.stack(out, dim=1)


class DuplexEARTTS(ModelPT):
    """Batch: ``target_tokens`` [B, T] (agent text channel, frame aligned), ``target_codes`` [B, T, K], ``target_lens`` [B]."""

    def __init__(self, cfg: DictConfig, trainer=None, audio_codec=None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self.tts = EARTTSModel(self._cfg.tts)
        self.audio_codec, self.tokenizer = audio_codec, tokenizer
        cb = getattr(audio_codec, "rvq_codebooks", None)
        if cb is not None:
            self.tts.set_rvq_embs(cb)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "tts"):                                                         # the base constructor calls this before the layers exist
            super()._setup_dataloaders_from_cfg()

    def _loader(self, c):
        from ..tts.code_datasets import build_code_dataloader

        m = self.tts
        return build_code_dataloader(c, num_codebooks=m.K, codebook_size=m.N, text_vocab=m.text_vocab, tokenizer=self.tokenizer, frame_aligned=True)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def forward(self, codes, tokens, lens=None):
        mask = None if lens is None else torch.arange(codes.shape[1], device=codes.device)[None] < lens[:, None]
        return self.tts(codes, tokens, mask)

    def training_step(self, batch, batch_idx):
        out = self(batch["target_codes"].long(), batch["target_tokens"].long(), batch.get("target_lens"))
        self.log_dict({"train_loss": out["loss"].detach()})
        return {"loss": out["loss"]}

    def validation_step(self, batch, batch_idx):
        with torch.no_grad():
            out = self(batch["target_codes"].long(), batch["target_tokens"].long(), batch.get("target_lens"))
        return {"val_loss": out["loss"]}

    @torch.no_grad()
    def offline_inference(self, tokens: torch.Tensor, decode_audio: bool = False, **gen) -> Dict[str, Any]:
        self.eval()
        codes = self.tts.generate(tokens, **gen)
        res: Dict[str, Any] = {"codes": codes}
        if decode_audio and self.audio_codec is not None:
            lens = torch.full((codes.shape[0],), codes.shape[1], device=codes.device)
            res["audio"], res["audio_len"] = self.audio_codec.decode(tokens=codes.transpose(1, 2), tokens_len=lens)
        return res


class DuplexS2SSpeechDecoderModel(ModelPT):
    """Duplex speech-to-speech with a separate speech decoder: the LLM (a ``DuplexSTTModel``) owns the text channel; a causal
    transformer reads ``proj(LLM hidden state) + embeddings of the previous frame's codes`` and predicts all codebooks."""

    def __init__(self, cfg: DictConfig, trainer=None, stt=None, audio_codec=None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        from .duplex import DuplexSTTModel

        cfg = self._cfg
        self.stt = stt if stt is not None else DuplexSTTModel(cfg, tokenizer=tokenizer)
        self.audio_codec = audio_codec
        self.K, self.N = int(cfg_get(cfg, "num_codebooks", 2)), int(cfg_get(cfg, "codebook_size", 16))
        self.speech_vocab_size = self.N + 3                                                 # + speech BOS / EOS / delay
        self.speech_bos_id = self.N
        self.decoder = CausalLM.from_config(dict(cfg.speech_decoder))
        hd = self.decoder.config.hidden_size
        self.decoder.model.embed_tokens = None
        self.decoder.lm_head = None
        self.hidden_proj = nn.Linear(self.stt.llm.config.hidden_size, hd)
        self.code_emb = nn.ModuleList(nn.Embedding(self.speech_vocab_size, hd) for _ in range(self.K))
        self.audio_head = nn.Linear(hd, self.K * self.speech_vocab_size)
        self.audio_loss_weight = float(cfg_get(cfg, "audio_loss_weight", 1.0))

    def setup_training_data(self, c):
        self._train_dl = None

    def setup_validation_data(self, c):
        self._validation_dl = None

    def _speech_inputs(self, hidden: torch.Tensor, prev_codes: torch.Tensor) -> torch.Tensor:
        x = self.hidden_proj(hidden)
        for k in range(self.K):
            x = x + self.code_emb[k](prev_codes[..., k]).to(x.dtype)
        return x

    def _audio_logits(self, hidden, prev_codes, cache=None):
        h = self.decoder(inputs_embeds=self._speech_inputs(hidden, prev_codes), cache=cache, return_hidden=True)["hidden_states"]
        return self.audio_head(h).view(*h.shape[:2], self.K, self.speech_vocab_size)

    def training_step(self, batch, batch_idx):
        inp = self.stt.prepare_inputs(batch)
        T, m = inp["T"], inp["mask"]
        out = self.stt.llm(inputs_embeds=self.stt._frame_inputs(inp["emb"], inp["prev_text"]), return_hidden=True)
        hidden = out["hidden_states"]
        text_loss = F.cross_entropy(self.stt.llm.lm_head(hidden)[m].float(), inp["text_labels"][m])
        codes = batch["target_codes"][:, :T].long()
        prev = torch.cat([torch.full_like(codes[:, :1], self.speech_bos_id), codes[:, :-1]], dim=1)
        logits = self._audio_logits(hidden, prev)
        audio_loss = F.cross_entropy(logits[m].float().reshape(-1, self.speech_vocab_size), codes[m].reshape(-1))
        loss = self.stt.text_loss_weight * text_loss + self.audio_loss_weight * audio_loss
        self.log_dict({"train_loss": loss.detach(), "text_loss": text_loss.detach(), "audio_loss": audio_loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def offline_inference(self, source_audio, source_audio_lens, decode_audio: bool = False) -> Dict[str, Any]:
        self.eval()
        stt = self.stt
        emb, emb_len = stt.perception(input_signal=source_audio, input_signal_length=source_audio_lens)
        B, T, _ = emb.shape
        cache = [dict() for _ in stt.llm.model.layers]
        dcache = [dict() for _ in self.decoder.model.layers]
        prev = torch.full((B, 1), stt.text_pad_id, dtype=torch.long, device=emb.device)
        prev_codes = torch.full((B, 1, self.K), self.speech_bos_id, dtype=torch.long, device=emb.device)
        toks, codes = [], []
        for t in range(T):
            o = stt.llm(inputs_embeds=stt._frame_inputs(emb[:, t:t + 1], prev), cache=cache, return_hidden=True)
            hid = o["hidden_states"][:, -1:]
            prev = stt.llm.lm_head(hid)[:, -1].argmax(-1, keepdim=True)
            prev_codes = self._audio_logits(hid, prev_codes, dcache)[:, -1:].argmax(-1)
            toks.append(prev)
            codes.append(prev_codes)
        tokens, codes = torch.cat(toks, 1), torch.cat(codes, 1)
        res = {"tokens": tokens, "codes": codes, "lengths": emb_len, "text": stt._tokens_to_text(tokens, emb_len)}
        if decode_audio and self.audio_codec is not None:
            c = codes.clamp(max=self.N - 1)
            res["audio"], res["audio_len"] = self.audio_codec.decode(tokens=c.transpose(1, 2), tokens_len=emb_len)
        return res


class NemotronVoiceChat(nn.Module):
    """Listening and speaking halves run in lock step: at frame ``t`` the STT half reads the user's audio frame and emits the
    agent's text token; the TTS half speaks the token of frame ``t-1`` (one frame of look-behind, so that speech never runs
    ahead of the text)."""

    def __init__(self, stt, tts: DuplexEARTTS):
        super().__init__()
        self.stt, self.tts = stt, tts

    @torch.no_grad()
    def init_state(self, batch_size: int, device) -> Dict[str, Any]:
        m = self.tts.tts
        return {"stt_cache": [dict() for _ in self.stt.llm.model.layers], "tts_cache": [dict() for _ in m.backbone.model.layers],
                "prev_text": torch.full((batch_size, 1), self.stt.text_pad_id, dtype=torch.long, device=device),
                "pending_text": torch.full((batch_size,), self.stt.text_pad_id, dtype=torch.long, device=device),
                "prev_latent": m.bos_emb.expand(batch_size, -1).to(device)}

    @torch.no_grad()
    def step(self, frame_emb: torch.Tensor, state: Dict[str, Any], **sampling) -> Tuple[torch.Tensor, torch.Tensor]:
        """frame_emb [B, 1, H] (perception output of one frame) -> (text token [B], codes [B, K])."""
        out = self.stt(self.stt._frame_inputs(frame_emb, state["prev_text"]), cache=state["stt_cache"])
        tok = out["text_logits"][:, -1].argmax(-1)
        codes, state["prev_latent"] = self.tts.tts.generate_step(state["prev_latent"], state["pending_text"], state["tts_cache"], **sampling)
        state["prev_text"], state["pending_text"] = tok[:, None], tok
        return tok, codes

    @torch.no_grad()
    def offline_inference(self, source_audio, source_audio_lens, **sampling) -> Dict[str, Any]:
        self.eval()
        emb, emb_len = self.stt.perception(input_signal=source_audio, input_signal_length=source_audio_lens)
        state = self.init_state(emb.shape[0], emb.device)
        toks, codes = [], []
        for t in range(emb.shape[1]):
            tk, cd = self.step(emb[:, t:t + 1], state, **sampling)
            toks.append(tk)
            codes.append(cd)
        tokens = torch.stack(toks, 1)
        return {"tokens": tokens, "codes": torch.stack(codes, 1), "lengths": emb_len, "text": self.stt._tokens_to_text(tokens, emb_len)}

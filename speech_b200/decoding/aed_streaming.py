"""Streaming (simultaneous) greedy decoding for attention encoder-decoder models: wait-k and AlignAtt policies, batched.

The encoder output of each stream grows chunk by chunk; after every chunk the decoder may emit tokens:

* **wait-k** — nothing until ``waitk_lagging`` chunks have arrived, then exactly one token per new chunk; everything up to EOS
  once the stream's audio has ended.
* **AlignAtt** — keep emitting while the candidate token's cross-attention (last decoder layer, mean over heads) peaks at
  least ``alignatt_thr`` frames before the end of the audio seen so far; a token that looks at the newest frames is withheld
  until more audio arrives.  At most ``max_tokens_per_alignatt_step`` tokens per chunk; no restriction on the last chunk.

Both stop a stream on EOS after its last chunk, on ``max_generation_length`` and — optionally — when the tail of the
hypothesis degenerates into a repeated n-gram.  Per-token frame positions are recorded so that latency (LAAL) can be computed.

Reference: ``parts/submodules/aed_decoding/aed_batched_streaming.py:28-546`` (``AEDStreamingState``,
``GreedyBatchedStreamingAEDComputer.run_waitk_decoding_step`` / ``run_alignatt_decoding_step``, ``detect_hallucinations``,
``compute_alignatt_lagging`` / ``compute_waitk_lagging``).  The decoder is re-run on the accepted prefix at every step (prefixes
are short and of different length per stream), so no per-stream cache surgery is needed when a candidate is rejected.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class AEDStreamingDecodingConfig:
    streaming_policy: str = "waitk"           # "waitk" | "alignatt"
    waitk_lagging: int = 2
    alignatt_thr: int = 8
    max_generation_length: int = 256
    max_tokens_per_alignatt_step: Optional[int] = 10
    hallucinations_detector: bool = True
    exclude_sink_frames: int = 0               # leading encoder frames ignored when locating the attention peak
    use_avgpool_for_alignatt: bool = False
    frame_chunk_size: int = 1                  # encoder frames per audio chunk (for the initial wait-k lag)


@dataclass
class AEDStreamingState:
    pred_tokens_ids: torch.Tensor              # [B, max_generation_length] prompt + hypothesis, padded with EOS
    current_context_lengths: torch.Tensor      # [B] tokens held per stream (prompt included)
    prompt_lengths: torch.Tensor               # [B]
    active_samples: torch.Tensor               # [B] bool, False once a stream is finished
    tokens_frame_alignment: torch.Tensor       # [B, max_generation_length] encoder frames available when the token was emitted
    chunks_seen: int = 0
    is_last_chunk_batch: Optional[torch.Tensor] = None

    def hypotheses(self, eos: int) -> List[List[int]]:
        out = []
        for b in range(self.pred_tokens_ids.shape[0]):
            seq = self.pred_tokens_ids[b, int(self.prompt_lengths[b]): int(self.current_context_lengths[b])].tolist()
            out.append([t for t in seq if t != eos])
        return out


class GreedyBatchedStreamingAEDComputer:
    def __init__(self, embedding, decoder, classifier, eos: int, cfg: AEDStreamingDecodingConfig):
        if cfg.streaming_policy not in ("waitk", "alignatt"):
            raise ValueError("streaming AED decoding supports only the alignatt or waitk policy")
        self.embedding, self.decoder, self.classifier, self.eos, self.cfg = embedding, decoder, classifier, eos, cfg
        self._xatt_in = None
        self._hook = None

    # ------------------------------------------------------------------ state
    def init_state(self, decoder_input_ids: torch.Tensor, prompt_lengths: Optional[torch.Tensor] = None) -> AEDStreamingState:
        B, P = decoder_input_ids.shape
        dev = decoder_input_ids.device
        L = self.cfg.max_generation_length
        toks = torch.full((B, L), self.eos, dtype=torch.long, device=dev)
        toks[:, :P] = decoder_input_ids
        pl = prompt_lengths.long().clone() if prompt_lengths is not None else torch.full((B,), P, dtype=torch.long, device=dev)
        return AEDStreamingState(toks, pl.clone(), pl, torch.ones(B, dtype=torch.bool, device=dev),
                                 torch.zeros((B, L), dtype=torch.long, device=dev))

    # ------------------------------------------------------------------ one decoder evaluation on the accepted prefixes
    def _step(self, state: AEDStreamingState, enc, enc_mask, want_attention: bool):
        lens = state.current_context_lengths
        n = int(lens.max())
        ids = state.pred_tokens_ids[:, :n]
        mask = (torch.arange(n, device=ids.device)[None, :] < lens[:, None]).long()
        emb = self.embedding(ids, start_pos=0)
        if emb.dtype != enc.dtype:
            emb = emb.to(enc.dtype)
        last_block = self.decoder.layers[-1]
        if want_attention and self._hook is None:
            self._hook = last_block.second_sub_layer.register_forward_pre_hook(self._capture, with_kwargs=True)
        self._xatt_in = None
        x = self.decoder(emb, mask, enc, enc_mask)
        idx = (lens - 1).clamp(min=0)
        h = x[torch.arange(x.shape[0], device=x.device), idx].unsqueeze(1)
        logp = self.classifier(hidden_states=h)[:, 0]
        att = None
        if want_attention and self._xatt_in is not None:
            q_in, k_in = self._xatt_in
            mha = last_block.second_sub_layer
            H, dk = mha.num_attention_heads, mha.attn_head_size
            B = q_in.shape[0]
            q = torch.nn.functional.linear(q_in[torch.arange(B, device=q_in.device), idx].float(), mha.query_net.weight, mha.query_net.bias)
            k = torch.nn.functional.linear(k_in.float(), mha.key_net.weight, mha.key_net.bias)
            sc = torch.einsum("bhd,bthd->bht", q.view(B, H, dk), k.view(B, -1, H, dk)) / math.sqrt(dk)
            sc = sc.masked_fill(~enc_mask.bool()[:, None, :], float("-inf"))
            att = torch.softmax(sc, dim=-1).mean(1)                        # [B, T_enc]
        return logp, att

    def _capture(self, module, args, kwargs):
        queries = args[0] if args else kwargs["queries"]
        keys = args[1] if len(args) > 1 else kwargs["keys"]
        self._xatt_in = (queries, keys)
        return None

    def close(self):
        if self._hook is not None:
            self._hook.remove()
            self._hook = None

    # ------------------------------------------------------------------ safeguards
    def detect_hallucinations(self, state: AEDStreamingState) -> torch.Tensor:
        """True where the hypothesis ends in the same n-gram (n = 1..4) repeated at least 4 times."""
        B = state.pred_tokens_ids.shape[0]
        bad = torch.zeros(B, dtype=torch.bool, device=state.pred_tokens_ids.device)
        for b in range(B):
            seq = state.pred_tokens_ids[b, int(state.prompt_lengths[b]): int(state.current_context_lengths[b])].tolist()
            for n in (1, 2, 3, 4):
                if len(seq) >= 4 * n and all(seq[-n:] == seq[-(r + 1) * n: len(seq) - r * n] for r in range(1, 4)):
                    bad[b] = True
        return bad

    def _accept(self, state: AEDStreamingState, tokens: torch.Tensor, take: torch.Tensor, enc_len: torch.Tensor):
        b = torch.nonzero(take, as_tuple=False).squeeze(1)
        if b.numel() == 0:
            return
        pos = state.current_context_lengths[b]
        state.pred_tokens_ids[b, pos] = tokens[b]
        state.tokens_frame_alignment[b, pos] = enc_len[b]
        state.current_context_lengths[b] = pos + 1

    # ------------------------------------------------------------------ policies
    @torch.no_grad()
    def __call__(self, encoder_output: torch.Tensor, encoder_output_len: torch.Tensor, is_last_chunk_batch: torch.Tensor,
                 state: AEDStreamingState) -> AEDStreamingState:
        """encoder_output [B, T, D]: all encoder frames available so far; is_last_chunk_batch [B] bool."""
        cfg = self.cfg
        state.chunks_seen += 1
        state.is_last_chunk_batch = is_last_chunk_batch
        last = is_last_chunk_batch.bool()
        enc_len = encoder_output_len.long()
        if int(enc_len.max()) // max(cfg.frame_chunk_size, 1) < cfg.waitk_lagging and not bool(last.all()):
            return state                                                    # initial lag: wait for more audio
        enc_mask = torch.arange(encoder_output.shape[1], device=encoder_output.device)[None, :] < enc_len[:, None]
        limit = cfg.max_generation_length - 1
        emitted = torch.zeros_like(state.current_context_lengths)
        inner = state.active_samples.clone()
        while bool(inner.any()):
            logp, att = self._step(state, encoder_output, enc_mask, want_attention=cfg.streaming_policy == "alignatt")
            nxt = logp.argmax(-1)
            is_eos = nxt == self.eos
            state.active_samples &= ~(is_eos & last)                       # EOS ends a stream only when its audio has ended
            inner &= ~is_eos
            if cfg.streaming_policy == "alignatt":
                a = att.clone()
                if cfg.exclude_sink_frames > 0:
                    a[:, : cfg.exclude_sink_frames] = 0.0
                if cfg.use_avgpool_for_alignatt:
                    a = torch.nn.functional.avg_pool1d(a.unsqueeze(1), 7, 1, 3, count_include_pad=False).squeeze(1)
                peak = a.masked_fill(~enc_mask, -1.0).argmax(-1)
                inner &= ((enc_len - (peak + 1)) >= cfg.alignatt_thr) | last
            self._accept(state, nxt, inner, enc_len)
            emitted += inner.long()
            if cfg.hallucinations_detector:
                bad = self.detect_hallucinations(state) & inner
                state.active_samples &= ~bad
                inner &= ~bad
            full = state.current_context_lengths >= limit
            state.active_samples &= ~full
            inner &= ~full
            if cfg.streaming_policy == "waitk":
                inner &= last                                               # one token per chunk until the audio ends
            elif cfg.max_tokens_per_alignatt_step is not None:
                inner &= (emitted < cfg.max_tokens_per_alignatt_step) | last
        return state

    # ------------------------------------------------------------------ latency
    @staticmethod
    def compute_laal(state: AEDStreamingState, audio_frames: torch.Tensor, frame_seconds: float) -> List[float]:
        """Length-adaptive average lagging (seconds): mean over tokens of ``d_i - (i - 1) * |audio| / max(|hyp|, |ref|)`` with
        ``d_i`` the audio available when token i was emitted."""
        out = []
        for b in range(state.pred_tokens_ids.shape[0]):
            p, n = int(state.prompt_lengths[b]), int(state.current_context_lengths[b])
            d = state.tokens_frame_alignment[b, p:n].float() * frame_seconds
            if d.numel() == 0:
                out.append(0.0)
                continue
            total = float(audio_frames[b]) * frame_seconds
            i = torch.arange(d.numel(), dtype=torch.float32, device=d.device)
            tau = int((d < total).sum().clamp(min=1))
            out.append(float((d - i * total / d.numel())[:tau].mean()))
        return out

"""Frame-synchronous inference engine of the duplex speech-to-text model.

At every perception frame the LLM reads ``user audio frame + embedding of the agent token emitted on the previous frame
(+ embedding of the recognised user token of the previous frame)`` and emits the agent's next text token (and, when the model
predicts the user channel, the user's next token), with a KV cache so that each frame costs one single-token LLM step.
Features, following ``speechlm2/streaming/duplex_stt_inference.py:25-386``:

* a text *prompt* (system / context tokens) placed in front of the audio frames: on prompt positions the input is the prompt
  token's embedding and nothing is generated;
* *forced turn taking*: when the recognised user channel ends a turn (user EOS, or ``pad_window`` silent frames after speech)
  and the agent has not started within ``threshold`` frames, agent BOS is forced; when the user barges in (user BOS) and the
  agent has not stopped, agent EOS is forced;
* trailing silence padding (``input_pad_len`` samples) so that the agent can finish after the user stops;
* incremental use: :meth:`DuplexSTTStreamingInference.start` / :meth:`feed` accept audio chunk by chunk.  The perception
  encoder is run over a sliding window (``left_context_s`` seconds of past audio) and only the frames of the new chunk are
  passed on, so the cost per chunk does not grow with the length of the conversation.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class DuplexState:
    cache: List[dict]
    gen_text: List[torch.Tensor] = field(default_factory=list)       # one [B] tensor per position
    gen_asr: List[torch.Tensor] = field(default_factory=list)
    is_prompt: List[torch.Tensor] = field(default_factory=list)      # [B] bool per position
    t: int = 0
    audio: Optional[torch.Tensor] = None                              # [B, S] samples received so far (window kept)
    audio_start: int = 0                                               # sample index of audio[:, 0] in the stream
    frames_done: int = 0                                               # perception frames already consumed


class DuplexSTTStreamingInference:
    def __init__(self, model, force_turn_taking: Optional[bool] = None, threshold: Optional[int] = None, pad_window: Optional[int] = None,
                 left_context_s: float = 10.0):
        self.model = model
        cfg = model.cfg
        self.force = bool(cfg.get("force_turn_taking", False)) if force_turn_taking is None else force_turn_taking
        self.threshold = int(cfg.get("force_turn_taking_threshold", 40)) if threshold is None else threshold
        self.pad_window = int(cfg.get("force_turn_taking_pad_window", 25)) if pad_window is None else pad_window
        self.text_w = float(cfg.get("duplex_text_channel_weight", 1.0))
        self.asr_w = float(cfg.get("duplex_asr_text_weight", 1.0))
        self.left_context_s = left_context_s
        self.user_bos = getattr(model, "user_bos_id", model.text_bos_id)
        self.user_eos = getattr(model, "user_eos_id", model.text_eos_id)

    # ------------------------------------------------------------------ one position
    def _prev_embedding(self, st: DuplexState, B: int, device) -> torch.Tensor:
        m = self.model
        if st.t == 0:
            prev_text = torch.full((B,), m.text_pad_id, dtype=torch.long, device=device)
            prev_asr = prev_text
        else:
            prev_text, prev_asr = st.gen_text[-1], (st.gen_asr[-1] if st.gen_asr else None)
        e = m.embed_tokens(prev_text) * self.text_w
        if getattr(m, "predict_user_text", False):
            e = e + m.embed_asr_tokens(prev_asr) * self.asr_w
        return e

    def _force_turn_taking(self, st: DuplexState, text: torch.Tensor, asr: torch.Tensor, is_prompt: torch.Tensor) -> torch.Tensor:
        m, t = self.model, st.t
        if not self.force or t < self.pad_window or not st.gen_asr:
            return text
        hist_text = torch.stack(st.gen_text[max(0, t - self.threshold):], dim=1)              # [B, <=threshold]
        hist_asr = torch.stack(st.gen_asr[t - self.pad_window:], dim=1)                        # [B, pad_window]
        silent = (hist_asr == m.text_pad_id).all(dim=1)
        if t - self.pad_window > 0:
            silent = silent & (st.gen_asr[t - self.pad_window - 1] != m.text_pad_id)           # silence that follows speech
        else:
            silent = torch.zeros_like(silent)
        user_done = (asr == self.user_eos) | silent
        user_starts = (asr == self.user_bos) & ~user_done
        agent_started = (hist_text == m.text_bos_id).any(dim=1)
        agent_stopped = (hist_text == m.text_eos_id).any(dim=1)
        text = torch.where(user_done & ~agent_started & ~is_prompt, torch.full_like(text, m.text_bos_id), text)
        text = torch.where(user_starts & ~agent_stopped & ~is_prompt, torch.full_like(text, m.text_eos_id), text)
        return text

    @torch.no_grad()
    def step(self, st: DuplexState, frame_emb: torch.Tensor, prompt_token: Optional[torch.Tensor] = None,
             is_prompt: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """One position for the whole batch.  ``frame_emb`` [B, H]: the audio frame (zeros on prompt positions);
        ``prompt_token`` [B] / ``is_prompt`` [B]: rows that are still inside their prompt take the prompt token as this
        position's agent token instead of generating one."""
        m = self.model
        B, dev = frame_emb.shape[0], frame_emb.device
        if is_prompt is None:
            is_prompt = torch.zeros(B, dtype=torch.bool, device=dev)
        x = frame_emb + self._prev_embedding(st, B, dev).to(frame_emb.dtype)
        out = m(x.unsqueeze(1), cache=st.cache)
        text = out["text_logits"][:, -1].argmax(dim=-1)
        asr = out["asr_logits"][:, -1].argmax(dim=-1) if "asr_logits" in out else None
        if prompt_token is not None:
            text = torch.where(is_prompt, prompt_token, text)
            if asr is not None:
                asr = torch.where(is_prompt, torch.full_like(asr, m.text_pad_id), asr)
        if asr is not None:
            text = self._force_turn_taking(st, text, asr, is_prompt)
            st.gen_asr.append(asr)
        st.gen_text.append(text)
        st.is_prompt.append(is_prompt)
        st.t += 1
        return {"text": text, "asr": asr}

    # ------------------------------------------------------------------ whole utterances
    @torch.no_grad()
    def offline_inference(self, input_signal: torch.Tensor, input_signal_lens: torch.Tensor, prompt_tokens: Optional[torch.Tensor] = None,
                          prompt_token_lens: Optional[torch.Tensor] = None, input_pad_len: int = 0) -> Dict[str, Any]:
        m = self.model
        m.eval()
        if input_pad_len > 0:
            input_signal = torch.nn.functional.pad(input_signal, (0, input_pad_len))
            input_signal_lens = input_signal_lens + input_pad_len
        emb, emb_len = m.perception(input_signal=input_signal, input_signal_length=input_signal_lens)
        B, T, H = emb.shape
        dev = emb.device
        P = int(prompt_token_lens.max()) if prompt_tokens is not None else 0
        st = DuplexState(cache=[dict() for _ in m.llm.model.layers])
        # prompts are right-aligned in front of the audio so that every row's audio starts at position P
        for p in range(P):
            k = p - (P - prompt_token_lens.to(dev))                       # index into each row's prompt
            inside = k >= 0
            tok = prompt_tokens.to(dev).gather(1, k.clamp(min=0).unsqueeze(1)).squeeze(1)
            tok = torch.where(inside, tok, torch.full_like(tok, m.text_pad_id))
            self.step(st, torch.zeros(B, H, dtype=emb.dtype, device=dev), prompt_token=tok, is_prompt=torch.ones(B, dtype=torch.bool, device=dev))
        for t in range(T):
            self.step(st, emb[:, t])
        return self._collect(st, emb_len, P)

    def _collect(self, st: DuplexState, emb_len: torch.Tensor, P: int) -> Dict[str, Any]:
        m = self.model
        text = torch.stack(st.gen_text[P:], dim=1) if len(st.gen_text) > P else torch.zeros((emb_len.shape[0], 0), dtype=torch.long)
        res = {"tokens": text, "lengths": emb_len, "text": m._tokens_to_text(text, emb_len)}
        if st.gen_asr:
            asr = torch.stack(st.gen_asr[P:], dim=1)
            res["asr_tokens"] = asr
            res["asr_text"] = m._tokens_to_text(asr, emb_len)
        return res

    # ------------------------------------------------------------------ chunk by chunk
    def start(self, batch_size: int, device=None, prompt_tokens: Optional[torch.Tensor] = None,
              prompt_token_lens: Optional[torch.Tensor] = None) -> DuplexState:
        m = self.model
        m.eval()
        device = device or next(m.parameters()).device
        st = DuplexState(cache=[dict() for _ in m.llm.model.layers])
        if prompt_tokens is not None:
            H = m.llm.config.hidden_size
            P = int(prompt_token_lens.max())
            for p in range(P):
                k = p - (P - prompt_token_lens.to(device))
                tok = prompt_tokens.to(device).gather(1, k.clamp(min=0).unsqueeze(1)).squeeze(1)
                tok = torch.where(k >= 0, tok, torch.full_like(tok, m.text_pad_id))
                self.step(st, torch.zeros(batch_size, H, device=device), prompt_token=tok,
                          is_prompt=torch.ones(batch_size, dtype=torch.bool, device=device))
        st.prompt_positions = st.t
        return st

    @torch.no_grad()
    def feed(self, st: DuplexState, audio_chunk: torch.Tensor) -> Dict[str, Any]:
        """``audio_chunk`` [B, S_new]: appends the samples, encodes the window that ends with them and steps the LLM over the
        frames that are new.  Returns the agent (and user) tokens of those frames."""
        m = self.model
        sr = int(getattr(m.perception.preprocessor, "_sample_rate", 16000)) if hasattr(m.perception, "preprocessor") else 16000
        st.audio = audio_chunk if st.audio is None else torch.cat([st.audio, audio_chunk], dim=1)
        keep = int(self.left_context_s * sr) + audio_chunk.shape[1]
        if st.audio.shape[1] > keep:
            cut = st.audio.shape[1] - keep
            # keep the window start on a frame boundary of the encoder so that frame indices stay aligned with the stream
            spf = max(1, int(round(sr * m.perception.token_equivalent_duration))) if hasattr(m.perception, "token_equivalent_duration") else 1280
            cut = cut // spf * spf
            st.audio, st.audio_start = st.audio[:, cut:], st.audio_start + cut
        B = st.audio.shape[0]
        lens = torch.full((B,), st.audio.shape[1], dtype=torch.long, device=st.audio.device)
        emb, emb_len = m.perception(input_signal=st.audio, input_signal_length=lens)
        spf = st.audio.shape[1] / max(1, emb.shape[1])
        first_global = int(round(st.audio_start / spf))
        new_from = st.frames_done - first_global
        toks, asrs = [], []
        for t in range(max(0, new_from), emb.shape[1]):
            o = self.step(st, emb[:, t])
            toks.append(o["text"])
            if o["asr"] is not None:
                asrs.append(o["asr"])
        st.frames_done = first_global + emb.shape[1]
        out = {"tokens": torch.stack(toks, dim=1) if toks else torch.zeros((B, 0), dtype=torch.long, device=st.audio.device)}
        if asrs:
            out["asr_tokens"] = torch.stack(asrs, dim=1)
        n = torch.full((B,), out["tokens"].shape[1], dtype=torch.long)
        out["text"] = m._tokens_to_text(out["tokens"], n)
        return out

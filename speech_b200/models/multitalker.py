"""Multi-talker ASR around ``EncDecMultiTalkerRNNTBPEModel``: who-spoke-what transcription of overlapped recordings.

A diarizer gives per-frame speaker activities ``[B, T, S]``; for each active speaker the ASR model runs once with that speaker's
activity as target mask and the union of the others as background mask (speaker kernels inside the encoder), and the word
timestamps of all passes are merged into a SegLST transcript (one record per sentence: session, speaker, start, end, words).

* ``SpeakerTaggedASR.transcribe_offline`` — whole recordings.
* ``SpeakerTaggedASR.stream`` — chunk by chunk with one ASR instance (encoder cache + partial hypothesis) per speaker that
  has become active (``MultiTalkerInstanceManager``), speakers batched into one encoder step.
* ``mask_features`` — the alternative to kernels: silence the frames of the features where the target speaker is inactive.
* ``SpeakerTargetDataset`` — training examples ``(audio, len, tokens, len, spk_targets, bg_spk_targets)`` for a query speaker of
  a multi-speaker cut.

References: ``asr/models/multitalker_asr_models.py``, ``asr/parts/utils/multispk_transcribe_utils.py`` (``SpeakerTaggedASR``,
``MultiTalkerInstanceManager``, SegLST helpers), ``asr/data/audio_to_text_lhotse_speaker.py``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = ["MultiTalkerInstanceManager", "SpeakerTaggedASR", "SpeakerTargetDataset", "find_active_speakers", "get_simulated_softmax",
           "mask_features", "sentences_from_words", "write_seglst"]


# ------------------------------------------------------------------------------------------------ helpers
def find_active_speakers(diar_preds: torch.Tensor, threshold: float = 0.5, min_active_frames: int = 3, max_speakers: Optional[int] = None
                         ) -> List[List[int]]:
    """Per batch item the speaker indices active for at least ``min_active_frames`` frames, most active first."""
    act = (diar_preds > threshold).sum(dim=1)                           # [B, S]
    out = []
    for b in range(act.shape[0]):
        idx = [int(s) for s in act[b].argsort(descending=True) if int(act[b, s]) >= min_active_frames]
        out.append(idx[:max_speakers] if max_speakers else idx)
    return out


def get_simulated_softmax(speaker_sigmoid: torch.Tensor, min_sigmoid_val: float = 1e-2, limit_max_spks: Optional[int] = None) -> torch.Tensor:
    """Turns independent per-speaker sigmoids ``[S]`` into a distribution over speakers for word-level speaker assignment: values
    under ``min_sigmoid_val`` are floored, speakers beyond ``limit_max_spks`` are zeroed, and the rest is normalised."""
    v = speaker_sigmoid.clone().float().clamp(min=min_sigmoid_val)
    if limit_max_spks is not None:
        v[limit_max_spks:] = 0.0
    return v / v.sum().clamp(min=1e-8)


def mask_features(features: torch.Tensor, mask: torch.Tensor, subsampling: int = 8, threshold: float = 0.5, fill: Optional[float] = None,
                  soft: bool = False) -> torch.Tensor:
    """``features`` [B, F, T], ``mask`` [B, T'] at the encoder frame rate: frames whose speaker activity is below ``threshold`` are
    replaced by ``fill`` (default: the minimum of the features, i.e. silence in log-mel); ``soft`` interpolates instead."""
    B, F_, T = features.shape
    m = mask.float().repeat_interleave(subsampling, dim=1)
    m = m[:, :T] if m.shape[1] >= T else torch.nn.functional.pad(m, (0, T - m.shape[1]))
    floor = features.amin(dim=(1, 2), keepdim=True) if fill is None else torch.full((B, 1, 1), fill, device=features.device, dtype=features.dtype)
    w = m.unsqueeze(1).to(features.dtype) if soft else (m > threshold).unsqueeze(1).to(features.dtype)
    return features * w + floor * (1 - w)


def sentences_from_words(words: Sequence[Dict[str, Any]], session_id: str, speaker: str, max_gap: float = 1.0,
                         sentence_end: str = ".?!") -> List[Dict[str, Any]]:
    """Groups ``{"word", "start_time", "end_time"}`` records into SegLST sentences: a sentence closes after a word ending in
    ``sentence_end`` or before a pause longer than ``max_gap`` seconds."""
    out: List[Dict[str, Any]] = []
    cur: List[Dict[str, Any]] = []

    def close():
        if cur:
            out.append({"session_id": session_id, "speaker": speaker, "start_time": round(cur[0]["start_time"], 3),
                        "end_time": round(cur[-1]["end_time"], 3), "words": " ".join(w["word"] for w in cur)})
            cur.clear()

    for w in words:
        if cur and w["start_time"] - cur[-1]["end_time"] > max_gap:
            close()
        cur.append(w)
        if w["word"] and w["word"][-1] in sentence_end:
            close()
    close()
    return out


def write_seglst(path: str, seglst: Sequence[Dict[str, Any]]):
    with open(path, "w", encoding="utf-8") as f:
        json.dump(sorted(seglst, key=lambda d: (d["session_id"], d["start_time"])), f, indent=2, ensure_ascii=False)


def _words_of(hyp, tokenizer, frame_sec: float, offset_frames: int = 0) -> List[Dict[str, Any]]:
    """Word records from a hypothesis' tokens and per-token frame indices (SentencePiece word starts open a word)."""
    ys = hyp.y_sequence.tolist() if torch.is_tensor(hyp.y_sequence) else list(hyp.y_sequence)
    ts = hyp.timestamp.tolist() if torch.is_tensor(hyp.timestamp) else list(hyp.timestamp or [])
    if isinstance(ts, dict):
        ts = ts.get("timestep", [])
    toks = tokenizer.ids_to_tokens([int(y) for y in ys])
    words: List[Dict[str, Any]] = []
    for tok, t in zip(toks, list(ts) + [ts[-1] if ts else 0] * (len(toks) - len(ts))):
        start = (int(t) + offset_frames) * frame_sec
        new = tok.startswith("▁") or not words
        piece = tok.replace("▁", "")
        if new:
            if not piece and tok == "▁":
                words.append({"word": "", "start_time": start, "end_time": start + frame_sec})
                continue
            words.append({"word": piece, "start_time": start, "end_time": start + frame_sec})
        else:
            words[-1]["word"] += piece
            words[-1]["end_time"] = start + frame_sec
    return [w for w in words if w["word"]]


# ------------------------------------------------------------------------------------------------ per-speaker streaming state
@dataclass
class _SpeakerInstance:
    speaker: int
    cache: Any                                                          # (cache_last_channel, cache_last_time, cache_last_channel_len)
    hypothesis: Any = None
    n_words_emitted: int = 0
    words: List[Dict[str, Any]] = field(default_factory=list)


class MultiTalkerInstanceManager:
    """One ASR instance per (session, speaker): created when a speaker first becomes active, from then on fed every chunk (with
    that speaker's mask) so that its encoder cache stays aligned with the recording."""

    def __init__(self, asr_model, max_num_of_spks: int = 4):
        self.asr, self.max_spks = asr_model, max_num_of_spks
        self.instances: Dict[int, _SpeakerInstance] = {}

    def reset(self):
        self.instances.clear()

    def get_speakers(self) -> List[int]:
        return sorted(self.instances)

    def add_speaker(self, speaker_id: int, template_cache=None):
        if speaker_id in self.instances or len(self.instances) >= self.max_spks:
            return
        dev = next(self.asr.parameters()).device
        cache = template_cache if template_cache is not None else self.asr.encoder.get_initial_cache_state(batch_size=1, device=dev)
        self.instances[speaker_id] = _SpeakerInstance(speaker_id, tuple(c.clone() for c in cache))

    def batched_caches(self, speakers: Sequence[int]):
        cs = [self.instances[s].cache for s in speakers]
        return (torch.cat([c[0] for c in cs], dim=1), torch.cat([c[1] for c in cs], dim=1), torch.cat([c[2] for c in cs], dim=0))

    def update(self, speakers: Sequence[int], caches, hyps):
        for i, s in enumerate(speakers):
            inst = self.instances[s]
            inst.cache = (caches[0][:, i:i + 1].clone(), caches[1][:, i:i + 1].clone(), caches[2][i:i + 1].clone())
            inst.hypothesis = hyps[i]


# ------------------------------------------------------------------------------------------------ the pipeline
class SpeakerTaggedASR:
    """``diarizer(audio [B, T], lens) -> activities [B, T', S]`` at the ASR encoder's frame rate (a ``SortformerEncLabelModel`` or
    any callable); ``asr_model``: an ``EncDecMultiTalkerRNNTBPEModel``."""

    def __init__(self, asr_model, diarizer: Callable, threshold: float = 0.5, min_active_frames: int = 3, max_num_of_spks: int = 4,
                 max_gap: float = 1.0, masked_asr: bool = False, frame_sec: Optional[float] = None):
        self.asr, self.diar = asr_model, diarizer
        self.threshold, self.min_active, self.max_spks, self.max_gap, self.masked_asr = threshold, min_active_frames, max_num_of_spks, max_gap, masked_asr
        pre = asr_model.preprocessor
        stride = getattr(pre, "window_stride", None) or getattr(getattr(pre, "featurizer", None), "hop_length", 160) / 16000.0
        self.frame_sec = frame_sec or float(stride) * int(asr_model.encoder.subsampling_factor)
        self.manager = MultiTalkerInstanceManager(asr_model, max_num_of_spks)

    @staticmethod
    def _targets(diar: torch.Tensor, spk: int) -> Tuple[torch.Tensor, torch.Tensor]:
        tgt = diar[..., spk]
        others = torch.cat([diar[..., :spk], diar[..., spk + 1:]], dim=-1)
        bg = others.max(dim=-1).values if others.shape[-1] else torch.zeros_like(tgt)
        return tgt, bg

    @torch.no_grad()
    def transcribe_offline(self, audio: torch.Tensor, lens: torch.Tensor, session_ids: Optional[Sequence[str]] = None) -> List[Dict[str, Any]]:
        asr = self.asr.eval()
        diar = self.diar(audio, lens).float()
        session_ids = list(session_ids) if session_ids is not None else [f"session_{b}" for b in range(audio.shape[0])]
        active = find_active_speakers(diar, self.threshold, self.min_active, self.max_spks)
        seglst: List[Dict[str, Any]] = []
        for b, spks in enumerate(active):
            for spk in spks:
                tgt, bg = self._targets(diar[b:b + 1], spk)
                if self.masked_asr:
                    feats, flen = asr.preprocessor(input_signal=audio[b:b + 1], length=lens[b:b + 1])
                    feats = mask_features(feats, tgt, subsampling=int(asr.encoder.subsampling_factor), threshold=self.threshold)
                    enc, enc_len = asr.forward(processed_signal=feats, processed_signal_length=flen)
                else:
                    asr.set_speaker_targets(tgt, bg)
                    try:
                        enc, enc_len = asr.forward(input_signal=audio[b:b + 1], input_signal_length=lens[b:b + 1])
                    finally:
                        asr.set_speaker_targets(None)
                hyp = asr.decoding.rnnt_decoder_predictions_tensor(encoder_output=enc.float(), encoded_lengths=enc_len, return_hypotheses=True)[0]
                words = _words_of(hyp, asr.tokenizer, self.frame_sec)
                seglst += sentences_from_words(words, session_ids[b], f"speaker_{spk}", self.max_gap)
        return sorted(seglst, key=lambda d: (d["session_id"], d["start_time"]))

    @torch.no_grad()
    def stream(self, audio: torch.Tensor, diar: Optional[torch.Tensor] = None, session_id: str = "session_0") -> List[Dict[str, Any]]:
        """One recording ``audio`` [T] chunk by chunk with the encoder's cache-aware geometry.  ``diar`` [T', S] may be given (e.g.
        from a streaming diarizer run alongside); otherwise the diarizer is called once on the whole signal and its output is
        consumed chunk by chunk.  Every speaker seen so far is one row of a batched encoder step; a speaker that appears late
        starts from an empty cache (its past was masked out anyway) and its word times are shifted to the recording's clock."""
        import math

        from .. import ops
        from ..utils.streaming_utils import CacheAwareStreamingAudioBuffer

        asr = self.asr.eval()
        self.manager.reset()
        dev = next(asr.parameters()).device
        audio = audio.reshape(-1).to(dev)
        if diar is None:
            diar = self.diar(audio[None], torch.tensor([audio.numel()], device=dev))[0]
        diar = diar.float().to(dev)
        if asr.encoder.streaming_cfg is None:
            asr.encoder.setup_streaming_params()
        buf = CacheAwareStreamingAudioBuffer(asr)
        buf.append_audio(audio)
        sf = int(asr.encoder.subsampling_factor)
        cfg = asr.encoder.streaming_cfg
        offset = 0
        for i, (feats, flens) in enumerate(buf):
            shift = cfg.shift_size[0 if i == 0 else 1] if isinstance(cfg.shift_size, (list, tuple)) else cfg.shift_size
            n_out = max(1, math.ceil(int(shift) / sf))
            d = diar[offset: offset + n_out][None]                      # [1, n_out, S]
            if d.shape[1] == 0:
                break
            for spk in find_active_speakers(d, self.threshold, 1, self.max_spks)[0]:
                if spk not in self.manager.instances:
                    self.manager.add_speaker(spk)
                    if spk in self.manager.instances:
                        self.manager.instances[spk].start_offset = offset
            spks = self.manager.get_speakers()
            if not spks:
                offset += n_out
                continue
            n = len(spks)
            tg = [self._targets(d, s) for s in spks]
            asr.set_speaker_targets(torch.cat([t for t, _ in tg], 0), torch.cat([b for _, b in tg], 0))
            try:
                clc, clt, clcl = self.manager.batched_caches(spks)
                with ops.compute_dtype(ops.get_compute_dtype()):
                    enc, enc_len, clc, clt, clcl = asr.encoder.cache_aware_stream_step(
                        processed_signal=feats.to(dev).expand(n, -1, -1).contiguous(), processed_signal_length=flens.to(dev).expand(n).contiguous(),
                        cache_last_channel=clc, cache_last_time=clt, cache_last_channel_len=clcl, keep_all_outputs=False,
                        drop_extra_pre_encoded=int(cfg.drop_extra_pre_encoded) if i > 0 else 0)
            finally:
                asr.set_speaker_targets(None)
            # decode the continuing speakers from their partial hypotheses and the new ones from scratch
            hyps: List[Any] = [None] * n
            for group in ([k for k, s in enumerate(spks) if self.manager.instances[s].hypothesis is not None],
                          [k for k, s in enumerate(spks) if self.manager.instances[s].hypothesis is None]):
                if not group:
                    continue
                idx = torch.tensor(group, device=dev)
                prev = [self.manager.instances[spks[k]].hypothesis for k in group]
                got = asr.decoding.rnnt_decoder_predictions_tensor(encoder_output=enc[idx].float(), encoded_lengths=enc_len[idx], return_hypotheses=True,
                                                                  partial_hypotheses=prev if prev[0] is not None else None)
                for k, h in zip(group, got):
                    hyps[k] = h
            self.manager.update(spks, (clc, clt, clcl), hyps)
            offset += int(enc_len.max())
        seglst: List[Dict[str, Any]] = []
        for s in self.manager.get_speakers():
            inst = self.manager.instances[s]
            if inst.hypothesis is None:
                continue
            words = _words_of(inst.hypothesis, asr.tokenizer, self.frame_sec, offset_frames=int(getattr(inst, "start_offset", 0)))
            seglst += sentences_from_words(words, session_id, f"speaker_{s}", self.max_gap)
        return sorted(seglst, key=lambda d: d["start_time"])


# ------------------------------------------------------------------------------------------------ training data
class SpeakerTargetDataset(torch.utils.data.Dataset):
    """Items of a multi-speaker corpus for speaker-kernel training.  Each example dict has ``audio`` (float array), ``segments``:
    ``[{"speaker", "start", "end", "text"}, ...]``.  One query speaker is drawn per access (the first when ``deterministic``):
    the text target is that speaker's segments in time order, ``spk_targets`` its frame-level activity and ``bg_spk_targets``
    the activity of everyone else, at ``frame_sec`` resolution."""

    def __init__(self, examples: Sequence[Dict[str, Any]], tokenizer, frame_sec: float = 0.08, sample_rate: int = 16000, deterministic: bool = False,
                 seed: int = 0):
        self.examples, self.tok, self.frame_sec, self.sr, self.det = list(examples), tokenizer, frame_sec, sample_rate, deterministic
        self.rng = np.random.default_rng(seed)

    def __len__(self):
        return len(self.examples)

    def __getitem__(self, i):
        ex = self.examples[i]
        audio = np.asarray(ex["audio"], dtype=np.float32)
        T = int(np.ceil(len(audio) / self.sr / self.frame_sec))
        speakers = sorted({s["speaker"] for s in ex["segments"]})
        q = speakers[0] if self.det else speakers[int(self.rng.integers(len(speakers)))]
        tgt, bg = np.zeros(T, dtype=np.float32), np.zeros(T, dtype=np.float32)
        for s in ex["segments"]:
            a, b = int(round(s["start"] / self.frame_sec)), min(T, int(round(s["end"] / self.frame_sec)))
            (tgt if s["speaker"] == q else bg)[a:b] = 1.0
        text = " ".join(s["text"] for s in sorted(ex["segments"], key=lambda s: s["start"]) if s["speaker"] == q)
        ids = self.tok.text_to_ids(text)
        return torch.from_numpy(audio), torch.tensor(ids, dtype=torch.long), torch.from_numpy(tgt), torch.from_numpy(bg)

    @staticmethod
    def collate(items):
        pad = torch.nn.utils.rnn.pad_sequence
        a, t, s, b = zip(*items)
        return (pad(a, batch_first=True), torch.tensor([len(x) for x in a]), pad(t, batch_first=True), torch.tensor([len(x) for x in t]),
                pad(s, batch_first=True), pad(b, batch_first=True))

"""Streaming recognition pipelines.

``BasePipeline.run`` drives a ``ContinuousBatchedRequestStreamer``: at every step up to ``batch_size`` live streams each
contribute one chunk; ``transcribe_step`` advances all of them together and finished streams are replaced by waiting ones
(reference: ``inference/pipelines/base_pipeline.py:569-604``).  Two families:

* cache-aware (``CacheAwareRNNTPipeline``, ``CacheAwareCTCPipeline``): the encoder runs chunk by chunk with attention /
  convolution caches held in a slot pool (``CacheAwareContextManager``) and the decoder continues from its previous state,
* buffered (``BufferedRNNTPipeline``, ``BufferedCTCPipeline``): every step re-encodes the last ``buffer_size`` seconds
  offline and keeps the tokens that fall into the newest chunk shifted back by the right-context delay.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..core.config import DictConfig, OmegaConf
from .bufferer import AudioBufferer
from .context_manager import CacheAwareContextManager
from .framing import ASRRequestOptions, ContinuousBatchedRequestStreamer, FeatureBuffer, Frame, RequestType
from .state import GreedyEndpointing, StreamingState, TextSegment, TokenTextAssembler, Word
from .wrappers import ASRInferenceWrapper, CacheAwareASRInferenceWrapper


def _get(cfg, path: str, default=None):
    cur = cfg
    for k in path.split("."):
        if cur is None:
            return default
        cur = cur.get(k, None) if hasattr(cur, "get") else getattr(cur, k, None)
    return default if cur is None else cur


@dataclass
class PipelineOutput:
    stream_id: int
    text: str = ""
    words: List[Word] = field(default_factory=list)
    segments: List[TextSegment] = field(default_factory=list)
    partial_text: str = ""

    def to_dict(self) -> Dict[str, Any]:
        return {"stream_id": self.stream_id, "text": self.text, "words": [w.to_dict() for w in self.words],
                "segments": [{"text": s.text, "start": round(s.start, 3), "end": round(s.end, 3)} for s in self.segments]}


class BasePipeline:
    request_type = RequestType.FRAME

    def __init__(self):
        self._states: Dict[int, StreamingState] = {}
        self._outputs: Dict[int, PipelineOutput] = {}
        self.step_times: List[float] = []

    # ------------------------------------------------------------------ state pool
    def get_state(self, stream_id: int, options: Optional[ASRRequestOptions] = None) -> StreamingState:
        st = self._states.get(stream_id)
        if st is None:
            st = StreamingState(stream_id, options)
            self._states[stream_id] = st
        return st

    def delete_state(self, stream_id: int) -> None:
        self._states.pop(stream_id, None)

    def open_session(self) -> None:
        self._states.clear()
        self._outputs.clear()
        self.step_times = []

    def close_session(self) -> None:
        self._states.clear()

    # ------------------------------------------------------------------ subclasses
    def get_request_generator(self) -> ContinuousBatchedRequestStreamer:
        raise NotImplementedError

    def transcribe_step(self, requests) -> None:
        raise NotImplementedError

    # ------------------------------------------------------------------ text bookkeeping shared by all pipelines
    def _finalize_utterance(self, st: StreamingState) -> None:
        seg = self.text.segment(st.tokens, st.timesteps, st.confidences)
        if seg is not None:
            st.final_segments.append(seg)
            st.final_transcript = (st.final_transcript + " " + seg.text).strip()
        st.cleanup_after_eou()
        st.hypothesis = None
        st.last_ctc_token = None

    def _after_tokens(self, st: StreamingState, is_last: bool) -> None:
        st.partial_transcript = self.text.ids_to_text(st.tokens).strip() if st.tokens else ""
        if self.endpointer.detect_eou(st, is_last=is_last):
            self._finalize_utterance(st)
        out = self._outputs.setdefault(st.stream_id, PipelineOutput(st.stream_id))
        out.text = st.get_transcript()
        out.partial_text = st.partial_transcript
        out.segments = list(st.final_segments)
        out.words = [w for s in st.final_segments for w in s.words]
        if is_last:
            st.is_finished = True
            self.delete_state(st.stream_id)

    # ------------------------------------------------------------------ driver
    def run(self, audio: Sequence[Any], options: Optional[Sequence[Optional[ASRRequestOptions]]] = None,
            progress_callback=None) -> Dict[int, PipelineOutput]:
        """Transcribe all sources as simulated live streams.  Returns ``{stream index: PipelineOutput}``."""
        self.open_session()
        gen = self.get_request_generator()
        gen.set_audio_filepaths(audio, options)
        for requests in gen:
            t0 = time.perf_counter()
            self.transcribe_step(requests)
            self.step_times.append(time.perf_counter() - t0)
            if progress_callback is not None:
                progress_callback(requests)
        self.audio_durations = gen.get_audio_durations()
        self.close_session()
        return dict(self._outputs)

    def rtfx(self) -> float:
        """Audio seconds processed per second of ``transcribe_step`` time of the last ``run``."""
        total = sum(self.step_times)
        return sum(getattr(self, "audio_durations", {}).values()) / total if total > 0 else float("nan")


# ====================================================================================== cache-aware pipelines
class _CacheAwarePipeline(BasePipeline):
    request_type = RequestType.FEATURE_BUFFER

    def __init__(self, cfg, asr_model: CacheAwareASRInferenceWrapper):
        super().__init__()
        cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg or {})
        self.cfg, self.asr_model = cfg, asr_model
        att = _get(cfg, "streaming.att_context_size", None)
        if att is not None:
            asr_model.set_default_att_context_size(list(att))
        self.sample_rate = int(_get(cfg, "streaming.sample_rate", asr_model.sample_rate))
        self.batch_size = int(_get(cfg, "streaming.batch_size", 64))
        self.num_slots = max(int(_get(cfg, "streaming.num_slots", 256)), self.batch_size)
        self.use_cache = bool(_get(cfg, "streaming.use_cache", True))
        self.chunk_frames = asr_model.shift_feature_frames(first=False)       # new feature frames per step
        self.first_chunk_frames = asr_model.shift_feature_frames(first=True)
        self.pre_cache = asr_model.pre_encode_cache_frames()
        self.drop_extra = asr_model.drop_extra_pre_encoded()
        self.chunk_samples = self.chunk_frames * asr_model.hop_length
        self.buffer_secs = float(_get(cfg, "streaming.buffer_size_in_secs",
                                      (self.chunk_frames + self.pre_cache + 2) * asr_model.window_stride + 0.05))
        self.context_manager = CacheAwareContextManager(asr_model, self.num_slots, self.use_cache, device=asr_model.device)
        self.endpointer = GreedyEndpointing(ms_per_frame=asr_model.seconds_per_timestep * 1e3,
                                            stop_history_eou_ms=int(_get(cfg, "endpointing.stop_history_eou", 800)))
        self.text = TokenTextAssembler(asr_model.ids_to_tokens, asr_model.ids_to_text, asr_model.seconds_per_timestep,
                                       confidence_aggregation=_get(cfg, "confidence.aggregation", "mean"))

    def open_session(self) -> None:
        super().open_session()
        self.context_manager.reset()

    def get_request_generator(self) -> ContinuousBatchedRequestStreamer:
        from .bufferer import BatchedCacheFeatureBufferer

        buf = BatchedCacheFeatureBufferer(sample_rate=self.sample_rate, buffer_size_in_secs=self.buffer_secs,
                                          chunk_size_in_secs=self.chunk_samples / self.sample_rate,
                                          preprocessor=self.asr_model.asr_model.preprocessor, device=self.asr_model.device,
                                          pre_encode_cache_frames=self.pre_cache, first_chunk_frames=self.first_chunk_frames)
        return ContinuousBatchedRequestStreamer(n_frames_per_stream=self.chunk_samples, batch_size=self.batch_size,
                                                sample_rate=self.sample_rate, request_type=RequestType.FEATURE_BUFFER,
                                                bufferer=buf)

    def _run_group(self, reqs: List[FeatureBuffer], first: bool) -> None:
        ids = [r.stream_id for r in reqs]
        states = [self.get_state(r.stream_id, r.options) for r in reqs]
        T = max(r.size for r in reqs)
        # padding launches a kernel per stream: only for the (rare) streams whose chunk is shorter than the longest one
        feats = torch.stack([r.features if r.size == T else torch.nn.functional.pad(r.features, (0, T - r.size)) for r in reqs])
        lens = torch.tensor([r.valid_size for r in reqs], dtype=torch.long)
        ctx, mapping = self.context_manager.get_context(ids)
        result = self._decode_group(feats, lens, ctx, states, drop_extra=0 if first else self.drop_extra)
        new_ctx, enc_lens = result
        self.context_manager.update_cache(ids, new_ctx, mapping)
        for st, r, n in zip(states, reqs, enc_lens.tolist()):
            st.advance(int(n))
            self._after_tokens(st, is_last=r.is_last)
        self.context_manager.reset_slots(ids, [r.is_last for r in reqs])

    def transcribe_step(self, requests: List[FeatureBuffer]) -> None:
        first = [r for r in requests if r.is_first]
        rest = [r for r in requests if not r.is_first]
        # the first chunk of a stream has no pre-encode cache in front of it and must not drop encoder frames
        if first:
            self._run_group(first, first=True)
        if rest:
            self._run_group(rest, first=False)

    def _decode_group(self, feats, lens, ctx, states, drop_extra):
        raise NotImplementedError


class CacheAwareRNNTPipeline(_CacheAwarePipeline):
    """Greedy by default; ``asr.decoding.strategy: malsd_batch`` (with ``asr.decoding.beam.beam_size``) keeps a beam per stream
    between chunks, and the stream's running transcript is the beam's best entry."""

    def __init__(self, cfg, asr_model):
        super().__init__(cfg, asr_model)
        self.malsd = None
        if str(_get(self.cfg, "asr.decoding.strategy", "greedy_batch")) == "malsd_batch":
            self.malsd = asr_model.build_malsd_computer(beam_size=int(_get(self.cfg, "asr.decoding.beam.beam_size", 4)),
                                                        max_symbols_per_step=int(_get(self.cfg, "asr.decoding.beam.max_symbols_per_step", 10)))

    def _decode_group_beam(self, feats, lens, ctx, states, drop_extra):
        carries = [s.hypothesis for s in states]
        for st in states:
            if st.hypothesis is None:
                st.extra["utt_base"] = st.frame_offset          # utterance-local frame indices are shifted to the stream's clock
        best, new_ctx, enc_lens, new = self.asr_model.malsd_stream_step(self.malsd, feats, lens, ctx, carries, drop_extra_pre_encoded=drop_extra)
        for st, (toks, frames, _), c in zip(states, best, new):
            base = int(st.extra.get("utt_base", 0))
            st.tokens, st.timesteps = [int(t) for t in toks], [int(f) + base for f in frames]
            st.confidences = [1.0] * len(toks)
            st.last_emit_frame = st.timesteps[-1] if toks else -1
            st.hypothesis = c
        return new_ctx, enc_lens

    def _decode_group(self, feats, lens, ctx, states, drop_extra):
        if self.malsd is not None:
            return self._decode_group_beam(feats, lens, ctx, states, drop_extra)
        prev = [s.hypothesis for s in states]
        prev = prev if any(p is not None for p in prev) else None
        hyps, new_ctx, enc_lens, _ = self.asr_model.stream_step(feats, lens, ctx, previous_hypotheses=prev,
                                                                drop_extra_pre_encoded=drop_extra)
        for st, h in zip(states, hyps):
            seen = int(st.extra.get("rnnt_seen", 0)) if st.hypothesis is not None else 0
            ys = [int(t) for t in h.y_sequence.tolist()] if torch.is_tensor(h.y_sequence) else [int(t) for t in h.y_sequence]
            ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp)
            base = st.frame_offset if st.hypothesis is None else 0
            st.append_tokens(ys[seen:], [int(t) + base for t in ts[seen:]])
            if st.hypothesis is None and base:
                # a new utterance inside a running stream: shift the hypothesis' clock to the stream's clock
                h.timestamp = (torch.as_tensor(h.timestamp) + base)
                h.last_frame = base + int(h.last_frame or 0)
            st.hypothesis = h
            st.extra["rnnt_seen"] = len(ys)
        return new_ctx, enc_lens


class CacheAwareCTCPipeline(_CacheAwarePipeline):
    def _decode_group(self, feats, lens, ctx, states, drop_extra):
        _, new_ctx, enc_lens, frame_preds = self.asr_model.stream_step(feats, lens, ctx, previous_pred_out=None,
                                                                      drop_extra_pre_encoded=drop_extra)
        blank = self.asr_model.blank_id
        for st, preds, n in zip(states, frame_preds, enc_lens.tolist()):
            toks, times = [], []
            last = st.last_ctc_token
            for t, p in enumerate(preds[: int(n)].tolist()):
                if p != blank and p != last:
                    toks.append(p)
                    times.append(st.frame_offset + t)
                last = p
            st.last_ctc_token = last
            st.append_tokens(toks, times)
        return new_ctx, enc_lens


# ====================================================================================== buffered pipelines
class _BufferedPipeline(BasePipeline):
    def __init__(self, cfg, asr_model: ASRInferenceWrapper):
        super().__init__()
        cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg or {})
        self.cfg, self.asr_model = cfg, asr_model
        self.sample_rate = int(_get(cfg, "streaming.sample_rate", asr_model.sample_rate))
        self.batch_size = int(_get(cfg, "streaming.batch_size", 32))
        self.chunk_secs = float(_get(cfg, "streaming.chunk_size", 1.6))
        self.left_secs = float(_get(cfg, "streaming.left_padding_size", 1.6))
        self.right_secs = float(_get(cfg, "streaming.right_padding_size", 1.6))
        self.buffer_secs = self.chunk_secs + self.left_secs + self.right_secs
        self.chunk_samples = int(round(self.chunk_secs * self.sample_rate))
        spt = asr_model.seconds_per_timestep
        self.tokens_per_chunk = int(math.ceil(self.chunk_secs / spt))
        self.right_frames = int(round(self.right_secs / spt))
        self.buffer_frames = int(round(self.buffer_secs / spt))
        self.bufferer = AudioBufferer(self.sample_rate, self.buffer_secs)
        self.endpointer = GreedyEndpointing(ms_per_frame=spt * 1e3,
                                            stop_history_eou_ms=int(_get(cfg, "endpointing.stop_history_eou", 800)))
        self.text = TokenTextAssembler(asr_model.ids_to_tokens, asr_model.ids_to_text, spt,
                                       confidence_aggregation=_get(cfg, "confidence.aggregation", "mean"))

    def open_session(self) -> None:
        super().open_session()
        self.bufferer.reset()

    def get_request_generator(self) -> ContinuousBatchedRequestStreamer:
        # pad the tail so the last real chunk also travels through the right-context delay
        return ContinuousBatchedRequestStreamer(n_frames_per_stream=self.chunk_samples, batch_size=self.batch_size,
                                                sample_rate=self.sample_rate, request_type=RequestType.FRAME,
                                                tail_padding_in_samples=int(round(self.right_secs * self.sample_rate)))

    def _window_range(self, n_frames: int):
        """Encoder-frame range of a window that belongs to the newest chunk delayed by the right context."""
        hi = max(0, n_frames - self.right_frames)
        lo = max(0, hi - self.tokens_per_chunk)
        return lo, hi

    def transcribe_step(self, requests: List[Frame]) -> None:
        states = [self.get_state(r.stream_id, r.options) for r in requests]
        windows, _ = self.bufferer.update(requests)
        lens = torch.full((windows.shape[0],), windows.shape[1], dtype=torch.long)
        enc, enc_len = self.asr_model.encode_windows(windows, lens)
        self._decode_windows(enc, enc_len, states)
        for st, r in zip(states, requests):
            st.advance(self.tokens_per_chunk)
            self._after_tokens(st, is_last=r.is_last)

    def _decode_windows(self, enc, enc_len, states):
        raise NotImplementedError


class BufferedCTCPipeline(_BufferedPipeline):
    def _decode_windows(self, enc, enc_len, states):
        pred, conf = self.asr_model.ctc_frame_predictions(enc)
        blank = self.asr_model.blank_id
        for b, st in enumerate(states):
            n = int(enc_len[b])
            lo, hi = self._window_range(n)
            last = st.last_ctc_token
            toks, times, confs = [], [], []
            for k, t in enumerate(range(lo, hi)):
                p = int(pred[b, t])
                if p != blank and p != last:
                    toks.append(p)
                    times.append(max(0, st.frame_offset - self.right_frames + k))
                    confs.append(float(conf[b, t]))
                last = p
            st.last_ctc_token = last
            st.append_tokens(toks, times, confs)


class BufferedRNNTPipeline(_BufferedPipeline):
    def _decode_windows(self, enc, enc_len, states):
        hyps = self.asr_model.rnnt_decode(enc, enc_len)
        for b, (st, h) in enumerate(zip(states, hyps)):
            n = int(enc_len[b])
            lo, hi = self._window_range(n)
            ys = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
            ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp)
            toks = [int(y) for y, t in zip(ys, ts) if lo <= int(t) < hi]
            times = [max(0, st.frame_offset - self.right_frames + (int(t) - lo)) for t in ts if lo <= int(t) < hi]
            st.append_tokens(toks, times)


def merge_by_word_overlap(committed: List[str], new: List[str], max_overlap: int = 12) -> List[str]:
    """Join two word sequences whose end / start overlap: the longest suffix of ``committed`` that is a prefix of ``new`` is kept
    once (windows of a sliding buffer re-transcribe the words of their shared audio)."""
    for n in range(min(max_overlap, len(committed), len(new)), 0, -1):
        if committed[-n:] == new[:n]:
            return committed + new[n:]
    return committed + new


class BufferedSALMPipeline(BasePipeline):
    """Speech-LLM transcription of live streams: every step the model is prompted with the stream's current audio window
    (``left context | new chunk``) and asked for the transcript; the window's words are merged into the running transcript by
    their overlap with what earlier windows already produced, and words become final once the audio they came from has left the
    window (reference: ``inference/pipelines/buffered_salm_pipeline.py``).  ``salm`` needs ``generate(dialogs, audios,
    audio_lens, max_new_tokens)`` and a tokenizer with ``ids_to_text``."""

    def __init__(self, cfg, salm):
        super().__init__()
        cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg or {})
        self.cfg, self.salm = cfg, salm
        self.sample_rate = int(_get(cfg, "streaming.sample_rate", 16000))
        self.batch_size = int(_get(cfg, "streaming.batch_size", 8))
        self.chunk_secs = float(_get(cfg, "streaming.chunk_size", 2.0))
        self.left_secs = float(_get(cfg, "streaming.left_padding_size", 6.0))
        self.chunk_samples = int(round(self.chunk_secs * self.sample_rate))
        self.window_samples = int(round((self.chunk_secs + self.left_secs) * self.sample_rate))
        self.prompt = str(_get(cfg, "salm.prompt", "Transcribe the following: " + getattr(salm, "audio_locator_tag", "<|audioplaceholder|>")))
        self.max_new_tokens = int(_get(cfg, "salm.max_new_tokens", 64))
        self.bufferer = AudioBufferer(self.sample_rate, self.chunk_secs + self.left_secs)

    def open_session(self) -> None:
        super().open_session()
        self.bufferer.reset()

    def get_request_generator(self) -> ContinuousBatchedRequestStreamer:
        return ContinuousBatchedRequestStreamer(n_frames_per_stream=self.chunk_samples, batch_size=self.batch_size,
                                                sample_rate=self.sample_rate, request_type=RequestType.FRAME)

    def _ids_to_text(self, ids) -> str:
        tok = self.salm.tokenizer
        stop = {getattr(self.salm, "text_eos_id", -1), getattr(self.salm, "text_pad_id", -1)}
        ids = [int(t) for t in ids if int(t) not in stop]
        return tok.ids_to_text(ids) if ids else ""

    def transcribe_step(self, requests: List[Frame]) -> None:
        states = [self.get_state(r.stream_id, r.options) for r in requests]
        windows, left_pad = self.bufferer.update(requests)
        audios, lens = [], []
        for b in range(windows.shape[0]):
            tail = max(0, int(requests[b].size) - int(requests[b].length))   # zero padding of a short last chunk
            a = windows[b, int(left_pad[b]): windows.shape[1] - tail]   # only the audio heard so far
            audios.append(a)
            lens.append(a.shape[0])
        n = max(lens)
        batch = torch.stack([torch.nn.functional.pad(a, (0, n - a.shape[0])) for a in audios])
        dialogs = [[{"role": "user", "content": self.prompt}] for _ in requests]
        out = self.salm.generate(dialogs, audios=batch, audio_lens=torch.tensor(lens), max_new_tokens=self.max_new_tokens)
        for st, r, ids in zip(states, requests, out):
            words = self._ids_to_text(ids.tolist()).split()
            merged = merge_by_word_overlap(st.extra.get("salm_words", []), words)
            st.extra["salm_words"] = merged
            res = self._outputs.setdefault(st.stream_id, PipelineOutput(st.stream_id))
            res.text = res.partial_text = " ".join(merged)
            if r.is_last:
                st.is_finished = True
                self.delete_state(st.stream_id)


# ====================================================================================== builder
class PipelineBuilder:
    """``cfg.pipeline_type`` ∈ {cache_aware, buffered}; ``cfg.asr_decoding_type`` ∈ {rnnt, ctc} (auto from the model when
    absent).  ``cfg.asr.model_name`` may be a ``.nemo`` path; a model instance can be passed instead."""

    @staticmethod
    def build_pipeline(cfg, asr_model=None) -> BasePipeline:
        cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg or {})
        if asr_model is None:
            from ..models.asr_model import ASRModel

            asr_model = ASRModel.restore_from(_get(cfg, "asr.model_name"), map_location=_get(cfg, "asr.device", None))
        from .enums import PipelineType

        kind = PipelineType.from_str(_get(cfg, "pipeline_type", "cache_aware")).name.lower()      # rejects unknown names with the list of choices
        dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": None, None: None}[
            _get(cfg, "asr.compute_dtype", None) if _get(cfg, "asr.compute_dtype", None) in ("bfloat16", "float16") else None]
        device = _get(cfg, "asr.device", None)
        if kind == "cache_aware":
            from ..models.ctc_models import EncDecCTCModel
            from .wrappers import CacheAwareCTCInferenceWrapper, CacheAwareRNNTInferenceWrapper

            dec = (_get(cfg, "asr_decoding_type", None) or getattr(asr_model, "cur_decoder", None)
                   or ("ctc" if isinstance(asr_model, EncDecCTCModel) else "rnnt"))
            dcfg = _get(cfg, "asr.decoding", None)
            if dec == "rnnt" and dcfg is not None and str(_get(cfg, "asr.decoding.strategy", "")) == "malsd_batch":
                dcfg = None                        # the pipeline owns the beam search; the model's own decoding stays greedy
            w = (CacheAwareRNNTInferenceWrapper if dec == "rnnt" else CacheAwareCTCInferenceWrapper)(
                asr_model, device, dtype, dcfg, _get(cfg, "streaming.att_context_size", None))
            return (CacheAwareRNNTPipeline if dec == "rnnt" else CacheAwareCTCPipeline)(cfg, w)
        if kind == "buffered":
            w = ASRInferenceWrapper(asr_model, device, dtype, _get(cfg, "asr.decoding", None))
            dec = _get(cfg, "asr_decoding_type", None) or w.decoder_type
            return (BufferedRNNTPipeline if dec == "rnnt" else BufferedCTCPipeline)(cfg, w)
        raise ValueError(f"unknown pipeline_type {kind}")

    @staticmethod
    def build_salm_pipeline(cfg, salm) -> BasePipeline:
        return BufferedSALMPipeline(cfg, salm)

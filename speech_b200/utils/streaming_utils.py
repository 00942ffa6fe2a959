"""Classic chunked / buffered inference helpers (the API older scripts use).

* ``CacheAwareStreamingAudioBuffer`` — features of whole recordings computed once, then iterated chunk by chunk with the
  pre-encode cache prepended (``parts/utils/streaming_utils.py:1250-1520`` of the reference).
* ``FrameBatchASR`` / ``BatchedFrameASRRNNT`` — fixed-size frames with left/right context buffers; CTC keeps the
  middle tokens of every buffer, the transducer variant merges consecutive buffers by longest common subsequence or keeps
  the middle tokens (``:381-1250``).
* ``longest_common_subsequence_merge`` (``:30-230``) and ``ContextSize`` helpers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterator, List, Optional, Tuple

import numpy as np
import torch


@dataclass
class ContextSize:
    left: int
    chunk: int
    right: int

    def total(self) -> int:
        return self.left + self.chunk + self.right

    def subsample(self, factor: int) -> "ContextSize":
        return ContextSize(self.left // factor, self.chunk // factor, self.right // factor)

    def add_frames_get_removed_(self, num_frames: int, is_last_chunk: bool, expected_next_chunk: int = 0) -> int:
        """Grow the left context by the frames of the chunk just consumed; returns how many old frames fall out."""
        total_before = self.total()
        self.left += self.chunk
        self.chunk = num_frames if not is_last_chunk else num_frames
        removed = max(0, self.left + self.chunk + self.right - total_before)
        self.left -= removed
        return removed


def longest_common_subsequence_merge(X: List[int], Y: List[int], filepath: Optional[str] = None) -> Tuple[int, int, int, np.ndarray]:
    """Longest common *contiguous* alignment between the tail of ``X`` and the head of ``Y``.
    Returns ``(i, j, length, table)``: the match starts at ``X[i]`` and ``Y[j]`` and spans ``length`` tokens."""
    m, n = len(X), len(Y)
    L = np.zeros((m + 1, n + 1), dtype=np.int32)
    best, bi, bj = 0, 0, 0
    for i in range(1, m + 1):
        for j in range(1, n + 1):
            if X[i - 1] == Y[j - 1]:
                L[i, j] = L[i - 1, j - 1] + 1
                # prefer matches late in X and early in Y (the overlap region)
                if L[i, j] > best or (L[i, j] == best and (i - j) > (bi - bj)):
                    best, bi, bj = int(L[i, j]), i, j
    return bi - best, bj - best, best, L


def lcs_alignment_merge_buffer(buffer: List[int], data: List[int], delay: int, model=None, max_steps_per_timestep: int = 5,
                               min_lcs_length: int = 1, **_) -> List[int]:
    """Append ``data`` to ``buffer`` where the last ``delay`` tokens of the buffer overlap the head of ``data``."""
    if not buffer:
        return list(data)
    if delay < 1 or not data:
        return list(buffer) + list(data)
    search = delay * max_steps_per_timestep
    tail = buffer[-search:]
    head = data[:search]
    i, j, length, _ = longest_common_subsequence_merge(tail, head)
    if length < min_lcs_length:
        return list(buffer) + list(data)
    cut = len(buffer) - len(tail) + i + length
    return list(buffer[:cut]) + list(data[j + length:])


class CacheAwareStreamingAudioBuffer:
    """Holds the features of several recordings and yields ``(chunk_features [B, F, T], chunk_lengths [B])`` with the
    geometry of the model's encoder (``streaming_cfg``): first chunk ``chunk_size[0]`` frames without cache, later chunks
    ``chunk_size[1]`` frames preceded by ``pre_encode_cache_size`` cached frames, advancing by ``shift_size``."""

    def __init__(self, model, online_normalization: bool = False, pad_and_drop_preencoded: bool = False):
        self.model = model
        self.online_normalization = online_normalization
        self.pad_and_drop_preencoded = pad_and_drop_preencoded
        self.streaming_cfg = model.encoder.streaming_cfg
        self.preprocessor = model.preprocessor
        self.input_features = int(model.encoder._feat_in)
        self.reset_buffer()

    def reset_buffer(self):
        self.buffer: Optional[torch.Tensor] = None
        self.streams_length: Optional[torch.Tensor] = None
        self.buffer_idx = 0
        self.step = 0

    def __len__(self):
        return 0 if self.buffer is None else int(self.buffer.shape[0])

    @torch.no_grad()
    def append_audio(self, audio, stream_id: int = -1):
        x = torch.as_tensor(audio, dtype=torch.float32).reshape(1, -1)
        dev = next(self.model.parameters()).device
        feats, flen = self.preprocessor(input_signal=x.to(dev), length=torch.tensor([x.shape[1]], device=dev))
        return self.append_processed_signal(feats, stream_id), flen

    def append_audio_file(self, path: str, stream_id: int = -1):
        from ..data.audio_to_text import load_audio

        return self.append_audio(load_audio(path), stream_id)

    def append_processed_signal(self, feats: torch.Tensor, stream_id: int = -1) -> int:
        T = feats.shape[-1]
        if self.buffer is None:
            self.buffer = feats
            self.streams_length = torch.tensor([T], device=feats.device)
            return 0
        if stream_id >= 0:
            raise NotImplementedError("appending to an existing stream is not supported")
        W = max(self.buffer.shape[-1], T)
        self.buffer = torch.cat([torch.nn.functional.pad(self.buffer, (0, W - self.buffer.shape[-1])),
                                 torch.nn.functional.pad(feats, (0, W - T))], dim=0)
        self.streams_length = torch.cat([self.streams_length, torch.tensor([T], device=feats.device)])
        return self.buffer.shape[0] - 1

    def is_buffer_empty(self) -> bool:
        return self.buffer is None or self.buffer_idx >= self.buffer.shape[-1]

    @staticmethod
    def _pick(v, first):
        return (v[0] if first else v[1]) if isinstance(v, (list, tuple)) else v

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        cfg = self.streaming_cfg
        while not self.is_buffer_empty():
            first = self.buffer_idx == 0
            chunk = self._pick(cfg.chunk_size, first)
            shift = self._pick(cfg.shift_size, first)
            cache = 0 if first else self._pick(cfg.pre_encode_cache_size, False)
            lo, hi = self.buffer_idx - cache, self.buffer_idx + chunk
            x = self.buffer[:, :, max(0, lo):hi]
            if lo < 0:
                x = torch.nn.functional.pad(x, (-lo, 0))
            if first and self.pad_and_drop_preencoded:
                c = self._pick(cfg.pre_encode_cache_size, False)
                x = torch.nn.functional.pad(x, (c, 0))
                cache = c
            lens = (self.streams_length - self.buffer_idx).clamp(min=0, max=chunk) + cache
            lens = torch.where(self.streams_length > self.buffer_idx, lens, torch.zeros_like(lens))
            self.buffer_idx += shift
            self.step += 1
            yield x, lens

    def get_all_audios(self):
        return self.buffer, self.streams_length


class FrameBatchASR:
    """Buffered CTC decoding of one long recording: frames of ``frame_len`` seconds inside a ``total_buffer`` second
    window; per window the frame-level argmax of the middle ``tokens_per_chunk`` steps is kept and the collected sequence
    is collapsed once at the end."""

    def __init__(self, asr_model, frame_len: float = 1.6, total_buffer: float = 4.0, batch_size: int = 4,
                 pad_to_buffer_len: bool = True):
        self.asr_model = asr_model
        self.frame_len, self.total_buffer, self.batch_size = frame_len, total_buffer, batch_size
        pre = asr_model.preprocessor
        feat = getattr(pre, "featurizer", pre)
        self.sr = int(getattr(feat, "sample_rate", 16000))
        self.stride = feat.hop_length / self.sr * asr_model.encoder.subsampling_factor
        self.tokens_per_chunk = int(math.ceil(frame_len / self.stride))
        self.delay = int(math.ceil((frame_len + (total_buffer - frame_len) / 2) / self.stride))
        self.blank_id = int((asr_model.ctc_decoding if hasattr(asr_model, "ctc_decoding") else asr_model.decoding).blank_id)
        self.reset()

    def reset(self):
        self.all_preds: List[torch.Tensor] = []
        self.samples: Optional[torch.Tensor] = None

    def read_audio_file(self, path_or_array, delay=None, model_stride_in_secs=None):
        if isinstance(path_or_array, str):
            from ..data.audio_to_text import load_audio

            path_or_array = load_audio(path_or_array, target_sr=self.sr)
        self.samples = torch.as_tensor(path_or_array, dtype=torch.float32).reshape(-1)

    def _windows(self):
        n_frame = int(self.frame_len * self.sr)
        n_buf = int(self.total_buffer * self.sr)
        pad = (n_buf - n_frame) // 2
        x = torch.nn.functional.pad(self.samples, (n_buf - n_frame, pad + n_frame))
        k = 0
        while k * n_frame < self.samples.numel() + pad:
            yield x[k * n_frame: k * n_frame + n_buf]
            k += 1

    @torch.no_grad()
    def infer_logits(self):
        dev = next(self.asr_model.parameters()).device
        m = self.asr_model
        dec = m.ctc_decoder if hasattr(m, "ctc_decoder") else m.decoder
        batch = []
        for w in self._windows():
            batch.append(w)
            if len(batch) == self.batch_size:
                self._run(batch, dev, dec)
                batch = []
        if batch:
            self._run(batch, dev, dec)

    def _run(self, batch, dev, dec):
        x = torch.stack(batch).to(dev)
        lens = torch.full((x.shape[0],), x.shape[1], device=dev, dtype=torch.long)
        feats, flen = self.asr_model.preprocessor(input_signal=x, length=lens)
        enc, _ = self.asr_model.encoder(audio_signal=feats, length=flen)
        lp = dec(encoder_output=enc)
        for p in lp.argmax(dim=-1).cpu():
            self.all_preds.append(p)

    def transcribe(self, tokens_per_chunk: Optional[int] = None, delay: Optional[int] = None, keep_logits: bool = False):
        self.infer_logits()
        tpc = tokens_per_chunk or self.tokens_per_chunk
        delay = delay or self.delay
        kept: List[int] = []
        for p in self.all_preds:
            n = len(p)
            kept.extend(p[max(0, n - 1 - delay): max(0, n - 1 - delay) + tpc].tolist())
        out, prev = [], self.blank_id
        for t in kept:
            if t != prev and t != self.blank_id:
                out.append(t)
            prev = t
        decoding = self.asr_model.ctc_decoding if hasattr(self.asr_model, "ctc_decoding") else self.asr_model.decoding
        return decoding.decode_tokens_to_str(out)


class BatchedFrameASRRNNT(FrameBatchASR):
    """Transducer variant: every window is decoded greedily; consecutive windows are merged with
    ``lcs_alignment_merge_buffer`` (``merge_algo='lcs'``) or by keeping the tokens whose frames fall into the middle chunk
    (``merge_algo='middle'``)."""

    def __init__(self, asr_model, frame_len=1.6, total_buffer=4.0, batch_size=4, max_steps_per_timestep: int = 5,
                 stateful_decoding: bool = False, merge_algo: str = "middle"):
        super().__init__(asr_model, frame_len, total_buffer, batch_size)
        self.blank_id = int(asr_model.decoding.blank_id)
        self.max_steps_per_timestep = max_steps_per_timestep
        self.merge_algo = merge_algo
        self.hyps = []

    def reset(self):
        super().reset()
        self.hyps = []

    def _run(self, batch, dev, dec):
        x = torch.stack(batch).to(dev)
        lens = torch.full((x.shape[0],), x.shape[1], device=dev, dtype=torch.long)
        feats, flen = self.asr_model.preprocessor(input_signal=x, length=lens)
        enc, enc_len = self.asr_model.encoder(audio_signal=feats, length=flen)
        hyps = self.asr_model.decoding.rnnt_decoder_predictions_tensor(enc, enc_len, return_hypotheses=True)
        for h, n in zip(hyps, enc_len.tolist()):
            self.hyps.append((h, int(n)))

    def transcribe(self, tokens_per_chunk: Optional[int] = None, delay: Optional[int] = None, **_):
        self.infer_logits()
        tpc = tokens_per_chunk or self.tokens_per_chunk
        delay = delay or self.delay
        merged: List[int] = []
        for h, n in self.hyps:
            ys = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
            ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp)
            lo = max(0, n - 1 - delay)
            if self.merge_algo == "lcs":
                upto = [y for y, t in zip(ys, ts) if t < lo + tpc]
                merged = lcs_alignment_merge_buffer(merged, [y for y, t in zip(ys, ts) if t >= max(0, lo - delay)] if merged else upto,
                                                    delay=delay, max_steps_per_timestep=self.max_steps_per_timestep)
            else:
                merged.extend(y for y, t in zip(ys, ts) if lo <= t < lo + tpc)
        return self.asr_model.decoding.decode_tokens_to_str(merged)


BatchedFrameASRTDT = BatchedFrameASRRNNT   # TDT models decode through the same transducer interface (durations handled by the decoder)


class FrameBatchMultiTaskAED:
    """Chunked inference for attention encoder-decoder models on long recordings: the audio is cut into windows of ``chunk_len``
    seconds (the final short remainder is merged into the previous window), each window is transcribed with the model's prompt
    and the texts are joined.  Reference: ``parts/utils/streaming_utils.py`` ``FrameBatchMultiTaskAED`` (window batching +
    prompt per window, text joined with spaces)."""

    def __init__(self, asr_model, chunk_len: float = 30.0, batch_size: int = 4, min_tail: float = 1.0, sample_rate: Optional[int] = None):
        self.asr_model, self.chunk_len, self.batch_size, self.min_tail = asr_model, chunk_len, batch_size, min_tail
        pre = getattr(asr_model, "preprocessor", None)
        feat = getattr(pre, "featurizer", pre)
        self.sr = int(sample_rate or getattr(feat, "sample_rate", 16000))
        self.samples: Optional[torch.Tensor] = None
        self.meta: dict = {}

    def read_audio_file(self, path_or_array, meta_data: Optional[dict] = None, **_):
        if isinstance(path_or_array, str):
            from ..data.audio_to_text import load_audio

            path_or_array = load_audio(path_or_array, target_sr=self.sr)
        self.samples = torch.as_tensor(path_or_array, dtype=torch.float32).reshape(-1)
        self.meta = dict(meta_data or {})

    def windows(self) -> List[torch.Tensor]:
        n = int(self.chunk_len * self.sr)
        chunks = list(self.samples.split(n))
        if len(chunks) > 1 and chunks[-1].numel() < int(self.min_tail * self.sr):
            chunks[-2] = torch.cat([chunks[-2], chunks[-1]])
            chunks.pop()
        return chunks

    @torch.no_grad()
    def transcribe(self, **transcribe_kwargs) -> str:
        texts: List[str] = []
        wins = self.windows()
        for s in range(0, len(wins), self.batch_size):
            batch = [w.numpy() for w in wins[s:s + self.batch_size]]
            hyps = self.asr_model.transcribe(batch, batch_size=len(batch), **{**self.meta, **transcribe_kwargs})
            hyps = hyps[0] if isinstance(hyps, tuple) else hyps
            texts += [h.text if hasattr(h, "text") else str(h) for h in hyps]
        return " ".join(t.strip() for t in texts if t and t.strip())

"""Buffers of the chunked / streaming inference scripts that are not tied to one model family.

* ``StreamingFeatureBufferer`` — samples in, a sliding window of log-mel features out (incremental: only the new chunk's
  frames are computed, with enough left samples for the STFT to be exact).
* ``AudioFeatureIterator`` / ``FeatureFrameBufferer`` / ``BatchedFeatureFrameBufferer`` — frames of features with a history
  buffer, for one or several recordings.
* ``ContextSizeBatch`` / ``StreamingBatchedAudioBuffer`` — a batch of audio streams kept as [left context | chunk | right
  context] in samples, with per-stream lengths: the buffer behind streaming transducer decoding with a limited left context
  and a look-ahead and no padding on the left.
* ``FrameBatchChunkedCTC`` / ``FrameBatchChunkedRNNT`` — non-overlapping chunks transcribed independently and joined.
* ``LongestCommonSubsequenceBatchedFrameASRRNNT`` — buffered transducer inference merged by LCS.
* ``SimpleAudioDataset`` / ``AudioBatch`` — a list of files as padded batches with ids.

Reference: ``asr/parts/utils/streaming_utils.py`` (same class names).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch

from .streaming_utils import BatchedFrameASRRNNT, ContextSize, FrameBatchASR, lcs_alignment_merge_buffer

__all__ = ["AudioBatch", "AudioFeatureIterator", "BatchedFeatureFrameBufferer", "ContextSizeBatch", "FeatureFrameBufferer", "FrameBatchChunkedCTC",
           "FrameBatchChunkedRNNT", "LongestCommonSubsequenceBatchedFrameASRRNNT", "SimpleAudioDataset", "StreamingBatchedAudioBuffer",
           "StreamingFeatureBufferer", "advance_context", "inplace_buffer_merge", "streaming_transcribe_rnnt"]


def inplace_buffer_merge(buffer: List[int], data: List[int], timesteps: int, model=None) -> List[int]:
    """Overwrites the last ``timesteps`` tokens of ``buffer`` with the head of ``data`` and appends the rest (the newer window is
    trusted where two windows overlap)."""
    if len(buffer) < timesteps or timesteps < 1:
        buffer += list(data)
        return buffer
    n = min(timesteps, len(data))
    buffer[len(buffer) - timesteps: len(buffer) - timesteps + n] = data[:n]
    buffer += list(data[timesteps:])
    return buffer


# ------------------------------------------------------------------------------------------------ features from samples
class StreamingFeatureBufferer:
    """``buffer`` holds the features of the last ``buffer_len`` seconds.  ``append(chunk_samples)`` emits every frame whose analysis
    window is complete (frames are centred, so the newest ``n_fft / 2`` samples wait for the next chunk) computed from enough
    history that the emitted frames equal those of the whole signal; ``flush()`` emits the tail at the end of the stream.
    Per-utterance normalisation needs the whole utterance and must be off, or fixed statistics are passed in."""

    def __init__(self, asr_model, chunk_size: float, buffer_size: float, fixed_mean: Optional[torch.Tensor] = None, fixed_std: Optional[torch.Tensor] = None):
        pre = asr_model.preprocessor
        feat = getattr(pre, "featurizer", pre)
        self.pre = pre
        self.sr = int(getattr(feat, "sample_rate", 16000))
        self.hop = int(feat.hop_length)
        self.n_fft = int(getattr(feat, "n_fft", 512))
        self.n_feat = int(asr_model.encoder._feat_in)
        self.chunk_frames = int(round(chunk_size * self.sr / self.hop))
        self.buffer_frames = int(round(buffer_size * self.sr / self.hop))
        self.mean, self.std = fixed_mean, fixed_std
        self.zero_level = float(np.log(2.0 ** -24))
        self.guard = -(-self.n_fft // self.hop) + 1                   # frames of history in front of the first emitted frame
        self.reset()

    def reset(self):
        self.buffer = torch.full((self.n_feat, self.buffer_frames), self.zero_level)
        self.tail = torch.zeros(0)                                     # samples from global index `base` on
        self.base = 0
        self.received = 0
        self.frames_seen = 0                                           # frames emitted so far

    @torch.no_grad()
    def _emit(self, upto_frame: int) -> torch.Tensor:
        if upto_frame < self.frames_seen or self.tail.numel() == 0:
            return torch.zeros(self.n_feat, 0)
        dev = next(self.pre.parameters(), torch.zeros(1)).device
        feats, _ = self.pre(input_signal=self.tail[None].to(dev), length=torch.tensor([self.tail.numel()], device=dev))
        off = self.base // self.hop
        f = feats[0, :, self.frames_seen - off: upto_frame + 1 - off].float().cpu()
        if self.mean is not None:
            f = (f - self.mean[:, None]) / (self.std[:, None] + 1e-5)
        self.frames_seen += f.shape[1]
        new_base = max(0, (self.frames_seen - self.guard) * self.hop)
        self.tail, self.base = self.tail[new_base - self.base:], new_base
        if f.shape[1]:
            self.buffer = torch.cat([self.buffer[:, f.shape[1]:], f], dim=1)[:, -self.buffer_frames:]
        return f

    def append(self, samples) -> torch.Tensor:
        x = torch.as_tensor(samples, dtype=torch.float32).reshape(-1)
        self.tail = torch.cat([self.tail, x])
        self.received += x.numel()
        self._emit((self.received - self.n_fft // 2) // self.hop if self.received >= self.n_fft // 2 else -1)
        return self.buffer

    def flush(self) -> torch.Tensor:
        """End of the stream: the frames that were waiting for samples that will not come."""
        self._emit(self.received // self.hop)
        return self.buffer

    def get_buffer(self) -> torch.Tensor:
        return self.buffer


class AudioFeatureIterator:
    """Features of one recording cut into frames of ``frame_len`` seconds (the last one zero-padded)."""

    def __init__(self, samples, frame_len: float, preprocessor, device="cpu", pad_to_frame_len: bool = True):
        x = torch.as_tensor(samples, dtype=torch.float32).reshape(1, -1).to(device)
        feat = getattr(preprocessor, "featurizer", preprocessor)
        self.frame = int(round(frame_len * feat.sample_rate / feat.hop_length))
        with torch.no_grad():
            f, n = preprocessor(input_signal=x, length=torch.tensor([x.shape[1]], device=device))
        self.features = f[0, :, : int(n[0])].cpu()
        self.pad, self.pos = pad_to_frame_len, 0

    def __iter__(self):
        return self

    def __next__(self) -> torch.Tensor:
        if self.pos >= self.features.shape[1]:
            raise StopIteration
        f = self.features[:, self.pos: self.pos + self.frame]
        self.pos += self.frame
        if f.shape[1] < self.frame and self.pad:
            f = torch.nn.functional.pad(f, (0, self.frame - f.shape[1]))
        return f


class FeatureFrameBufferer:
    """Consumes a frame iterator and yields, per frame, the buffer ``[features, total_buffer frames]`` whose tail is that frame."""

    def __init__(self, asr_model, frame_len: float = 1.6, batch_size: int = 4, total_buffer: float = 4.0, pad_to_buffer_len: bool = True):
        feat = getattr(asr_model.preprocessor, "featurizer", asr_model.preprocessor)
        self.n_feat = int(asr_model.encoder._feat_in)
        self.frame = int(round(frame_len * feat.sample_rate / feat.hop_length))
        self.total = int(round(total_buffer * feat.sample_rate / feat.hop_length))
        self.batch_size, self.zero = batch_size, float(np.log(2.0 ** -24))
        self.reset()

    def reset(self):
        self.buffer = torch.full((self.n_feat, self.total), self.zero)
        self.iterator: Optional[Iterator[torch.Tensor]] = None
        self.done = False

    def set_frame_reader(self, it: Iterator[torch.Tensor]):
        self.iterator, self.done = iter(it), False

    def get_frame_buffers(self, frames: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        out = []
        for f in frames:
            self.buffer = torch.cat([self.buffer[:, f.shape[1]:], f], dim=1)
            out.append(self.buffer.clone())
        return out

    def get_batch_frames(self) -> List[torch.Tensor]:
        frames = []
        while not self.done and len(frames) < self.batch_size:
            try:
                frames.append(next(self.iterator))
            except StopIteration:
                self.done = True
        return frames

    def get_buffers_batch(self) -> List[torch.Tensor]:
        return self.get_frame_buffers(self.get_batch_frames())


class BatchedFeatureFrameBufferer:
    """One ``FeatureFrameBufferer`` per recording advanced in lockstep: ``get_buffers_batch`` returns the current buffer of every
    recording that still has frames, and which recordings those are."""

    def __init__(self, asr_model, frame_len: float = 1.6, batch_size: int = 4, total_buffer: float = 4.0):
        self.make = lambda: FeatureFrameBufferer(asr_model, frame_len, 1, total_buffer)
        self.batch_size = batch_size
        self.buffers: List[FeatureFrameBufferer] = []

    def reset(self):
        self.buffers = []

    def set_frame_reader(self, it: Iterator[torch.Tensor], idx: int):
        while len(self.buffers) <= idx:
            self.buffers.append(self.make())
        self.buffers[idx].set_frame_reader(it)

    def get_buffers_batch(self) -> Tuple[List[torch.Tensor], List[int]]:
        out, ids = [], []
        for i, b in enumerate(self.buffers):
            if b.iterator is None or b.done:
                continue
            got = b.get_buffers_batch()
            if got:
                out.append(got[0])
                ids.append(i)
        return out, ids


# ------------------------------------------------------------------------------------------------ left | chunk | right accounting
def advance_context(cur: ContextSize, num_frames: int, is_last_chunk: bool, expected: ContextSize) -> int:
    """A stream receives ``num_frames`` more frames.  What was the chunk becomes left context; the new frames join the right
    context; then ``expected.chunk`` frames move from the right context into the chunk (all of them on the last chunk).  Returns
    how many of the oldest frames must be dropped for the total to stay within ``expected.total()``."""
    if num_frames > expected.chunk + expected.right:
        raise ValueError(f"{num_frames} new frames exceed the chunk plus right context of {expected}")
    cur.left += cur.chunk
    cur.right += num_frames
    if is_last_chunk:
        cur.chunk, cur.right = cur.right, 0
    elif cur.right > expected.chunk:
        cur.chunk, cur.right = expected.chunk, cur.right - expected.chunk
    else:
        cur.chunk = 0
    drop = max(0, cur.total() - expected.total())
    cur.left -= drop
    return drop


@dataclass
class ContextSizeBatch:
    left: torch.Tensor
    chunk: torch.Tensor
    right: torch.Tensor

    def total(self) -> torch.Tensor:
        return self.left + self.chunk + self.right

    def subsample(self, factor: int) -> "ContextSizeBatch":
        d = lambda t: torch.div(t, factor, rounding_mode="floor")  # noqa: E731
        return ContextSizeBatch(d(self.left), d(self.chunk), d(self.right))

    def add_frames_(self, num_frames: torch.Tensor, is_last: torch.Tensor, expected: ContextSize):
        """Per-stream version of ``advance_context`` (streams of a batch end at different times)."""
        self.left = self.left + self.chunk
        self.right = self.right + num_frames
        self.chunk = torch.where(is_last, self.right, torch.full_like(self.right, expected.chunk))
        self.right = torch.where(is_last, torch.zeros_like(self.right), self.right - expected.chunk)
        self.left = torch.where(self.chunk > 0, self.left, torch.zeros_like(self.left))
        extra = (self.total() - expected.total()).clamp(min=0)
        self.left = (self.left - extra).clamp(min=0)


class StreamingBatchedAudioBuffer:
    """``samples`` [B, <= expected.total()]: the newest audio of every stream.  ``add_audio_batch_`` appends a chunk and forgets
    the samples that fell out of the left context; ``context_size`` describes the (padded) batch, ``context_size_batch`` every
    stream by its true length."""

    def __init__(self, batch_size: int, context_samples: ContextSize, dtype: torch.dtype = torch.float32, device="cpu"):
        self.batch_size, self.expected = batch_size, context_samples
        self.samples = torch.zeros((batch_size, 0), dtype=dtype, device=device)
        self.context_size = ContextSize(0, 0, 0)
        z = lambda: torch.zeros(batch_size, dtype=torch.long, device=device)  # noqa: E731
        self.context_size_batch = ContextSizeBatch(z(), z(), z())

    def add_audio_batch_(self, audio_batch: torch.Tensor, audio_lengths: torch.Tensor, is_last_chunk: bool, is_last_chunk_batch: torch.Tensor):
        self.samples = torch.cat([self.samples, audio_batch.to(self.samples)], dim=1)
        drop = advance_context(self.context_size, audio_batch.shape[1], is_last_chunk, self.expected)
        self.context_size_batch.add_frames_(audio_lengths.to(self.context_size_batch.left), is_last_chunk_batch, self.expected)
        if drop:
            self.samples = self.samples[:, drop:]


# ------------------------------------------------------------------------------------------------ chunked (no overlap) inference
class FrameBatchChunkedCTC(FrameBatchASR):
    """Long recordings cut into independent ``frame_len`` second chunks (no context buffers); token ids are concatenated."""

    def __init__(self, asr_model, frame_len: float = 20.0, batch_size: int = 4, **_):
        super().__init__(asr_model, frame_len, frame_len, batch_size)

    def _windows(self):
        n = int(self.frame_len * self.sr)
        for k in range(0, self.samples.numel(), n):
            w = self.samples[k:k + n]
            yield torch.nn.functional.pad(w, (0, n - w.numel())) if w.numel() < n else w

    def transcribe(self, **_):
        self.infer_logits()
        out, prev = [], self.blank_id
        for p in self.all_preds:
            for t in p.tolist():
                if t != prev and t != self.blank_id:
                    out.append(t)
                prev = t
            prev = self.blank_id
        decoding = self.asr_model.ctc_decoding if hasattr(self.asr_model, "ctc_decoding") else self.asr_model.decoding
        return decoding.decode_tokens_to_str(out)


class FrameBatchChunkedRNNT(BatchedFrameASRRNNT):
    def __init__(self, asr_model, frame_len: float = 20.0, batch_size: int = 4, **_):
        super().__init__(asr_model, frame_len, frame_len, batch_size)

    _windows = FrameBatchChunkedCTC._windows

    def transcribe(self, **_):
        self.infer_logits()
        ids: List[int] = []
        for h, _n in self.hyps:
            ids += h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
        return self.asr_model.decoding.decode_tokens_to_str(ids)


class LongestCommonSubsequenceBatchedFrameASRRNNT(BatchedFrameASRRNNT):
    """Buffered transducer inference whose consecutive windows are joined where their token sequences overlap; ``alignment_basepath``
    (debug dumps of the alignments) is accepted and ignored."""

    def __init__(self, asr_model, frame_len=1.6, total_buffer=4.0, batch_size=4, max_steps_per_timestep: int = 5, stateful_decoding: bool = False,
                 alignment_basepath: Optional[str] = None):
        super().__init__(asr_model, frame_len, total_buffer, batch_size, max_steps_per_timestep, stateful_decoding, merge_algo="lcs")

    def transcribe(self, tokens_per_chunk: Optional[int] = None, delay: Optional[int] = None, **_):
        self.infer_logits()
        delay = delay or self.delay
        tpc = tokens_per_chunk or self.tokens_per_chunk
        merged: List[int] = []
        for k, (h, n) in enumerate(self.hyps):
            ys = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
            ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp)
            lo = max(0, n - 1 - delay)
            # tokens from the start of the previous chunk's position up to the end of this chunk: the first part repeats what the
            # buffer already ends with, which is what the LCS finds
            cur = [y for y, t in zip(ys, ts) if max(0, lo - tpc) <= t < lo + tpc]
            merged = cur if not merged else lcs_alignment_merge_buffer(merged, cur, delay=tpc, max_steps_per_timestep=self.max_steps_per_timestep)
        return self.asr_model.decoding.decode_tokens_to_str(merged)


# ------------------------------------------------------------------------------------------------ file batches
class AudioBatch(NamedTuple):
    audio_signals: torch.Tensor
    audio_signal_lengths: torch.Tensor
    ids: torch.Tensor

    @staticmethod
    def collate_fn(items: Sequence[Tuple[torch.Tensor, int]]) -> "AudioBatch":
        lens = torch.tensor([a.numel() for a, _ in items])
        x = torch.zeros(len(items), int(lens.max()))
        for i, (a, _) in enumerate(items):
            x[i, : a.numel()] = a
        return AudioBatch(x, lens, torch.tensor([i for _, i in items]))


class SimpleAudioDataset(torch.utils.data.Dataset):
    def __init__(self, audio_filenames: Sequence, sample_rate: int = 16000):
        self.files, self.sr = list(audio_filenames), sample_rate

    def __len__(self):
        return len(self.files)

    def __getitem__(self, i):
        from ..data.audio_to_text import load_audio

        f = self.files[i]
        a = load_audio(f, target_sr=self.sr) if isinstance(f, str) else f
        return torch.as_tensor(np.asarray(a), dtype=torch.float32).reshape(-1), i


# ------------------------------------------------------------------------------------------------ streaming transducer inference
@torch.no_grad()
def streaming_transcribe_rnnt(model, audio: torch.Tensor, lengths: torch.Tensor, chunk_secs: float = 2.0, left_context_secs: float = 10.0,
                              right_context_secs: float = 2.0):
    """Transducer decoding of a batch of recordings with a limited left context and a look-ahead, without left padding: every step
    encodes ``[left | chunk | right]`` (whatever of it exists yet), decodes only the encoder frames of the chunk and carries the
    decoder state on.  Latency is chunk + right context.  Returns the final hypotheses.
    Reference script: ``examples/asr/asr_chunked_inference/rnnt/speech_to_text_streaming_infer_rnnt.py``."""
    feat = getattr(model.preprocessor, "featurizer", model.preprocessor)
    sr, hop = int(getattr(feat, "sample_rate", 16000)), int(feat.hop_length)
    sub = int(model.encoder.subsampling_factor)
    unit = hop * sub                                                   # samples per encoder frame
    frames = lambda secs: max(0, int(round(secs * sr / unit)))  # noqa: E731
    exp = ContextSize(frames(left_context_secs) * unit, max(1, frames(chunk_secs)) * unit, frames(right_context_secs) * unit)
    dev = next(model.parameters()).device
    B, T = audio.shape
    buf = StreamingBatchedAudioBuffer(B, exp, torch.float32, dev)
    hyps = None
    pos, first = 0, True
    lengths = lengths.to(dev)
    while pos < T:
        n = min((exp.chunk + exp.right) if first else exp.chunk, T - pos)
        last = pos + n >= T
        buf.add_audio_batch_(audio[:, pos:pos + n].to(dev), (lengths - pos).clamp(min=0, max=n), last, lengths <= pos + n)
        pos, first = pos + n, False
        c, cb = buf.context_size, buf.context_size_batch
        if c.chunk == 0:
            continue
        enc, enc_len = model.forward(input_signal=buf.samples, input_signal_length=cb.total().clamp(min=1))
        ef = cb.subsample(unit)
        lo = c.left // unit
        n_chunk = enc.shape[2] - lo if last else c.chunk // unit
        chunk_enc = enc[:, :, lo: lo + n_chunk]
        # per stream: frames of the chunk that are real audio
        chunk_len = (enc_len - ef.left).clamp(min=0, max=n_chunk) if last else torch.minimum(ef.chunk, (enc_len - ef.left).clamp(min=0))
        active = chunk_len > 0
        if not bool(active.any()):
            continue
        got = model.decoding.rnnt_decoder_predictions_tensor(encoder_output=chunk_enc.float(), encoded_lengths=chunk_len.clamp(min=1),
                                                             return_hypotheses=True, partial_hypotheses=hyps)
        if hyps is None:
            hyps = got
        else:
            hyps = [g if bool(a) else h for g, h, a in zip(got, hyps, active.tolist())]
    return hyps

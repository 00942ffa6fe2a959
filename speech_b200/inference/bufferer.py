"""Audio and feature buffering for streaming recognition.

* ``AudioBufferer`` — per-stream ring buffer of the last ``buffer_size_in_secs`` of samples (buffered pipelines decode the
  whole window every step and keep only the middle tokens).
* ``BatchedCacheFeatureBufferer`` — audio ring buffers for a batch of streams; every update recomputes log-mel features of
  the windows in ONE preprocessor call and returns, per stream, the feature frames of the newest chunk preceded by the
  pre-encode cache frames the subsampling convolutions need.

Feature frames are bit-compatible with an offline pass over the whole recording: a frame is only released once its whole
analysis window lies inside the buffer, which costs ``lookahead_frames`` (= ceil(n_fft / 2 / hop), 2 frames = 20 ms for the
default front-end) of extra audio in the first chunk of a stream; afterwards every chunk releases exactly ``chunk_frames``
frames.  The stream's last chunk releases whatever is left up to the offline frame count.
Reference: ``inference/streaming/buffering/{audio_bufferer,cache_feature_bufferer}.py`` and the legacy
``CacheAwareStreamingAudioBuffer`` (``parts/utils/streaming_utils.py``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .framing import FeatureBuffer, Frame


class AudioBufferer:
    """Rows of one ``[capacity, buffer_size]`` tensor hold the streams' windows, so that shifting the new samples of a whole
    batch of streams in is a handful of batched tensor operations (a per-stream ``cat`` costs more host time than the math)."""

    def __init__(self, sample_rate: int, buffer_size_in_secs: float):
        self.sample_rate = sample_rate
        self.buffer_size = int(round(buffer_size_in_secs * sample_rate))
        self.store = torch.zeros((0, self.buffer_size), dtype=torch.float32)
        self.row: Dict[int, int] = {}
        self.free: List[int] = []
        self.filled: Dict[int, int] = {}

    @property
    def buffers(self) -> Dict[int, torch.Tensor]:
        return {sid: self.store[r] for sid, r in self.row.items()}

    def reset(self):
        self.store = torch.zeros((0, self.buffer_size), dtype=torch.float32)
        self.row.clear()
        self.free.clear()
        self.filled.clear()

    def rm_stream(self, stream_id: int):
        r = self.row.pop(stream_id, None)
        if r is not None:
            self.free.append(r)
        self.filled.pop(stream_id, None)

    def _row_for(self, f: Frame) -> int:
        r = self.row.get(f.stream_id)
        if r is None:
            if not self.free:
                grow = max(16, self.store.shape[0])
                self.free = list(range(self.store.shape[0], self.store.shape[0] + grow))
                self.store = torch.cat([self.store, torch.zeros((grow, self.buffer_size), dtype=torch.float32)])
            r = self.free.pop()
            self.row[f.stream_id] = r
            self.store[r].zero_()
            self.filled[f.stream_id] = 0
        elif f.is_first:
            self.store[r].zero_()
            self.filled[f.stream_id] = 0
        return r

    def update(self, frames: List[Frame]):
        """Shift every frame into its stream's window.  Returns ``(windows [B, buffer_size], left_padding [B])`` where
        left padding counts the samples of the window that precede the start of the stream."""
        rows = [self._row_for(f) for f in frames]
        groups: Dict[int, List[int]] = {}
        for k, f in enumerate(frames):
            groups.setdefault(min(f.size, self.buffer_size), []).append(k)
        for n, ks in groups.items():
            idx = torch.tensor([rows[k] for k in ks], dtype=torch.long)
            new = torch.stack([frames[k].samples[-n:].to(torch.float32) for k in ks]) if n > 0 else None
            cur = self.store.index_select(0, idx)
            if n > 0:
                cur = torch.cat([cur[:, n:], new.cpu()], dim=1)
            self.store.index_copy_(0, idx, cur)
        pads = []
        for f in frames:
            n = min(f.size, self.buffer_size)
            self.filled[f.stream_id] = min(self.buffer_size, self.filled[f.stream_id] + n)
            pads.append(self.buffer_size - self.filled[f.stream_id])
        out = self.store.index_select(0, torch.tensor(rows, dtype=torch.long))
        for f in frames:
            if f.is_last:
                self.rm_stream(f.stream_id)
        return out, torch.tensor(pads, dtype=torch.long)


class BatchedCacheFeatureBufferer:
    def __init__(self, sample_rate: int, buffer_size_in_secs: float, chunk_size_in_secs: float, preprocessor, device=None,
                 pre_encode_cache_frames: int = 0, first_chunk_frames: Optional[int] = None, right_pad_features: bool = False):
        self.preprocessor = preprocessor
        self.device = device
        feat = getattr(preprocessor, "featurizer", preprocessor)
        self.featurizer = feat
        self.hop = int(getattr(feat, "hop_length", int(0.01 * sample_rate)))
        n_fft = int(getattr(feat, "n_fft", 512))
        self.lookahead_frames = int(math.ceil((n_fft // 2) / self.hop))
        self.chunk_samples = int(round(chunk_size_in_secs * sample_rate))
        self.chunk_frames = int(math.ceil(self.chunk_samples / self.hop))
        self.first_chunk_frames = int(first_chunk_frames) if first_chunk_frames else self.chunk_frames
        self.cache_frames = int(pre_encode_cache_frames)
        need = (max(self.chunk_frames, self.first_chunk_frames) + self.cache_frames + self.lookahead_frames + 1) * self.hop
        self.audio = AudioBufferer(sample_rate, max(buffer_size_in_secs, need / sample_rate))
        self.right_pad_features = right_pad_features
        self.delivered: Dict[int, int] = {}

    # geometry the streamer needs to cut the audio so that every update releases whole chunks
    def first_frame_samples(self) -> int:
        return (self.first_chunk_frames + self.lookahead_frames) * self.hop

    def tail_padding_samples(self) -> int:
        return (self.lookahead_frames + 1) * self.hop

    def set_pre_encode_cache(self, frames: int) -> None:
        self.cache_frames = int(frames)
        need = (max(self.chunk_frames, self.first_chunk_frames) + self.cache_frames + self.lookahead_frames + 1) * self.hop
        if need > self.audio.buffer_size:
            self.audio = AudioBufferer(self.audio.sample_rate, need / self.audio.sample_rate)

    def _offline_frames(self, n_samples: int) -> int:
        if hasattr(self.featurizer, "get_seq_len"):
            return int(self.featurizer.get_seq_len(torch.tensor([n_samples]))[0])
        return n_samples // self.hop + 1

    @torch.no_grad()
    def update(self, frames: List[Frame]) -> List[FeatureBuffer]:
        windows, _ = self.audio.update(frames)
        dev = self.device or windows.device
        windows = windows.to(dev)
        lens = torch.full((windows.shape[0],), windows.shape[1], dtype=torch.long, device=dev)
        was_training = getattr(self.preprocessor, "training", False)
        if was_training:
            self.preprocessor.eval()
        feats, _ = self.preprocessor(input_signal=windows, length=lens)  # [B, F, T]
        if was_training:
            self.preprocessor.train()
        # window frame j is centred on window sample j*hop; frames up to `end` have their analysis window inside the buffer
        end = windows.shape[1] // self.hop - self.lookahead_frames
        out = []
        for i, f in enumerate(frames):
            if f.is_first:
                self.delivered[f.stream_id] = 0
            new = self.first_chunk_frames if f.is_first else self.chunk_frames
            cache = 0 if f.is_first else self.cache_frames
            if f.is_last:
                # the tail is zero-padded audio, exactly what the offline front-end sees beyond the end of the recording
                end_i = windows.shape[1] // self.hop + 1
                total = self._offline_frames(f.total_samples if f.total_samples >= 0 else 0)
                remaining = max(0, total - self.delivered.get(f.stream_id, 0))
                # frames of this (padded) chunk start where the previous release stopped
                lo = end - new
                x = feats[i, :, max(0, lo - cache):min(end_i, lo + max(new, remaining))]
                valid_new = min(remaining, x.shape[1] - cache)
            else:
                lo = end - new
                x = feats[i, :, max(0, lo - cache):end]
                valid_new = new
            if x.shape[1] < cache + new:
                x = torch.nn.functional.pad(x, (0, cache + new - x.shape[1]))
            self.delivered[f.stream_id] = self.delivered.get(f.stream_id, 0) + valid_new
            if f.is_last:
                self.delivered.pop(f.stream_id, None)
            out.append(FeatureBuffer(features=x, stream_id=f.stream_id, is_first=f.is_first, is_last=f.is_last,
                                     length=cache + valid_new, options=f.options))
        return out

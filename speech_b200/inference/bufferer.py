"""Audio and feature buffering for streaming recognition.

* ``AudioBufferer`` — per-stream ring buffer of the last ``buffer_size_in_secs`` of samples (buffered pipelines decode the
  whole window every step and keep only the middle tokens).
* ``BatchedCacheFeatureBufferer`` — audio ring buffers for a batch of streams; every update recomputes log-mel features of
  the windows in ONE preprocessor call and returns, per stream, the feature frames of the newest chunk preceded by the
  pre-encode cache frames the subsampling convolutions need.
Reference: ``inference/streaming/buffering/{audio_bufferer,cache_feature_bufferer}.py`` and the legacy
``CacheAwareStreamingAudioBuffer`` (``parts/utils/streaming_utils.py``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .framing import FeatureBuffer, Frame


class AudioBufferer:
    def __init__(self, sample_rate: int, buffer_size_in_secs: float):
        self.sample_rate = sample_rate
        self.buffer_size = int(round(buffer_size_in_secs * sample_rate))
        self.buffers: Dict[int, torch.Tensor] = {}
        self.filled: Dict[int, int] = {}

    def reset(self):
        self.buffers.clear()
        self.filled.clear()

    def rm_stream(self, stream_id: int):
        self.buffers.pop(stream_id, None)
        self.filled.pop(stream_id, None)

    def update(self, frames: List[Frame]):
        """Shift every frame into its stream's window.  Returns ``(windows [B, buffer_size], left_padding [B])`` where
        left padding counts the samples of the window that precede the start of the stream."""
        outs, pads = [], []
        for f in frames:
            buf = self.buffers.get(f.stream_id)
            if buf is None or f.is_first:
                buf = torch.zeros(self.buffer_size, dtype=torch.float32)
                self.filled[f.stream_id] = 0
            n = min(f.size, self.buffer_size)
            buf = torch.cat([buf[n:], f.samples[-n:].to(buf.dtype).cpu()])
            self.buffers[f.stream_id] = buf
            self.filled[f.stream_id] = min(self.buffer_size, self.filled[f.stream_id] + n)
            outs.append(buf)
            pads.append(self.buffer_size - self.filled[f.stream_id])
            if f.is_last:
                self.rm_stream(f.stream_id)
        return torch.stack(outs), torch.tensor(pads, dtype=torch.long)


class BatchedCacheFeatureBufferer:
    def __init__(self, sample_rate: int, buffer_size_in_secs: float, chunk_size_in_secs: float, preprocessor, device=None,
                 pre_encode_cache_frames: int = 0, right_pad_features: bool = False):
        self.audio = AudioBufferer(sample_rate, buffer_size_in_secs)
        self.preprocessor = preprocessor
        self.device = device
        feat = getattr(preprocessor, "featurizer", preprocessor)
        self.hop = int(getattr(feat, "hop_length", int(0.01 * sample_rate)))
        self.chunk_samples = int(round(chunk_size_in_secs * sample_rate))
        self.chunk_frames = int(math.ceil(self.chunk_samples / self.hop))
        self.cache_frames = int(pre_encode_cache_frames)
        self.right_pad_features = right_pad_features
        if self.chunk_samples + self.cache_frames * self.hop > self.audio.buffer_size:
            raise ValueError("the audio buffer must cover one chunk plus the pre-encode cache")

    def set_pre_encode_cache(self, frames: int) -> None:
        self.cache_frames = int(frames)

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
        T = (windows.shape[1] // self.hop)  # frames fully inside the window (the trailing centre-padded frame is dropped)
        want = self.chunk_frames + self.cache_frames
        out = []
        for i, f in enumerate(frames):
            x = feats[i, :, max(0, T - want):T]
            if x.shape[1] < want:
                x = torch.nn.functional.pad(x, (want - x.shape[1], 0))
            valid_chunk = int(math.ceil(f.valid_size / self.hop))
            length = self.cache_frames + valid_chunk
            if f.is_first and self.cache_frames:
                # nothing precedes the first chunk: drop the cache part so the encoder sees exactly the chunk
                x = x[:, self.cache_frames:]
                length = valid_chunk
            out.append(FeatureBuffer(features=x, stream_id=f.stream_id, is_first=f.is_first, is_last=f.is_last, length=length,
                                     options=f.options))
        return out

"""Requests of the streaming pipelines and the continuous-batching streamer that produces them.

A *stream* is one audio source cut into fixed-size chunks.  The streamer keeps up to ``batch_size`` streams alive, yields
one chunk per live stream at every step and admits the next waiting stream as soon as one ends, so the accelerator batch
stays full for the whole run (reference: ``inference/streaming/framing/{request,request_options,multi_stream}.py``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence, Union

import numpy as np
import torch


class RequestType(enum.Enum):
    FRAME = "frame"                    # raw audio samples
    FEATURE_BUFFER = "feature_buffer"  # pre-computed log-mel features


@dataclass
class ASRRequestOptions:
    enable_itn: bool = False
    enable_pnc: bool = True
    enable_nmt: bool = False
    stop_history_eou: Optional[int] = None   # ms of trailing silence that ends an utterance (-1: use pipeline default)
    asr_output_granularity: str = "word"     # "word" | "segment"
    language_code: Optional[str] = None
    biasing_cfg: Optional[Dict[str, Any]] = None
    source_language: Optional[str] = None
    target_language: Optional[str] = None

    def augment_with_defaults(self, **defaults) -> "ASRRequestOptions":
        out = ASRRequestOptions(**self.__dict__)
        for k, v in defaults.items():
            if getattr(out, k, None) is None:
                setattr(out, k, v)
        return out


@dataclass
class Frame:
    samples: torch.Tensor            # [n] float32
    stream_id: int
    is_first: bool = False
    is_last: bool = False
    length: int = -1                 # valid samples (<= len(samples)); -1 = all
    options: Optional[ASRRequestOptions] = None
    total_samples: int = -1          # on the last frame: length of the whole stream without tail padding

    @property
    def size(self) -> int:
        return int(self.samples.shape[0])

    @property
    def valid_size(self) -> int:
        return self.size if self.length < 0 else int(self.length)


@dataclass
class FeatureBuffer:
    features: torch.Tensor           # [F, T]
    stream_id: int
    is_first: bool = False
    is_last: bool = False
    length: int = -1
    right_pad_features: Optional[torch.Tensor] = None
    options: Optional[ASRRequestOptions] = None

    @property
    def size(self) -> int:
        return int(self.features.shape[1])

    @property
    def valid_size(self) -> int:
        return self.size if self.length < 0 else int(self.length)


Request = Union[Frame, FeatureBuffer]


class MonoStream:
    """One audio source cut into chunks of ``frame_size`` samples; the last chunk is zero-padded when ``pad_last_frame``."""

    def __init__(self, samples: torch.Tensor, stream_id: int, frame_size: int, pad_last_frame: bool = True,
                 options: Optional[ASRRequestOptions] = None, first_frame_size: Optional[int] = None, tail_padding: int = 0):
        self.samples = samples.reshape(-1).float()
        self.true_length = int(self.samples.shape[0])
        if tail_padding:
            self.samples = torch.nn.functional.pad(self.samples, (0, int(tail_padding)))
        self.stream_id, self.frame_size, self.pad_last = stream_id, int(frame_size), pad_last_frame
        self.first_frame_size = int(first_frame_size) if first_frame_size else self.frame_size
        self.options = options
        self.pos = 0
        self.n = int(self.samples.shape[0])

    def done(self) -> bool:
        return self.pos >= self.n and self.pos > 0

    def next_frame(self) -> Frame:
        size = self.first_frame_size if self.pos == 0 else self.frame_size
        s, e = self.pos, min(self.n, self.pos + size)
        chunk = self.samples[s:e]
        valid = e - s
        if valid < size and self.pad_last:
            chunk = torch.nn.functional.pad(chunk, (0, size - valid))
        self.pos = s + size
        last = self.pos >= self.n
        return Frame(samples=chunk, stream_id=self.stream_id, is_first=(s == 0), is_last=last, length=valid,
                     options=self.options, total_samples=self.true_length if last else -1)


class ContinuousBatchedRequestStreamer:
    """Iterates ``List[Request]`` batches over many audio sources with continuous batching.

    ``request_type=FEATURE_BUFFER`` converts every frame to log-mel features with a per-stream feature bufferer
    (see ``bufferer.BatchedCacheFeatureBufferer``) before yielding.
    """

    def __init__(self, n_frames_per_stream: int, batch_size: int, sample_rate: int = 16000,
                 request_type: RequestType = RequestType.FRAME, preprocessor=None, buffer_size_in_secs: Optional[float] = None,
                 device=None, pad_last_frame: bool = True, right_pad_features: bool = False, tail_padding_in_samples: int = 0,
                 first_frame_size: Optional[int] = None, bufferer=None):
        self.frame_size, self.batch_size, self.sample_rate = int(n_frames_per_stream), int(batch_size), sample_rate
        self.first_frame_size = first_frame_size
        self.request_type, self.device = request_type, device
        self.pad_last_frame = pad_last_frame
        self.tail_padding = int(tail_padding_in_samples)
        self.sources: List[Any] = []
        self.options: List[Optional[ASRRequestOptions]] = []
        self.elapsed_durations: Dict[int, float] = {}
        self.bufferer = bufferer
        if request_type is RequestType.FEATURE_BUFFER and bufferer is None:
            from .bufferer import BatchedCacheFeatureBufferer

            if preprocessor is None or buffer_size_in_secs is None:
                raise ValueError("feature-buffer requests need a preprocessor and buffer_size_in_secs")
            self.bufferer = BatchedCacheFeatureBufferer(sample_rate=sample_rate, buffer_size_in_secs=buffer_size_in_secs,
                                                        chunk_size_in_secs=self.frame_size / sample_rate,
                                                        preprocessor=preprocessor, device=device,
                                                        right_pad_features=right_pad_features)
        if self.bufferer is not None:
            # cut the audio so that every update releases whole chunks of offline-exact feature frames
            self.first_frame_size = self.first_frame_size or self.bufferer.first_frame_samples()
            self.tail_padding = self.tail_padding or self.bufferer.tail_padding_samples()

    def set_audio_filepaths(self, audio: Sequence[Union[str, np.ndarray, torch.Tensor]],
                            options: Optional[Sequence[Optional[ASRRequestOptions]]] = None) -> None:
        self.sources = list(audio)
        self.options = list(options) if options is not None else [None] * len(self.sources)
        self.elapsed_durations = {}

    def _open(self, stream_id: int) -> MonoStream:
        src = self.sources[stream_id]
        if isinstance(src, str):
            from ..data.audio_to_text import load_audio

            x = torch.from_numpy(np.asarray(load_audio(src, target_sr=self.sample_rate), dtype=np.float32))
        else:
            x = torch.as_tensor(src, dtype=torch.float32)
        self.elapsed_durations[stream_id] = x.numel() / self.sample_rate
        return MonoStream(x, stream_id, self.frame_size, self.pad_last_frame, self.options[stream_id],
                          first_frame_size=self.first_frame_size, tail_padding=self.tail_padding)

    def get_audio_durations(self) -> Dict[int, float]:
        return dict(self.elapsed_durations)

    def __iter__(self) -> Iterator[List[Request]]:
        next_id = 0
        live: List[MonoStream] = []
        total = len(self.sources)
        while next_id < total or live:
            while len(live) < self.batch_size and next_id < total:
                live.append(self._open(next_id))
                next_id += 1
            frames = [s.next_frame() for s in live]
            live = [s for s, f in zip(live, frames) if not f.is_last]
            if self.bufferer is not None:
                yield self.bufferer.update(frames)
            else:
                yield frames

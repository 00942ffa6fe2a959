"""Per-stream recognition state, greedy end-of-utterance endpointing and token → word assembly for the streaming
pipelines (reference: ``inference/streaming/state/state.py``, ``streaming/endpointing/greedy/*``,
``streaming/text/text_processing.py``, ``utils/bpe_decoder.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Sequence

from .framing import ASRRequestOptions


@dataclass
class Word:
    text: str
    start: float
    end: float
    conf: float = 1.0

    def to_dict(self):
        return {"word": self.text, "start": round(self.start, 3), "end": round(self.end, 3), "conf": round(self.conf, 4)}


@dataclass
class TextSegment:
    text: str
    start: float
    end: float
    words: List[Word] = field(default_factory=list)
    conf: float = 1.0


class StreamingState:
    """Everything a pipeline remembers about one stream between steps."""

    def __init__(self, stream_id: int = -1, options: Optional[ASRRequestOptions] = None):
        self.stream_id = stream_id
        self.options = options or ASRRequestOptions()
        self.reset()

    def reset(self) -> None:
        self.tokens: List[int] = []          # tokens of the utterance in progress
        self.timesteps: List[int] = []       # encoder-frame index (global) of every token
        self.confidences: List[float] = []
        self.frame_offset = 0                # encoder frames consumed so far
        self.last_emit_frame = -1            # frame of the most recent non-blank
        self.last_ctc_token: Optional[int] = None
        self.hypothesis = None               # transducer partial hypothesis (decoder state inside)
        self.final_segments: List[TextSegment] = []
        self.final_transcript = ""
        self.partial_transcript = ""
        self.current_step_transcript = ""
        self.eou_detected = False
        self.is_finished = False
        self.extra: dict = {}

    # ------------------------------------------------------------------ updates
    def append_tokens(self, tokens: Sequence[int], timesteps: Sequence[int], confidences: Optional[Sequence[float]] = None):
        tokens, timesteps = list(tokens), list(timesteps)
        self.tokens.extend(int(t) for t in tokens)
        self.timesteps.extend(int(t) for t in timesteps)
        self.confidences.extend(list(confidences) if confidences is not None else [1.0] * len(tokens))
        if timesteps:
            self.last_emit_frame = max(self.last_emit_frame, int(timesteps[-1]))

    def advance(self, n_frames: int) -> None:
        self.frame_offset += int(n_frames)

    def trailing_silence_frames(self) -> int:
        if self.last_emit_frame < 0:
            return self.frame_offset if self.tokens else 0
        return self.frame_offset - 1 - self.last_emit_frame

    def cleanup_after_eou(self) -> None:
        self.tokens, self.timesteps, self.confidences = [], [], []
        self.last_emit_frame = -1
        self.partial_transcript = ""
        self.eou_detected = False

    def get_transcript(self) -> str:
        return (self.final_transcript + " " + self.partial_transcript).strip()


class GreedyEndpointing:
    """An utterance ends when ``stop_history_eou`` ms of encoder frames passed without a new non-blank token (and at least
    one token exists), or when the stream ends."""

    def __init__(self, ms_per_frame: float, stop_history_eou_ms: int = 800, residue_tokens_at_end: int = 0):
        self.ms_per_frame = float(ms_per_frame)
        self.default_ms = int(stop_history_eou_ms)
        self.residue = residue_tokens_at_end

    def frames_for(self, state: StreamingState) -> int:
        ms = state.options.stop_history_eou
        ms = self.default_ms if ms is None or ms < 0 else ms
        return max(1, int(round(ms / self.ms_per_frame)))

    def detect_eou(self, state: StreamingState, is_last: bool = False) -> bool:
        if is_last:
            return True
        if not state.tokens:
            return False
        return state.trailing_silence_frames() >= self.frames_for(state)


class TokenTextAssembler:
    """Tokens (+ frame indices, confidences) → words with times.  Works for SentencePiece-style tokenizers (word-initial
    pieces start with ``▁``), WordPiece (continuations start with ``##``) and character vocabularies."""

    def __init__(self, ids_to_tokens: Callable[[List[int]], List[str]], ids_to_text: Callable[[List[int]], str],
                 seconds_per_frame: float, confidence_aggregation: str = "mean", word_separator: str = " "):
        self.ids_to_tokens, self.ids_to_text = ids_to_tokens, ids_to_text
        self.spf = float(seconds_per_frame)
        self.agg = {"mean": lambda c: sum(c) / max(1, len(c)), "min": min, "max": max,
                    "prod": lambda c: _prod(c)}[confidence_aggregation]
        self.sep = word_separator

    def words(self, tokens: List[int], timesteps: List[int], confidences: Optional[List[float]] = None) -> List[Word]:
        if not tokens:
            return []
        confidences = confidences if confidences else [1.0] * len(tokens)
        pieces = self.ids_to_tokens(list(tokens))
        groups: List[List[int]] = []
        is_char_vocab = all(len(p) <= 1 for p in pieces)
        for i, p in enumerate(pieces):
            if is_char_vocab:
                if p == self.sep or p == "":
                    groups.append([])
                    continue
                if not groups:
                    groups.append([])
                groups[-1].append(i)
                continue
            starts_word = p.startswith("▁") or (not p.startswith("##") and "▁" not in "".join(pieces) and
                                                      any(q.startswith("##") for q in pieces))
            if starts_word or not groups:
                groups.append([i])
            else:
                groups[-1].append(i)
        out = []
        for g in groups:
            if not g:
                continue
            text = self.ids_to_text([tokens[i] for i in g]).strip()
            if not text:
                continue
            out.append(Word(text=text, start=timesteps[g[0]] * self.spf, end=(timesteps[g[-1]] + 1) * self.spf,
                            conf=float(self.agg([confidences[i] for i in g]))))
        return out

    def segment(self, tokens, timesteps, confidences=None) -> Optional[TextSegment]:
        ws = self.words(tokens, timesteps, confidences)
        if not ws:
            return None
        return TextSegment(text=self.sep.join(w.text for w in ws), start=ws[0].start, end=ws[-1].end, words=ws,
                           conf=float(self.agg([w.conf for w in ws])))


def _prod(xs):
    p = 1.0
    for x in xs:
        p *= x
    return p

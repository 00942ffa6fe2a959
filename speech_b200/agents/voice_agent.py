"""Voice agent: a frame pipeline that chains streaming speech recognition, diarization, turn taking, a language model and speech
synthesis — microphone frames in, transcripts / replies / synthesised audio out.

The reference implements these as services for the ``pipecat`` framework (``agents/voice_agent/pipecat/services/nemo/stt.py``,
``streaming_asr.py``, ``diar.py`` / ``streaming_diar.py``, ``llm.py``, ``tts.py``, ``turn_taking.py``, ``audio_logger.py``, with a
websocket transport and tool-calling mixins).  ``pipecat`` is an optional package; the same roles are provided here on a small
self-contained frame bus: every processor receives frames, may emit new ones, and passes on what it does not consume.
Models are injected (any object with the documented call signature), so the services work with this framework's streaming
pipelines, Sortformer, ``CausalLM`` and MagpieTTS, or with stand-ins in tests.
"""
from __future__ import annotations

import json
import os
import re
import time
import wave
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import numpy as np


# ---------------------------------------------------------------------------------------------- frames
@dataclass
class Frame:
    timestamp: float = 0.0


@dataclass
class AudioRawFrame(Frame):
    audio: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    sample_rate: int = 16000


@dataclass
class TTSAudioFrame(AudioRawFrame):
    text: str = ""


@dataclass
class TranscriptionFrame(Frame):
    text: str = ""
    is_final: bool = False
    speaker: Optional[str] = None


@dataclass
class DiarResultFrame(Frame):
    speaker_probs: Optional[np.ndarray] = None     # [frames, speakers]
    dominant: Optional[int] = None


@dataclass
class UserStartedSpeakingFrame(Frame):
    pass


@dataclass
class UserStoppedSpeakingFrame(Frame):
    pass


@dataclass
class BotInterruptionFrame(Frame):
    pass


@dataclass
class LLMTextFrame(Frame):
    text: str = ""


@dataclass
class ToolCallFrame(Frame):
    name: str = ""
    arguments: Dict[str, Any] = field(default_factory=dict)
    result: Any = None


@dataclass
class EndFrame(Frame):
    pass


# ---------------------------------------------------------------------------------------------- bus
class FrameProcessor:
    def process(self, frame: Frame) -> Iterable[Frame]:
        """Return the frames that continue down the pipeline (the input frame itself when it is not consumed)."""
        return [frame]


class Pipeline:
    def __init__(self, processors: Sequence[FrameProcessor]):
        self.processors = list(processors)

    def push(self, frame: Frame) -> List[Frame]:
        frames = [frame]
        for p in self.processors:
            nxt: List[Frame] = []
            for f in frames:
                nxt.extend(p.process(f))
            frames = nxt
        return frames

    def run(self, frames: Iterable[Frame]) -> List[Frame]:
        out: List[Frame] = []
        for f in frames:
            out.extend(self.push(f))
        return out


# ---------------------------------------------------------------------------------------------- services
class StreamingSTTService(FrameProcessor):
    """``stream_step(audio_chunk) -> (partial_text, is_final)`` is called on every audio frame; partial transcripts are emitted as
    interim frames, finals when the recogniser (or the turn-taking service downstream) ends the utterance."""

    def __init__(self, stream_step: Callable[[np.ndarray], Any], reset: Optional[Callable[[], None]] = None, emit_interim: bool = True):
        self.stream_step, self.reset, self.emit_interim = stream_step, reset, emit_interim
        self.last_text = ""

    def process(self, frame):
        if isinstance(frame, AudioRawFrame) and not isinstance(frame, TTSAudioFrame):
            res = self.stream_step(frame.audio)
            text, final = (res if isinstance(res, tuple) else (res, False))
            out: List[Frame] = [frame]
            if text is not None and (final or (self.emit_interim and text != self.last_text)):
                out.append(TranscriptionFrame(frame.timestamp, text, bool(final)))
                self.last_text = "" if final else text
                if final and self.reset is not None:
                    self.reset()
            return out
        if isinstance(frame, UserStoppedSpeakingFrame) and self.last_text:
            text, self.last_text = self.last_text, ""
            if self.reset is not None:
                self.reset()
            return [frame, TranscriptionFrame(frame.timestamp, text, True)]
        return [frame]


class StreamingDiarService(FrameProcessor):
    """``diar_step(audio_chunk) -> [frames, speakers]`` activity probabilities; tags later transcripts with the dominant speaker."""

    def __init__(self, diar_step: Callable[[np.ndarray], np.ndarray], threshold: float = 0.5, speaker_names: Optional[List[str]] = None):
        self.diar_step, self.threshold, self.names = diar_step, threshold, speaker_names
        self.activity: Optional[np.ndarray] = None

    def process(self, frame):
        if isinstance(frame, AudioRawFrame) and not isinstance(frame, TTSAudioFrame):
            probs = np.asarray(self.diar_step(frame.audio))
            act = probs.mean(0) if probs.ndim == 2 and probs.shape[0] else np.zeros(0)
            self.activity = act if self.activity is None or self.activity.shape != act.shape else 0.7 * self.activity + 0.3 * act
            dom = int(np.argmax(self.activity)) if self.activity.size and float(self.activity.max()) >= self.threshold else None
            return [frame, DiarResultFrame(frame.timestamp, probs, dom)]
        if isinstance(frame, TranscriptionFrame) and frame.speaker is None and self.activity is not None and self.activity.size:
            if float(self.activity.max()) >= self.threshold:
                k = int(np.argmax(self.activity))
                frame.speaker = self.names[k] if self.names else f"speaker_{k}"
        return [frame]


class TurnTakingService(FrameProcessor):
    """Energy / silence based end-of-turn detection with barge-in: the user is speaking while the frame RMS exceeds
    ``speech_threshold``; ``max_silence`` seconds of quiet end the turn; speech that starts while the bot talks interrupts it.
    Back-channel phrases ("uh-huh", "okay") do not interrupt."""

    BACKCHANNELS = {"uh-huh", "uh huh", "mm-hmm", "mhm", "okay", "ok", "yeah", "right", "i see"}

    def __init__(self, speech_threshold: float = 0.01, max_silence: float = 0.6, min_speech: float = 0.1):
        self.thr, self.max_silence, self.min_speech = speech_threshold, max_silence, min_speech
        self.speaking, self.bot_speaking = False, False
        self.silence = self.speech = 0.0
        self.last_partial = ""

    def process(self, frame):
        if isinstance(frame, TTSAudioFrame):
            self.bot_speaking = True
            return [frame]
        if isinstance(frame, TranscriptionFrame) and not frame.is_final:
            self.last_partial = frame.text
            return [frame]
        if not isinstance(frame, AudioRawFrame):
            return [frame]
        dur = len(frame.audio) / float(frame.sample_rate)
        rms = float(np.sqrt(np.mean(np.square(frame.audio)))) if len(frame.audio) else 0.0
        out: List[Frame] = [frame]
        if rms >= self.thr:
            self.speech += dur
            self.silence = 0.0
            if not self.speaking and self.speech >= self.min_speech:
                self.speaking = True
                out.append(UserStartedSpeakingFrame(frame.timestamp))
                if self.bot_speaking and self.last_partial.strip().lower() not in self.BACKCHANNELS:
                    out.append(BotInterruptionFrame(frame.timestamp))
                    self.bot_speaking = False
        else:
            self.silence += dur
            if self.speaking and self.silence >= self.max_silence:
                self.speaking, self.speech, self.last_partial = False, 0.0, ""
                out.append(UserStoppedSpeakingFrame(frame.timestamp))
            elif not self.speaking:
                self.speech = 0.0
        return out


class LLMService(FrameProcessor):
    """Keeps the conversation, calls ``generate(messages) -> str`` on every final user transcript and emits the reply.  Replies of
    the form ``{"tool": name, "arguments": {...}}`` are dispatched to registered tools and the result is fed back once."""

    def __init__(self, generate: Callable[[List[Dict[str, str]]], str], system_prompt: Optional[str] = None, tools: Optional[Dict[str, Callable[..., Any]]] = None,
                 max_history: int = 32):
        self.generate, self.tools, self.max_history = generate, dict(tools or {}), max_history
        self.messages: List[Dict[str, str]] = [{"role": "system", "content": system_prompt}] if system_prompt else []

    def register_tool(self, name: str, fn: Callable[..., Any]) -> None:
        self.tools[name] = fn

    def _trim(self):
        head = self.messages[:1] if self.messages and self.messages[0]["role"] == "system" else []
        tail = self.messages[len(head):][-self.max_history:]
        self.messages = head + tail

    def process(self, frame):
        if isinstance(frame, BotInterruptionFrame):
            return [frame]
        if not (isinstance(frame, TranscriptionFrame) and frame.is_final and frame.text.strip()):
            return [frame]
        who = f"[{frame.speaker}] " if frame.speaker else ""
        self.messages.append({"role": "user", "content": who + frame.text})
        reply = self.generate(self.messages)
        out: List[Frame] = [frame]
        call = self._parse_tool_call(reply)
        if call is not None and call["tool"] in self.tools:
            result = self.tools[call["tool"]](**call.get("arguments", {}))
            out.append(ToolCallFrame(frame.timestamp, call["tool"], call.get("arguments", {}), result))
            self.messages.append({"role": "assistant", "content": reply})
            self.messages.append({"role": "tool", "content": json.dumps({"name": call["tool"], "result": result}, default=str)})
            reply = self.generate(self.messages)
        self.messages.append({"role": "assistant", "content": reply})
        self._trim()
        out.append(LLMTextFrame(frame.timestamp, reply))
        return out

    @staticmethod
    def _parse_tool_call(reply: str) -> Optional[Dict[str, Any]]:
        m = re.search(r"\{.*\}", reply, flags=re.S)
        if not m:
            return None
        try:
            obj = json.loads(m.group(0))
        except json.JSONDecodeError:
            return None
        return obj if isinstance(obj, dict) and "tool" in obj else None


class TTSService(FrameProcessor):
    """``synthesize(text) -> (audio, sample_rate)``; replies are split into sentences so that audio starts early, and an
    interruption drops what is still queued."""

    def __init__(self, synthesize: Callable[[str], Any], sentence_split: bool = True):
        self.synthesize, self.sentence_split = synthesize, sentence_split
        self.interrupted = False

    def process(self, frame):
        if isinstance(frame, BotInterruptionFrame):
            self.interrupted = True
            return [frame]
        if isinstance(frame, UserStoppedSpeakingFrame):
            self.interrupted = False
            return [frame]
        if not isinstance(frame, LLMTextFrame):
            return [frame]
        parts = [s.strip() for s in re.split(r"(?<=[.!?])\s+", frame.text) if s.strip()] if self.sentence_split else [frame.text]
        out: List[Frame] = [frame]
        for s in parts:
            if self.interrupted:
                break
            audio, sr = self.synthesize(s)
            out.append(TTSAudioFrame(frame.timestamp, np.asarray(audio, np.float32), int(sr), s))
        return out


class AudioLogger(FrameProcessor):
    """Writes user and bot audio of a session to WAV files and the conversation to a JSON-lines log."""

    def __init__(self, log_dir: str, session_id: str = "session"):
        self.dir = os.path.join(log_dir, session_id)
        os.makedirs(self.dir, exist_ok=True)
        self.user: List[np.ndarray] = []
        self.bot: List[np.ndarray] = []
        self.sr = {"user": 16000, "bot": 16000}
        self.events = open(os.path.join(self.dir, "events.jsonl"), "a", encoding="utf-8")

    def process(self, frame):
        if isinstance(frame, TTSAudioFrame):
            self.bot.append(frame.audio)
            self.sr["bot"] = frame.sample_rate
        elif isinstance(frame, AudioRawFrame):
            self.user.append(frame.audio)
            self.sr["user"] = frame.sample_rate
        elif isinstance(frame, (TranscriptionFrame, LLMTextFrame, ToolCallFrame)):
            d = {k: v for k, v in frame.__dict__.items() if isinstance(v, (str, int, float, bool, dict, type(None)))}
            self.events.write(json.dumps({"type": type(frame).__name__, "wall": time.time(), **d}, default=str) + "\n")
            self.events.flush()
        elif isinstance(frame, EndFrame):
            self.close()
        return [frame]

    def close(self):
        for name, chunks in (("user", self.user), ("bot", self.bot)):
            if chunks:
                x = np.clip(np.concatenate(chunks), -1, 1)
                with wave.open(os.path.join(self.dir, name + ".wav"), "wb") as w:
                    w.setnchannels(1)
                    w.setsampwidth(2)
                    w.setframerate(self.sr[name])
                    w.writeframes((x * 32767).astype("<i2").tobytes())
        if not self.events.closed:
            self.events.close()


def build_voice_agent(stt_step, generate, synthesize, diar_step=None, log_dir: Optional[str] = None, system_prompt: Optional[str] = None,
                      tools: Optional[Dict[str, Callable[..., Any]]] = None, **turn_kw) -> Pipeline:
    """Microphone → STT (→ diarization) → turn taking → LLM → TTS (→ logger)."""
    procs: List[FrameProcessor] = [StreamingSTTService(stt_step)]
    if diar_step is not None:
        procs.append(StreamingDiarService(diar_step))
    procs += [TurnTakingService(**turn_kw), _FinalOnTurnEnd(), LLMService(generate, system_prompt, tools), TTSService(synthesize)]
    if log_dir is not None:
        procs.append(AudioLogger(log_dir))
    return Pipeline(procs)


class _FinalOnTurnEnd(FrameProcessor):
    """Promotes the latest interim transcript to a final one when the user's turn ends."""

    def __init__(self):
        self.partial: Optional[TranscriptionFrame] = None

    def process(self, frame):
        if isinstance(frame, TranscriptionFrame):
            if frame.is_final:
                self.partial = None
            else:
                self.partial = frame
            return [frame]
        if isinstance(frame, UserStoppedSpeakingFrame) and self.partial is not None:
            p, self.partial = self.partial, None
            return [frame, TranscriptionFrame(frame.timestamp, p.text, True, p.speaker)]
        return [frame]

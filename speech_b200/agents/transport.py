"""Websocket transport of the voice agent: a client streams microphone audio, the server streams back the bot's speech and
JSON events.

Wire protocol (one websocket connection = one conversation):

* client -> server, binary: little-endian 16-bit PCM mono at ``sample_rate``, any chunk length;
* client -> server, text: JSON ``{"type": "config", "sample_rate": 16000}`` (before the first audio), ``{"type": "end"}``;
* server -> client, binary: the bot's speech, 16-bit PCM mono at the synthesiser's rate;
* server -> client, text: JSON events ``{"type": "transcript", "text", "final", "speaker"}``, ``{"type": "bot_text", "text"}``,
  ``{"type": "tool_call", "name", "arguments", "result"}``, ``{"type": "user_started"}``, ``{"type": "user_stopped"}``,
  ``{"type": "interruption"}`` (the client drops audio it has not played yet), ``{"type": "audio_format", "sample_rate"}``,
  ``{"type": "end"}``.

The reference serves the same role with pipecat's websocket transports and a browser client (``examples/voice_agent/server``,
``nemo/agents/voice_agent/pipecat/transports``); here the transport is a small adapter between any websocket object with
``receive()`` / ``send_bytes()`` / ``send_text()`` coroutines (Starlette / FastAPI, aiohttp through :class:`AiohttpSocket`) and a
:class:`speech_b200.agents.voice_agent.Pipeline`.
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import numpy as np

from .voice_agent import (AudioRawFrame, BotInterruptionFrame, EndFrame, Frame, LLMTextFrame, Pipeline, ToolCallFrame, TranscriptionFrame,
                          TTSAudioFrame, UserStartedSpeakingFrame, UserStoppedSpeakingFrame)


def pcm16_to_float(data: bytes) -> np.ndarray:
    return np.frombuffer(data[: len(data) // 2 * 2], dtype="<i2").astype(np.float32) / 32768.0


def float_to_pcm16(x: np.ndarray) -> bytes:
    return (np.clip(np.asarray(x, dtype=np.float32), -1.0, 1.0) * 32767.0).astype("<i2").tobytes()


def frame_to_event(f: Frame) -> Optional[Dict[str, Any]]:
    if isinstance(f, TranscriptionFrame):
        return {"type": "transcript", "text": f.text, "final": bool(f.is_final), "speaker": f.speaker, "t": f.timestamp}
    if isinstance(f, LLMTextFrame):
        return {"type": "bot_text", "text": f.text, "t": f.timestamp}
    if isinstance(f, ToolCallFrame):
        return {"type": "tool_call", "name": f.name, "arguments": f.arguments, "result": f.result if isinstance(f.result, (str, int, float, bool, type(None), list, dict)) else str(f.result)}
    if isinstance(f, UserStartedSpeakingFrame):
        return {"type": "user_started", "t": f.timestamp}
    if isinstance(f, UserStoppedSpeakingFrame):
        return {"type": "user_stopped", "t": f.timestamp}
    if isinstance(f, BotInterruptionFrame):
        return {"type": "interruption", "t": f.timestamp}
    if isinstance(f, EndFrame):
        return {"type": "end"}
    return None


class WebsocketAudioTransport:
    """Runs one conversation: ``await transport.serve(ws)``.  ``frame_ms``: the pipeline is fed fixed-size frames regardless of
    how the client chunks its audio (the streaming recogniser and the turn-taking timers count frames)."""

    def __init__(self, pipeline: Pipeline, sample_rate: int = 16000, frame_ms: float = 80.0, tts_chunk_ms: float = 200.0):
        self.pipeline, self.sr, self.frame_ms, self.tts_chunk_ms = pipeline, sample_rate, frame_ms, tts_chunk_ms
        self.samples_in = 0
        self._buf = np.zeros(0, np.float32)
        self._tts_rate_sent: Optional[int] = None

    async def _emit(self, ws, frames: List[Frame]) -> None:
        for f in frames:
            if isinstance(f, TTSAudioFrame):
                if self._tts_rate_sent != f.sample_rate:
                    await ws.send_text(json.dumps({"type": "audio_format", "sample_rate": int(f.sample_rate)}))
                    self._tts_rate_sent = f.sample_rate
                if f.text:
                    await ws.send_text(json.dumps({"type": "bot_speech", "text": f.text}))
                step = max(1, int(f.sample_rate * self.tts_chunk_ms / 1000))
                for i in range(0, len(f.audio), step):
                    await ws.send_bytes(float_to_pcm16(f.audio[i:i + step]))
                continue
            ev = frame_to_event(f)
            if ev is not None:
                await ws.send_text(json.dumps(ev))

    async def _feed(self, ws, audio: np.ndarray) -> None:
        self._buf = np.concatenate([self._buf, audio])
        n = max(1, int(self.sr * self.frame_ms / 1000))
        while len(self._buf) >= n:
            chunk, self._buf = self._buf[:n], self._buf[n:]
            t = self.samples_in / self.sr
            self.samples_in += n
            await self._emit(ws, self.pipeline.push(AudioRawFrame(t, chunk, self.sr)))

    async def serve(self, ws) -> None:
        while True:
            msg = await ws.receive()
            kind = msg.get("type")
            if kind in ("websocket.disconnect", "close", "closed"):
                break
            data, text = msg.get("bytes"), msg.get("text")
            if data:
                await self._feed(ws, pcm16_to_float(data))
            elif text:
                try:
                    ctl = json.loads(text)
                except ValueError:
                    await ws.send_text(json.dumps({"type": "error", "message": "text messages must be JSON"}))
                    continue
                if ctl.get("type") == "config":
                    if self.samples_in:
                        await ws.send_text(json.dumps({"type": "error", "message": "config must come before the first audio"}))
                    else:
                        self.sr = int(ctl.get("sample_rate", self.sr))
                elif ctl.get("type") == "end":
                    if len(self._buf):                      # flush the partial frame, zero padded
                        n = max(1, int(self.sr * self.frame_ms / 1000))
                        await self._feed(ws, np.zeros(n - len(self._buf), np.float32))
                    await self._emit(ws, self.pipeline.push(EndFrame(self.samples_in / self.sr)))
                    await ws.send_text(json.dumps({"type": "end"}))
                    break


class AiohttpSocket:
    """Adapter giving an ``aiohttp`` websocket (server or client side) the ``receive`` / ``send_bytes`` / ``send_text`` shape."""

    def __init__(self, ws):
        self.ws = ws

    async def receive(self) -> Dict[str, Any]:
        import aiohttp

        m = await self.ws.receive()
        if m.type == aiohttp.WSMsgType.BINARY:
            return {"type": "message", "bytes": m.data}
        if m.type == aiohttp.WSMsgType.TEXT:
            return {"type": "message", "text": m.data}
        return {"type": "close"}

    async def send_bytes(self, b: bytes) -> None:
        await self.ws.send_bytes(b)

    async def send_text(self, t: str) -> None:
        await self.ws.send_str(t)

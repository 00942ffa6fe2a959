"""Command-line client of the voice-agent server: streams a WAV file in real time (or as fast as possible with ``--fast``), prints
the events and writes the bot's speech to a WAV file.

    python examples/voice_agent/client.py ws://127.0.0.1:8765/ws question.wav answer.wav [--fast]
"""
import asyncio
import json
import sys

import numpy as np


async def run(url: str, wav_in: str, wav_out: str, fast: bool = False, chunk_ms: float = 80.0):
    import aiohttp

    from speech_b200.agents.transport import float_to_pcm16, pcm16_to_float
    from speech_b200.data.audio_to_text import load_audio, save_wav

    sr = 16000
    audio = np.asarray(load_audio(wav_in, target_sr=sr), dtype=np.float32)
    audio = np.concatenate([audio, np.zeros(sr, np.float32)])          # a second of silence lets the agent take its turn
    out, out_sr = [], 22050
    async with aiohttp.ClientSession() as sess:
        async with sess.ws_connect(url, max_msg_size=0) as ws:
            await ws.send_str(json.dumps({"type": "config", "sample_rate": sr}))

            async def sender():
                n = int(sr * chunk_ms / 1000)
                for i in range(0, len(audio), n):
                    await ws.send_bytes(float_to_pcm16(audio[i:i + n]))
                    if not fast:
                        await asyncio.sleep(chunk_ms / 1000)
                await ws.send_str(json.dumps({"type": "end"}))

            task = asyncio.ensure_future(sender())
            async for m in ws:
                if m.type == aiohttp.WSMsgType.BINARY:
                    out.append(pcm16_to_float(m.data))
                elif m.type == aiohttp.WSMsgType.TEXT:
                    ev = json.loads(m.data)
                    if ev.get("type") == "audio_format":
                        out_sr = int(ev["sample_rate"])
                    elif ev.get("type") == "interruption":
                        out.clear()
                    print(ev)
                    if ev.get("type") == "end":
                        break
                else:
                    break
            await task
    if out:
        save_wav(wav_out, np.concatenate(out), out_sr)
        print(f"wrote {wav_out} ({sum(len(o) for o in out) / out_sr:.2f} s)")


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if len(args) != 3:
        raise SystemExit(__doc__)
    asyncio.run(run(args[0], args[1], args[2], fast="--fast" in sys.argv))

"""Voice-agent websocket server: streaming speech recognition -> turn taking -> language model -> speech synthesis, one
conversation per websocket connection (protocol: ``speech_b200/agents/transport.py``).

    python examples/voice_agent/server.py asr_model=stt.nemo [tts_model=tts.nemo] [llm_path=/models/qwen] port=8765
    python examples/voice_agent/client.py ws://127.0.0.1:8765/ws question.wav answer.wav

Without ``llm_path`` the bot answers with a rule (it repeats what it understood), without ``tts_model`` it answers with a short tone
per word, so the server can be brought up and the transport exercised before the models are in place.
(reference: ``examples/voice_agent/server/server.py``)."""
import numpy as np

from speech_b200.agents.transport import WebsocketAudioTransport
from speech_b200.agents.voice_agent import build_voice_agent
from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.utils.logging import logging

DEFAULTS = {"asr_model": None, "tts_model": None, "llm_path": None, "host": "127.0.0.1", "port": 8765, "sample_rate": 16000, "frame_ms": 80.0,
            "system_prompt": "You are a helpful voice assistant. Answer briefly.", "log_dir": None, "max_new_tokens": 64,
            "decode_every_frames": 4, "turn": {"max_silence": 0.64, "speech_threshold": 0.01, "min_speech": 0.1}}


def make_stt(cfg):
    """``step(chunk) -> (partial text, False)``.  With a model, the audio of the running utterance is kept and re-transcribed every
    ``decode_every_frames`` frames (turns are short; a cache-aware streaming model can be plugged in through
    ``speech_b200.inference`` instead); the buffer restarts after ``turn.max_silence`` of quiet."""
    thr, max_sil = float(cfg.turn.speech_threshold), float(cfg.turn.max_silence)
    if cfg.asr_model is None:
        # no recogniser: report speech activity only, so that turn taking and the reply path can be tried
        def step(chunk):
            return ("(speech)" if float(np.sqrt((chunk ** 2).mean() + 1e-12)) > thr else None), False
        return step
    from speech_b200.models.asr_model import ASRModel

    model = ASRModel.restore_from(cfg.asr_model).eval()
    state = {"buf": np.zeros(0, np.float32), "quiet": 0.0, "frames": 0, "text": ""}

    def step(chunk):
        loud = float(np.sqrt((chunk ** 2).mean() + 1e-12)) > thr
        state["quiet"] = 0.0 if loud else state["quiet"] + len(chunk) / cfg.sample_rate
        if state["quiet"] >= max_sil and not loud:
            state.update(buf=np.zeros(0, np.float32), frames=0, text="")
            return None, False
        state["buf"] = np.concatenate([state["buf"], chunk])
        state["frames"] += 1
        if state["frames"] % int(cfg.decode_every_frames) == 0 and len(state["buf"]) > 0.2 * cfg.sample_rate:
            hyp = model.transcribe([state["buf"]], batch_size=1)
            hyp = hyp[0] if isinstance(hyp, tuple) else hyp
            state["text"] = hyp[0].text if hasattr(hyp[0], "text") else str(hyp[0])
        return (state["text"] or None), False
    return step


def make_llm(cfg):
    if cfg.llm_path is None:
        return lambda history: "You said: " + (history[-1]["content"] if history else "")
    import torch

    from speech_b200.speechlm.llm import CausalLM
    from speech_b200.tokenizers import build_tokenizer

    lm = CausalLM.from_pretrained(cfg.llm_path).eval()
    tok = build_tokenizer({"type": "hf", "pretrained_model_name": cfg.llm_path})

    def generate(history):
        prompt = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in history) + "<|im_start|>assistant\n"
        ids = torch.tensor([tok.text_to_ids(prompt)])
        out = lm.generate(input_ids=ids, max_new_tokens=cfg.max_new_tokens, eos_token_id=lm.config.eos_token_id)
        return tok.ids_to_text(out[0].tolist()).split("<|im_end|>")[0].strip()
    return generate


def make_tts(cfg):
    if cfg.tts_model is None:
        def synth(text):
            sr, words = 22050, max(1, len(text.split()))
            t = np.arange(int(0.12 * sr)) / sr
            beep = (0.2 * np.sin(2 * np.pi * 440 * t) * np.hanning(len(t))).astype(np.float32)
            return np.concatenate([np.concatenate([beep, np.zeros(int(0.05 * sr), np.float32)]) for _ in range(words)]), sr
        return synth
    from speech_b200.tts.magpietts import MagpieTTSModel

    tts = MagpieTTSModel.restore_from(cfg.tts_model).eval()
    return lambda text: (tts.generate_speech(text).cpu().numpy(), int(getattr(tts._codec, "sample_rate", 22050)))


def build_app(cfg):
    from fastapi import FastAPI, WebSocket

    stt, llm, tts = make_stt(cfg), make_llm(cfg), make_tts(cfg)
    app = FastAPI()

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.websocket("/ws")
    async def ws_endpoint(ws: WebSocket):
        await ws.accept()
        agent = build_voice_agent(stt, llm, tts, log_dir=cfg.log_dir, system_prompt=cfg.system_prompt, **OmegaConf.to_container(cfg.turn))
        try:
            await WebsocketAudioTransport(agent, cfg.sample_rate, cfg.frame_ms).serve(ws)
        finally:
            try:
                await ws.close()
            except Exception:
                pass
    return app


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    import uvicorn

    logging.info(f"voice agent on ws://{cfg.host}:{cfg.port}/ws")
    uvicorn.run(build_app(cfg), host=cfg.host, port=int(cfg.port), log_level="warning")


if __name__ == "__main__":
    main()

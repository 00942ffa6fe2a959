"""Evaluate the full duplex voice-chat stack (listening half + speaking half in lock step) on recorded user turns: agent text per
frame, agent audio, turn-taking statistics against the reference turns, and response text quality when references exist.

python examples/speechlm2/nemotron_voicechat_eval.py stt=duplex_stt.nemo tts=eartts.nemo codec=codec.nemo manifest=test.json output_dir=vc_eval
Manifest lines: ``{"audio_filepath": user channel, "text": reference agent text (optional), "user_end_time": seconds (optional)}``.
(reference script: ``examples/speechlm2/nemotron_voicechat_eval.py``)."""
import json
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.data.audio_to_text import load_audio, read_manifest, save_wav
from speech_b200.speechlm.duplex import DuplexSTTModel
from speech_b200.speechlm.ear_tts import DuplexEARTTS, NemotronVoiceChat
from speech_b200.speechlm.metrics import TurnTakingMetrics
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"stt": None, "tts": None, "codec": None, "manifest": None, "output_dir": "voicechat_eval", "cuda": None, "sample_rate": 22050, "sampling": {"temperature": 0.8}}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    stt = DuplexSTTModel.restore_from(cfg.stt, map_location=dev).to(dev).eval()
    tts = DuplexEARTTS.restore_from(cfg.tts, map_location=dev).to(dev).eval()
    codec = ModelPT.restore_from(cfg.codec, map_location=dev).to(dev).eval() if cfg.codec else None
    chat = NemotronVoiceChat(stt, tts).to(dev)
    os.makedirs(cfg.output_dir, exist_ok=True)
    frame_sec = float(stt.perception.token_equivalent_duration)
    tt = TurnTakingMetrics(eos_token_id=stt.text_eos_id, bos_token_id=stt.text_bos_id, latency_multiplier=frame_sec)
    hyps, refs = [], []
    for k, it in enumerate(read_manifest(cfg.manifest)):
        x = torch.as_tensor(load_audio(it["audio_filepath"]), dtype=torch.float32, device=dev)
        out = chat.offline_inference(x[None], torch.tensor([x.numel()], device=dev), **dict(cfg.sampling))
        text = out["text"][0]
        hyps.append(text)
        rec = {"text": text, "frames": int(out["lengths"][0])}
        if codec is not None:
            lens = out["lengths"]
            audio, alen = codec.decode(tokens=out["codes"].transpose(1, 2), tokens_len=lens)
            p = os.path.join(cfg.output_dir, f"agent_{k:05d}.wav")
            save_wav(p, audio[0, : int(alen[0])].float().cpu().numpy(), cfg.sample_rate)
            rec["agent_audio"] = p
        if it.get("user_end_time") is not None:
            src = torch.full_like(out["tokens"], stt.text_pad_id)
            src[0, min(src.shape[1] - 1, int(round(float(it["user_end_time"]) / frame_sec)))] = stt.text_eos_id
            tt.update("voicechat", src, out["tokens"])
        if it.get("text"):
            refs.append(it["text"])
        with open(os.path.join(cfg.output_dir, f"result_{k:05d}.json"), "w") as f:
            json.dump(rec, f, indent=2)
    summary = {"items": len(hyps)}
    if refs and len(refs) == len(hyps):
        summary["wer_vs_reference_response"] = word_error_rate(hyps, refs)
    summary.update({k: float(v) for k, v in tt.compute().items()})
    with open(os.path.join(cfg.output_dir, "summary.json"), "w") as f:
        json.dump(summary, f, indent=2)
    logging.info(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()

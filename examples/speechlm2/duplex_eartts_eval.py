"""Evaluate the streaming text-to-speech half of the duplex stack: synthesise the agent channel of every test item, then report
real-time factor and, when scorers are given, intelligibility (ASR WER / CER on the audio) and speaker similarity to the reference.

python examples/speechlm2/duplex_eartts_eval.py checkpoint=eartts.nemo codec=codec.nemo manifest=test.json output_dir=eval [asr_model=asr.nemo] [speaker_model=titanet.nemo]
Manifest lines: ``{"text": ..., "audio_filepath": reference (optional)}``.
(reference script: ``examples/speechlm2/duplex_eartts_eval.py``)."""
import json
import os
import time

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.data.audio_to_text import read_manifest, save_wav
from speech_b200.speechlm.ear_tts import DuplexEARTTS
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"checkpoint": None, "codec": None, "manifest": None, "output_dir": "eartts_eval", "asr_model": None, "speaker_model": None, "cuda": None,
            "frames_per_token": 4, "sample_rate": 22050, "sampling": {"temperature": 0.8}}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    codec = ModelPT.restore_from(cfg.codec, map_location=dev).to(dev).eval() if cfg.codec else None
    model = DuplexEARTTS.restore_from(cfg.checkpoint, map_location=dev).to(dev).eval()
    model.audio_codec = codec
    tok = model.tokenizer
    os.makedirs(cfg.output_dir, exist_ok=True)
    items = read_manifest(cfg.manifest)
    audio_sec = wall = 0.0
    paths = []
    for k, it in enumerate(items):
        ids = tok.text_to_ids(it["text"]) if tok is not None else [min(ord(c), model.tts.text_vocab - 1) for c in it["text"]]
        pad = getattr(model.tts, "text_pad_id", 0)
        frames = [i for t in ids for i in [t] + [pad] * (int(cfg.frames_per_token) - 1)]       # the text channel is frame aligned
        t0 = time.perf_counter()
        out = model.offline_inference(torch.tensor([frames], device=dev), decode_audio=codec is not None, **dict(cfg.sampling))
        if dev != "cpu":
            torch.cuda.synchronize()
        wall += time.perf_counter() - t0
        torch.save(out["codes"].cpu(), os.path.join(cfg.output_dir, f"codes_{k:05d}.pt"))
        if "audio" in out:
            n = int(out["audio_len"][0])
            p = os.path.join(cfg.output_dir, f"gen_{k:05d}.wav")
            save_wav(p, out["audio"][0, :n].float().cpu().numpy(), cfg.sample_rate)
            paths.append(p)
            audio_sec += n / cfg.sample_rate
    summary = {"items": len(items), "rtf": wall / audio_sec if audio_sec else None, "audio_seconds": audio_sec}
    if cfg.asr_model and paths:
        from speech_b200.models.asr_model import ASRModel

        asr = ASRModel.restore_from(cfg.asr_model, map_location=dev).to(dev).eval()
        hyp = [h.text if hasattr(h, "text") else h for h in asr.transcribe(paths, batch_size=8)]
        ref = [it["text"].lower() for it in items]
        summary["wer"], summary["cer"] = word_error_rate(hyp, ref), word_error_rate(hyp, ref, use_cer=True)
    if cfg.speaker_model and paths and all(it.get("audio_filepath") for it in items):
        from speech_b200.models import EncDecSpeakerLabelModel

        spk = EncDecSpeakerLabelModel.restore_from(cfg.speaker_model, map_location=dev).to(dev).eval()
        a = torch.as_tensor(spk.batch_inference(paths)[0])
        b = torch.as_tensor(spk.batch_inference([it["audio_filepath"] for it in items])[0])
        summary["speaker_similarity"] = float(torch.nn.functional.cosine_similarity(a, b).mean())
    with open(os.path.join(cfg.output_dir, "summary.json"), "w") as f:
        json.dump(summary, f, indent=2)
    logging.info(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()

"""Synthesise speech with MagpieTTS and report the real-time factor (reference: ``examples/tts/magpietts_inference.py``).

python examples/tts/magpietts_inference.py model_path=magpie.nemo text="Hello there." output=out.wav use_cfg=true cfg_scale=2.5"""
import time

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import save_wav
from speech_b200.tts.magpietts import MagpieTTSModel
from speech_b200.utils.logging import logging


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "text": None, "text_file": None, "output": "out.wav", "temperature": 0.7, "topk": 80,
                                            "use_cfg": True, "cfg_scale": 2.5, "max_decoder_steps": 500, "long_form": False}), cfg)
    model = MagpieTTSModel.restore_from(cfg.model_path).eval()
    text = cfg.text if cfg.text else open(cfg.text_file, encoding="utf-8").read()
    kw = dict(temperature=cfg.temperature, topk=cfg.topk, use_cfg=cfg.use_cfg, cfg_scale=cfg.cfg_scale, max_decoder_steps=cfg.max_decoder_steps)
    t0 = time.perf_counter()
    if cfg.long_form:
        audio = model.generate_speech(text, **kw)
    else:
        a, n = model.do_tts(text, **kw)
        audio = a[0, : int(n[0])]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    sr = model._codec.sample_rate
    save_wav(cfg.output, audio.float().cpu().numpy(), sr)
    logging.info(f"{audio.numel() / sr:.2f} s of audio in {dt:.2f} s (RTF {dt / max(audio.numel() / sr, 1e-9):.3f})")


if __name__ == "__main__":
    main()

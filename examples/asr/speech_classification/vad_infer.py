"""Voice activity detection with a window-classification model (MarbleNet): frame posteriors by overlapped windows, smoothing,
thresholding with hysteresis, duration filtering; writes one RTTM per recording and a manifest that points to them.

python examples/asr/speech_classification/vad_infer.py vad.model_path=vad.nemo dataset=manifest.json out_dir=vad_out \
    vad.parameters.window_length_in_sec=0.63 vad.parameters.shift_length_in_sec=0.08 vad.parameters.postprocessing.onset=0.5
(reference script: ``examples/asr/speech_classification/vad_infer.py``)."""
import json
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.utils import vad_utils as V
from speech_b200.utils.logging import logging

DEFAULTS = {"dataset": None, "out_dir": "vad_out", "cuda": None, "frame_model": False,
            "vad": {"model_path": None, "parameters": {"window_length_in_sec": 0.63, "shift_length_in_sec": 0.08, "smoothing": "median", "speech_class": 1,
                                                        "postprocessing": {"onset": 0.5, "offset": 0.3, "pad_onset": 0.2, "pad_offset": 0.2, "min_duration_on": 0.2,
                                                                           "min_duration_off": 0.2, "filter_speech_first": True}}}}


def frame_posteriors(model, audio: torch.Tensor, p, frame_model: bool) -> tuple:
    if not frame_model:
        return V.generate_vad_frame_pred(model, audio, window_length_in_sec=p.window_length_in_sec, shift_length_in_sec=p.shift_length_in_sec,
                                         speech_class=p.speech_class, smoothing_method=p.smoothing or "mean"), 0.01
    dev = next(model.parameters()).device
    with torch.no_grad():
        logits = model(input_signal=audio[None].to(dev), input_signal_length=torch.tensor([audio.numel()], device=dev))
    logits = logits[0] if isinstance(logits, (tuple, list)) else logits
    probs = torch.softmax(logits.float(), dim=-1)[0, :, p.speech_class].cpu()
    return probs, audio.numel() / 16000.0 / max(1, probs.numel())


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    model = ModelPT.restore_from(cfg.vad.model_path, map_location=dev).to(dev).eval()
    os.makedirs(cfg.out_dir, exist_ok=True)
    pp = {k: float(v) for k, v in dict(cfg.vad.parameters.postprocessing).items()}
    rows = []
    for it in read_manifest(cfg.dataset):
        x = torch.as_tensor(load_audio(it["audio_filepath"], offset=float(it.get("offset", 0) or 0), duration=it.get("duration")), dtype=torch.float32)
        probs, unit = frame_posteriors(model, x, cfg.vad.parameters, bool(cfg.frame_model))
        seg = V.generate_vad_segment_table(probs, pp, unit)
        uid = os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        rttm = os.path.join(cfg.out_dir, uid + ".rttm")
        V.write_rttm(rttm, seg, uid)
        torch.save(probs, os.path.join(cfg.out_dir, uid + ".frame.pt"))
        rows.append(dict(it, rttm_filepath=rttm, speech_seconds=float((seg[:, 1] - seg[:, 0]).sum()) if seg.numel() else 0.0))
    out = os.path.join(cfg.out_dir, "vad_out.json")
    with open(out, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    logging.info(f"{len(rows)} recordings -> {out}")
    return rows


if __name__ == "__main__":
    main()

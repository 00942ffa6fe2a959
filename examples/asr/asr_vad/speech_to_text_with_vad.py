"""Transcribe long recordings with voice activity detection in front: the VAD segments (merged up to ``max_segment`` seconds) are
transcribed as a batch and joined per recording, so silence and noise never reach the recogniser.

python examples/asr/asr_vad/speech_to_text_with_vad.py asr_model=asr.nemo vad_model=vad.nemo manifest_filepath=long.json output_filename=out.json
(reference script: ``examples/asr/asr_vad/speech_to_text_with_vad.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils import vad_utils as V
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"asr_model": None, "vad_model": None, "manifest_filepath": None, "output_filename": "asr_with_vad.json", "batch_size": 16, "cuda": None,
            "max_segment": 20.0, "use_energy_vad": False,
            "vad": {"window_length_in_sec": 0.63, "shift_length_in_sec": 0.08, "smoothing": "median",
                    "postprocessing": {"onset": 0.5, "offset": 0.3, "pad_onset": 0.2, "pad_offset": 0.2, "min_duration_on": 0.2, "min_duration_off": 0.3}}}


def group_segments(seg: torch.Tensor, max_len: float):
    """Neighbouring speech segments are joined while the joined stretch stays under ``max_len`` seconds."""
    out = []
    for a, b in seg.tolist():
        if out and b - out[-1][0] <= max_len:
            out[-1][1] = b
        else:
            out.append([a, b])
    return out


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    asr = ASRModel.restore_from(cfg.asr_model, map_location=dev).to(dev).eval()
    vad = None if cfg.use_energy_vad else ModelPT.restore_from(cfg.vad_model, map_location=dev).to(dev).eval()
    pp = {k: float(v) for k, v in dict(cfg.vad.postprocessing).items()}
    items = read_manifest(cfg.manifest_filepath)
    preds = []
    for it in items:
        x = load_audio(it["audio_filepath"])
        if vad is None:
            from speech_b200.models.diarizers import energy_vad

            seg = torch.tensor(energy_vad(x, 16000), dtype=torch.float32).reshape(-1, 2)
        else:
            probs = V.generate_vad_frame_pred(vad, torch.as_tensor(x), window_length_in_sec=cfg.vad.window_length_in_sec,
                                              shift_length_in_sec=cfg.vad.shift_length_in_sec, smoothing_method=cfg.vad.smoothing)
            seg = V.generate_vad_segment_table(probs, pp)
        pieces = [x[int(a * 16000): int(b * 16000)] for a, b in group_segments(seg, cfg.max_segment)]
        pieces = [p for p in pieces if len(p) >= 1600]
        hyps = asr.transcribe(pieces, batch_size=cfg.batch_size) if pieces else []
        preds.append(" ".join((h.text if hasattr(h, "text") else h).strip() for h in hyps).strip())
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, p in zip(items, preds):
            f.write(json.dumps(dict(it, pred_text=p), ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(preds, [it['text'] for it in items]):.2f}%")
    return preds


if __name__ == "__main__":
    main()

"""Transcribe a manifest (unless it already has predictions) and score it: WER / CER, optionally without punctuation and case.

python examples/asr/speech_to_text_eval.py model_path=m.nemo dataset_manifest=test.json output_filename=eval.json \
    use_cer=false text_processing.do_lowercase=true text_processing.rm_punctuation=true tolerance=null only_score_manifest=false
(reference script: ``examples/asr/speech_to_text_eval.py``)."""
import json
import re
import sys

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"model_path": None, "pretrained_name": None, "dataset_manifest": None, "output_filename": "evaluation_transcripts.json", "batch_size": 32,
            "cuda": None, "use_cer": False, "tolerance": None, "only_score_manifest": False, "scores_per_sample": False,
            "text_processing": {"do_lowercase": False, "rm_punctuation": False, "punctuation_marks": ".,?!", "separate_punctuation": False}}


def clean(text: str, tp) -> str:
    if tp.separate_punctuation:
        text = re.sub(f"([{re.escape(tp.punctuation_marks)}])", r" \1 ", text)
    if tp.rm_punctuation:
        text = re.sub(f"[{re.escape(tp.punctuation_marks)}]", " ", text)
    if tp.do_lowercase:
        text = text.lower()
    return re.sub(r"\s+", " ", text).strip()


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    items = read_manifest(cfg.dataset_manifest)
    if not cfg.only_score_manifest:
        dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
        model = (ASRModel.restore_from(cfg.model_path, map_location=dev) if cfg.model_path else ASRModel.from_pretrained(cfg.pretrained_name)).to(dev).eval()
        hyps = model.transcribe([it["audio_filepath"] for it in items], batch_size=cfg.batch_size)
        for it, h in zip(items, hyps):
            it["pred_text"] = h.text if hasattr(h, "text") else h
    elif any("pred_text" not in it for it in items):
        raise ValueError("only_score_manifest=true needs a `pred_text` field in every line")
    refs = [clean(it["text"], cfg.text_processing) for it in items]
    hyps = [clean(it["pred_text"], cfg.text_processing) for it in items]
    name = "CER" if cfg.use_cer else "WER"
    score = word_error_rate(hyps, refs, use_cer=bool(cfg.use_cer))
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, r, h in zip(items, refs, hyps):
            if cfg.scores_per_sample:
                it = dict(it, **{name.lower(): word_error_rate([h], [r], use_cer=bool(cfg.use_cer))})
            f.write(json.dumps(it, ensure_ascii=False) + "\n")
    logging.info(f"Dataset {name} = {100 * score:.2f}%")
    print(f"{name}: {score:.4f}")
    if cfg.tolerance is not None and score > float(cfg.tolerance):
        logging.error(f"{name} {score:.4f} exceeds the tolerance {cfg.tolerance}")
        sys.exit(1)
    return score


if __name__ == "__main__":
    main()

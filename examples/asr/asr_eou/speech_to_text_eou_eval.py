"""Evaluate end-of-utterance detection of an EOU transducer: the model's predicted end time per utterance against the reference
end; reports precision / recall, early cut-offs and latency percentiles.

python examples/asr/asr_eou/speech_to_text_eou_eval.py model_path=eou.nemo dataset_manifest=test.json [collar=0.1]
(reference script: ``examples/asr/asr_eou/speech_to_text_eou_eval.py``)."""
import json

import numpy as np
import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.models.asr_variants import evaluate_eou
from speech_b200.utils.logging import logging

DEFAULTS = {"model_path": None, "dataset_manifest": None, "output_filename": "eou_eval.json", "batch_size": 16, "collar": 0.0, "cuda": None}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    model = ASRModel.restore_from(cfg.model_path, map_location=dev).to(dev).eval()
    items = read_manifest(cfg.dataset_manifest)
    hyps = model.transcribe([it["audio_filepath"] for it in items], batch_size=cfg.batch_size, return_hypotheses=True)
    if not hasattr(model, "eou_predictions_from_hypothesis"):
        raise ValueError(f"{type(model).__name__} has no end-of-utterance tokens")
    tp = fp = fn = n = 0
    latency, early = [], []
    for it, h in zip(items, hyps):
        r = evaluate_eou(model.eou_predictions_from_hypothesis(h), [{"start_time": 0.0, "end_time": float(it.get("eou_time", it["duration"]))}],
                         collar=float(cfg.collar))
        tp, fp, fn, n = tp + r.true_positives, fp + r.false_positives, fn + r.false_negatives, n + r.num_utterances
        latency += r.latency
        early += r.early_cutoff

    lat = np.asarray(latency or [0.0])
    summary = {"precision": tp / max(1, tp + fp), "recall": tp / max(1, n), "early_cutoffs": len(early), "missing": fn,
               "latency_p50": float(np.percentile(lat, 50)), "latency_p90": float(np.percentile(lat, 90))}
    with open(cfg.output_filename, "w") as f:
        json.dump(summary, f, indent=2)
    logging.info(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()

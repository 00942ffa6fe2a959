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
    hyps = model.transcribe([it["audio_filepath"] for it in items], batch_size=cfg.batch_size, return_hypotheses=True, timestamps=True)
    spf = float(model.cfg.preprocessor.get("window_stride", 0.01)) * int(model.encoder.subsampling_factor)
    eou_id = getattr(model, "eou_token_id", None)
    preds, refs = [], []
    for it, h in zip(items, hyps):
        ys = [int(t) for t in (h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else h.y_sequence)]
        ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp if not isinstance(h.timestamp, dict) else h.timestamp.get("timestep", []))
        hit = [t for y, t in zip(ys, ts) if eou_id is not None and y == eou_id]
        end = (hit[-1] + 1) * spf if hit else (ts[-1] + 1) * spf if ts else 0.0
        preds.append({"start_time": 0.0, "end_time": float(end), "eou_pred": bool(hit) or eou_id is None})
        refs.append({"start_time": 0.0, "end_time": float(it.get("eou_time", it["duration"]))})
    r = evaluate_eou(preds, refs, collar=float(cfg.collar))
    lat = np.asarray(r.latency or [0.0])
    summary = {"precision": r.true_positives / max(1, r.true_positives + r.false_positives), "recall": r.true_positives / max(1, r.num_utterances),
               "early_cutoffs": len(r.early_cutoff), "missing": r.false_negatives, "latency_p50": float(np.percentile(lat, 50)), "latency_p90": float(np.percentile(lat, 90))}
    with open(cfg.output_filename, "w") as f:
        json.dump(summary, f, indent=2)
    logging.info(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()

"""Frame-level voice activity detection (one posterior per 20 ms frame from a frame-classification model) with optional
evaluation against RTTM / label references (AUROC and detection error rate).

python examples/asr/speech_classification/frame_vad_infer.py vad.model_path=frame_vad.nemo dataset=manifest.json out_dir=frame_vad_out [evaluate=true]
(reference script: ``examples/asr/speech_classification/frame_vad_infer.py``)."""
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner, open_dict
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.utils import vad_utils as V
from speech_b200.utils.logging import logging

import vad_infer  # noqa: E402  (same folder)


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(vad_infer.DEFAULTS), OmegaConf.create({"evaluate": False}), cfg)
    with open_dict(cfg):
        cfg.frame_model = True
    rows = vad_infer.main.__wrapped__(cfg) if hasattr(vad_infer.main, "__wrapped__") else vad_infer.main(cfg)
    if cfg.evaluate:
        tot = {"miss": 0.0, "FA": 0.0, "total": 0.0}
        aucs = []
        for r in rows:
            ref_path = r.get("rttm_ref_filepath") or r.get("label")
            if not ref_path or not os.path.exists(str(ref_path)):
                continue
            ref = V.read_rttm_as_segments(ref_path)
            hyp = V.read_rttm_as_segments(r["rttm_filepath"])
            sc = V.detection_error_rate(ref, hyp)
            for k in ("miss", "FA"):
                tot[k] += sc[k] * sc["total"]
            tot["total"] += sc["total"]
            probs = torch.load(os.path.splitext(r["rttm_filepath"])[0] + ".frame.pt")
            unit = float(r.get("duration", 0.0) or 0.0) / max(1, probs.numel()) or 0.02
            labels = V.extract_labels(ref_path, [i * unit for i in range(probs.numel())])
            aucs.append(V.frame_auroc(probs, torch.tensor(labels)))
        if tot["total"] > 0:
            logging.info(f"DetER {(tot['miss'] + tot['FA']) / tot['total']:.2f}%  miss {tot['miss'] / tot['total']:.2f}%  FA {tot['FA'] / tot['total']:.2f}%  "
                         f"AUROC {sum(aucs) / max(1, len(aucs)):.4f}")
    return rows


if __name__ == "__main__":
    main()

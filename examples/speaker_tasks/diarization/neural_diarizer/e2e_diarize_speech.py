"""End-to-end (Sortformer) diarization of a manifest, offline or streaming; writes RTTM files
(reference: ``examples/speaker_tasks/diarization/neural_diarizer/e2e_diarize_speech.py``).

python .../e2e_diarize_speech.py model_path=sortformer.nemo dataset_manifest=m.json out_rttm_dir=rttm streaming=false"""
import os

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.data.diarization import write_rttm
from speech_b200.models import SortformerEncLabelModel


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "out_rttm_dir": "pred_rttms", "batch_size": 1,
                                            "streaming": False, "postprocessing": {"onset": 0.5, "offset": 0.5, "min_duration_on": 0.1, "min_duration_off": 0.1}}), cfg)
    model = SortformerEncLabelModel.restore_from(cfg.model_path).eval()
    model.streaming_mode = bool(cfg.streaming)
    items = read_manifest(cfg.dataset_manifest)
    res = model.diarize([it["audio_filepath"] for it in items], batch_size=cfg.batch_size, postprocessing=dict(cfg.postprocessing))
    os.makedirs(cfg.out_rttm_dir, exist_ok=True)
    for it, segs in zip(items, res):
        name = os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        parsed = [(float(s.split()[0]), float(s.split()[1]), s.split()[2]) for s in segs]
        write_rttm(os.path.join(cfg.out_rttm_dir, name + ".rttm"), parsed, uniq_id=name)


if __name__ == "__main__":
    main()

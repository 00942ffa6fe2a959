"""Clustering diarization of a manifest of recordings; writes RTTM files (reference: ``.../clustering_diarizer/offline_diar_infer.py``).

python .../offline_diar_infer.py --config-path ../conf --config-name diar_infer_general diarizer.manifest_filepath=m.json diarizer.out_dir=out"""
from speech_b200.core.config import hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models import ClusteringDiarizer


@hydra_runner(config_path="../conf", config_name="diar_infer_general")
def main(cfg):
    items = read_manifest(cfg.diarizer.manifest_filepath)
    ClusteringDiarizer(cfg).diarize([it["audio_filepath"] for it in items], [it.get("num_speakers") for it in items])


if __name__ == "__main__":
    main()

"""Train a speaker identification / verification model (TitaNet, ECAPA).

Usage: python examples/speaker_tasks/recognition/speaker_reco.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/speaker_tasks/recognition/speaker_reco.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecSpeakerLabelModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../diarization/conf", config_name="titanet-small")
def main(cfg):
    run_training(EncDecSpeakerLabelModel, cfg)


if __name__ == "__main__":
    main()

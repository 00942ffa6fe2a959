"""Train the Sortformer end-to-end diarizer.

Usage: python examples/speaker_tasks/diarization/neural_diarizer/sortformer_diar_train.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/speaker_tasks/diarization/neural_diarizer/sortformer_diar_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import SortformerEncLabelModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf", config_name="sortformer_diarizer_4spk")
def main(cfg):
    run_training(SortformerEncLabelModel, cfg)


if __name__ == "__main__":
    main()

"""Train an utterance-level speech classification model (commands, language id).

Usage: python examples/asr/speech_classification/speech_to_label.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/speech_classification/speech_to_label.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecClassificationModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf", config_name="marblenet_3x2x64")
def main(cfg):
    run_training(EncDecClassificationModel, cfg)


if __name__ == "__main__":
    main()

"""Train the text-audio aligner (forward-sum loss over a convolutional attention).

Usage: python examples/tts/aligner.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/aligner.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.classic import AlignerModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="aligner")
def main(cfg):
    run_training(AlignerModel, cfg)


if __name__ == "__main__":
    main()

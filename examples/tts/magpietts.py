"""Train MagpieTTS.

Usage: python examples/tts/magpietts.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/magpietts.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.magpietts import MagpieTTSModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="magpietts")
def main(cfg):
    run_training(MagpieTTSModel, cfg)


if __name__ == "__main__":
    main()

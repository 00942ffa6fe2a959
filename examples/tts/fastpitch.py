"""Train FastPitch (parallel text-to-mel with pitch and duration predictors and a learned aligner).

Usage: python examples/tts/fastpitch.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/fastpitch.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.classic import FastPitchModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="fastpitch")
def main(cfg):
    run_training(FastPitchModel, cfg)


if __name__ == "__main__":
    main()

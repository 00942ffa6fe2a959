"""Train the HiFi-GAN vocoder (mel to waveform).

Usage: python examples/tts/hifigan.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/hifigan.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.classic import HifiGanModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="hifigan")
def main(cfg):
    run_training(HifiGanModel, cfg)


if __name__ == "__main__":
    main()

"""Train EasyMagpieTTS (decoder-only TTS over codec tokens; transformer or hybrid Mamba-2 / attention backbone).

Usage: python examples/tts/easy_magpietts.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/easy_magpietts.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.easy_magpie import EasyMagpieTTSModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="easy_magpietts")
def main(cfg):
    run_training(EasyMagpieTTSModel, cfg)


if __name__ == "__main__":
    main()

"""Train a Canary-style multitask attention encoder-decoder model.

Usage: python examples/asr/speech_multitask/speech_to_text_aed.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/speech_multitask/speech_to_text_aed.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecMultiTaskModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/speech_multitask", config_name="fast-conformer_aed")
def main(cfg):
    run_training(EncDecMultiTaskModel, cfg)


if __name__ == "__main__":
    main()

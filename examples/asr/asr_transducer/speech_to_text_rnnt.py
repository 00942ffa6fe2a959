"""Train a character-vocabulary transducer.

Usage: python examples/asr/asr_transducer/speech_to_text_rnnt.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/asr_transducer/speech_to_text_rnnt.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecRNNTModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_transducer_char")
def main(cfg):
    run_training(EncDecRNNTModel, cfg)


if __name__ == "__main__":
    main()

"""Train a transducer with end-of-utterance tokens.

Usage: python examples/asr/asr_eou/speech_to_text_rnnt_eou_train.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/asr_eou/speech_to_text_rnnt_eou_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecRNNTBPEEOUModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_transducer_bpe")
def main(cfg):
    run_training(EncDecRNNTBPEEOUModel, cfg)


if __name__ == "__main__":
    main()

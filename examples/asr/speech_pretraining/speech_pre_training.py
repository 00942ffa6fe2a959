"""Self-supervised pre-training with contrastive / MLM heads.

Usage: python examples/asr/speech_pretraining/speech_pre_training.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/speech_pretraining/speech_pre_training.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import SpeechEncDecSelfSupervisedModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/ssl", config_name="fastconformer_ssl")
def main(cfg):
    run_training(SpeechEncDecSelfSupervisedModel, cfg)


if __name__ == "__main__":
    main()

"""Self-supervised NEST pre-training (masked token prediction with a random-projection quantiser).

Usage: python examples/asr/speech_pretraining/masked_token_pred_pretrain.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/speech_pretraining/masked_token_pred_pretrain.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecMaskedTokenPredModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/ssl/nest", config_name="nest_fast-conformer")
def main(cfg):
    run_training(EncDecMaskedTokenPredModel, cfg)


if __name__ == "__main__":
    main()

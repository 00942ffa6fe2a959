"""Train an RNNT / TDT model with a sub-word tokenizer (set model.loss.loss_name=tdt for TDT).

Usage: python examples/asr/asr_transducer/speech_to_text_rnnt_bpe.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/asr_transducer/speech_to_text_rnnt_bpe.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecRNNTBPEModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_transducer_bpe")
def main(cfg):
    run_training(EncDecRNNTBPEModel, cfg)


if __name__ == "__main__":
    main()

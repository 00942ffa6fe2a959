"""Train a CTC model with a sub-word tokenizer (FastConformer-CTC-BPE).

Usage: python examples/asr/asr_ctc/speech_to_text_ctc_bpe.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/asr_ctc/speech_to_text_ctc_bpe.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecCTCModelBPE
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_ctc_bpe")
def main(cfg):
    run_training(EncDecCTCModelBPE, cfg)


if __name__ == "__main__":
    main()

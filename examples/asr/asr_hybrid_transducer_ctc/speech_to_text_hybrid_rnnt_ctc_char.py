"""Train a hybrid transducer + CTC model with a character vocabulary.

Usage: python examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_char.py key=value ...
(reference script: ``examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_char.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecHybridRNNTCTCModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer/hybrid_transducer_ctc", config_name="fastconformer_hybrid_transducer_ctc_char")
def main(cfg):
    run_training(EncDecHybridRNNTCTCModel, cfg)


if __name__ == "__main__":
    main()

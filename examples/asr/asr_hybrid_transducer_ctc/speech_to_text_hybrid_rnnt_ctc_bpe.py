"""Train a hybrid transducer + CTC model (loss = (1-w) rnnt + w ctc).

Usage: python examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_bpe.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_bpe.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecHybridRNNTCTCBPEModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer/hybrid_transducer_ctc", config_name="fastconformer_hybrid_transducer_ctc_bpe")
def main(cfg):
    run_training(EncDecHybridRNNTCTCBPEModel, cfg)


if __name__ == "__main__":
    main()

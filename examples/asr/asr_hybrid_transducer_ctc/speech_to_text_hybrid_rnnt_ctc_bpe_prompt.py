"""Train a prompt-conditioned hybrid transducer + CTC model.

Usage: python examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_bpe_prompt.py model.num_prompts=128 key=value ...
(reference script: ``examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_bpe_prompt.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecHybridRNNTCTCBPEModelWithPrompt
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer/hybrid_transducer_ctc", config_name="fastconformer_hybrid_transducer_ctc_bpe")
def main(cfg):
    run_training(EncDecHybridRNNTCTCBPEModelWithPrompt, cfg)


if __name__ == "__main__":
    main()

"""Train a transducer whose encoder output is conditioned on a prompt id per utterance (e.g. the target language).

Usage: python examples/asr/asr_transducer/speech_to_text_rnnt_bpe_prompt.py model.num_prompts=128 key=value ...
(reference script: ``examples/asr/asr_transducer/speech_to_text_rnnt_bpe_prompt.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecRNNTBPEModelWithPrompt
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_transducer_bpe")
def main(cfg):
    run_training(EncDecRNNTBPEModelWithPrompt, cfg)


if __name__ == "__main__":
    main()

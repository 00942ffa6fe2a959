"""Train SALM that also reads the hypotheses of the ASR model's own decoder (``model.perception.asr`` names a complete ASR model;
``model.asr_transcript_drop_prob`` blanks the hypothesis now and then).

Usage: python examples/speechlm2/salm_asr_decoder_train.py model.pretrained_llm=/models/qwen model.perception.asr=asr.nemo ...
(reference script: ``examples/speechlm2/salm_asr_decoder_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.duplex import SALMWithAsrDecoder
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="salm")
def main(cfg):
    run_training(SALMWithAsrDecoder, cfg)


if __name__ == "__main__":
    main()

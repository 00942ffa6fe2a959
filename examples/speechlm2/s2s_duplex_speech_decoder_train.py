"""Train the duplex speech-to-speech model whose speech channel is produced by a separate speech decoder reading the language
model's hidden states (the text channel stays with the LM head).

Usage: python examples/speechlm2/s2s_duplex_speech_decoder_train.py --config-name duplex_eartts key=value ...
(reference script: ``examples/speechlm2/s2s_duplex_speech_decoder_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.ear_tts import DuplexS2SSpeechDecoderModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="duplex_eartts")
def main(cfg):
    run_training(DuplexS2SSpeechDecoderModel, cfg)


if __name__ == "__main__":
    main()

"""Train the content / speaker disentangler on a self-supervised speech encoder (features for voice conversion and zero-shot TTS).

Usage: python examples/tts/ssl_tts.py --config-name ssl_tts key=value ...
(reference script: ``examples/tts/ssl_tts.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.classic import SSLDisentangler
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="ssl_tts")
def main(cfg):
    run_training(SSLDisentangler, cfg)


if __name__ == "__main__":
    main()

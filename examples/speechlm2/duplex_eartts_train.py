"""Train the duplex EAR-TTS speech generator (frame-aligned text channel -> codec latents through a mixture-of-Gaussians head).

Usage: python examples/speechlm2/duplex_eartts_train.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/speechlm2/duplex_eartts_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.ear_tts import DuplexEARTTS
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="duplex_eartts")
def main(cfg):
    run_training(DuplexEARTTS, cfg)


if __name__ == "__main__":
    main()

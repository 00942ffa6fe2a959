"""Train the neural audio codec.

Usage: python examples/tts/audio_codec.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/tts/audio_codec.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.tts.audio_codec import AudioCodecModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="audio_codec")
def main(cfg):
    run_training(AudioCodecModel, cfg)


if __name__ == "__main__":
    main()

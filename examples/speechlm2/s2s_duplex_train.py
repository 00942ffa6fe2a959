"""Train the duplex speech-to-speech model (agent text channel + agent audio-codec channel).

Usage: python examples/speechlm2/s2s_duplex_train.py --config-name duplex_stt model.num_codebooks=8 model.codebook_size=1024 ...
(reference script: ``examples/speechlm2/s2s_duplex_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.duplex import DuplexS2SModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="duplex_stt")
def main(cfg):
    run_training(DuplexS2SModel, cfg)


if __name__ == "__main__":
    main()

"""Train the duplex speech-to-text model (frame-synchronous agent text channel, optional user-text channel).

Usage: python examples/speechlm2/stt_duplex_train.py model.llm.hidden_size=... model.train_ds.manifest_filepath=...
(reference script: ``examples/speechlm2/stt_duplex_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.duplex import DuplexSTTModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="duplex_stt")
def main(cfg):
    run_training(DuplexSTTModel, cfg)


if __name__ == "__main__":
    main()

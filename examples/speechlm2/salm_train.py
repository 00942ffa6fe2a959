"""Train SALM (audio perception + LLM).

Usage: python examples/speechlm2/salm_train.py [--config-path DIR] [--config-name NAME] key=value ...
(reference script: ``examples/speechlm2/salm_train.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.speechlm.salm import SALM
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="salm")
def main(cfg):
    run_training(SALM, cfg)


if __name__ == "__main__":
    main()

"""Fine-tune FastPitch on a new speaker from a checkpoint (+init_from_nemo_model=fastpitch.nemo); the learning rate is constant and small.

Usage: python examples/tts/fastpitch_finetune.py +init_from_nemo_model=base.nemo model.train_ds.manifest_filepath=... model.optim.lr=2e-4 ~model.optim.sched
(reference script: ``examples/tts/fastpitch_finetune.py``)."""
from speech_b200.core.config import hydra_runner, open_dict
from speech_b200.tts.classic import FastPitchModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="fastpitch")
def main(cfg):
    if not (cfg.get("init_from_nemo_model") or cfg.get("init_from_pretrained_model") or cfg.get("init_from_ptl_ckpt")):
        raise ValueError("fine-tuning needs init_from_nemo_model / init_from_pretrained_model / init_from_ptl_ckpt")
    with open_dict(cfg):
        if cfg.model.get("optim") is not None and cfg.model.optim.get("sched") is not None:
            cfg.model.optim.sched = None
    run_training(FastPitchModel, cfg)


if __name__ == "__main__":
    main()

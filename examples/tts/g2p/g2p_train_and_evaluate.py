"""Train a grapheme-to-phoneme model (CTC over up-sampled characters, or a byte-level encoder-decoder) and report the phoneme
error rate on the validation / test manifests.

python examples/tts/g2p/g2p_train_and_evaluate.py model_type=ctc model.phonemes=phones.txt model.train_ds.manifest_filepath=train.json \
    model.validation_ds.manifest_filepath=dev.json [do_testing=true model.test_ds.manifest_filepath=test.json]
Manifest lines: ``{"text_graphemes": "hello", "text": "h ə l oʊ"}``.
(reference script: ``examples/tts/g2p/g2p_train_and_evaluate.py``)."""
from speech_b200.core.config import OmegaConf, hydra_runner, open_dict
from speech_b200.tts.g2p import CTCG2PModel, Seq2SeqG2PModel
from speech_b200.utils.exp_manager import exp_manager
from speech_b200.utils.launch import build_trainer
from speech_b200.utils.logging import logging

DEFAULTS = {"model_type": "ctc", "do_training": True, "do_testing": False, "pretrained_model": None,
            "model": {"phonemes": None, "graphemes": "abcdefghijklmnopqrstuvwxyz' -", "d_model": 256, "n_layers": 4, "n_heads": 4, "upsample": 2, "lowercase": True,
                      "train_ds": None, "validation_ds": None, "test_ds": None, "optim": {"name": "adamw", "lr": 1e-3, "sched": None}},
            "trainer": {"devices": 1, "accelerator": "auto", "max_epochs": 5, "max_steps": -1, "precision": 32, "log_every_n_steps": 50},
            "exp_manager": {"exp_dir": None, "name": "G2P", "create_tensorboard_logger": False}}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    if isinstance(cfg.model.phonemes, str):
        with open_dict(cfg):
            cfg.model.phonemes = [l.strip() for l in open(cfg.model.phonemes, encoding="utf-8") if l.strip()]
    cls = {"ctc": CTCG2PModel, "seq2seq": Seq2SeqG2PModel, "t5": Seq2SeqG2PModel}[cfg.model_type]
    trainer = build_trainer(cfg)
    exp_manager(trainer, cfg.get("exp_manager", None))
    model = cls.restore_from(cfg.pretrained_model) if cfg.pretrained_model else cls(cfg=cfg.model, trainer=trainer)
    model.set_trainer(trainer)
    if cfg.do_training:
        trainer.fit(model)
    if cfg.do_testing and cfg.model.test_ds is not None:
        model.setup_test_data(cfg.model.test_ds)
        per = [float(model.validation_step(b, i)["val_per"]) for i, b in enumerate(model._test_dl)]
        logging.info(f"test PER {100 * sum(per) / max(1, len(per)):.2f}%")
    return model


if __name__ == "__main__":
    main()

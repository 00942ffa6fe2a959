"""Fine-tune any ASR checkpoint on new data, optionally with a new tokenizer (the decoder / joint output layers are rebuilt, the
encoder is kept).

python examples/asr/speech_to_text_finetune.py init_from_nemo_model=base.nemo model.train_ds.manifest_filepath=train.json \
    model.validation_ds.manifest_filepath=dev.json [model.tokenizer.update_tokenizer=true model.tokenizer.dir=tok model.tokenizer.type=bpe] \
    trainer.max_steps=1000 model.optim.lr=1e-4
(reference script: ``examples/asr/speech_to_text_finetune.py``)."""
from speech_b200.core.config import OmegaConf, hydra_runner, open_dict
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.exp_manager import exp_manager
from speech_b200.utils.launch import build_trainer
from speech_b200.utils.logging import logging

DEFAULTS = {"init_from_nemo_model": None, "init_from_pretrained_model": None,
            "model": {"train_ds": None, "validation_ds": None, "test_ds": None, "tokenizer": {"update_tokenizer": False, "dir": None, "type": "bpe"},
                      "optim": {"name": "adamw", "lr": 1e-4, "weight_decay": 1e-3, "sched": None}, "spec_augment": None, "char_labels": {"update_labels": False, "labels": None}},
            "trainer": {"devices": 1, "accelerator": "auto", "max_steps": 100, "max_epochs": None, "precision": 32, "log_every_n_steps": 10},
            "exp_manager": {"exp_dir": None, "name": "finetune", "create_tensorboard_logger": False}}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    trainer = build_trainer(cfg)
    exp_manager(trainer, cfg.get("exp_manager", None))
    if cfg.init_from_nemo_model:
        model = ASRModel.restore_from(cfg.init_from_nemo_model, map_location="cpu")
    elif cfg.init_from_pretrained_model:
        model = ASRModel.from_pretrained(cfg.init_from_pretrained_model, map_location="cpu")
    else:
        raise ValueError("one of init_from_nemo_model / init_from_pretrained_model is required")
    model.set_trainer(trainer)
    tok = cfg.model.tokenizer
    if tok.update_tokenizer:
        if not hasattr(model, "change_vocabulary"):
            raise ValueError(f"{type(model).__name__} cannot change its vocabulary")
        logging.info(f"new tokenizer from {tok.dir} ({tok.type}); output layers are re-initialised")
        model.change_vocabulary(new_tokenizer_dir=tok.dir, new_tokenizer_type=tok.type)
    elif cfg.model.char_labels.update_labels:
        model.change_vocabulary(new_vocabulary=list(cfg.model.char_labels.labels))
    for split, setup in (("train_ds", model.setup_training_data), ("validation_ds", model.setup_multiple_validation_data), ("test_ds", model.setup_multiple_test_data)):
        if cfg.model.get(split) is not None:
            setup(cfg.model[split])
    if cfg.model.spec_augment is not None and hasattr(model, "spec_augmentation"):
        from speech_b200.modules.spec_augment import SpectrogramAugmentation

        model.spec_augmentation = SpectrogramAugmentation(**{k: v for k, v in dict(cfg.model.spec_augment).items() if k != "_target_"})
    with open_dict(model.cfg):
        model.cfg.optim = cfg.model.optim
    model.setup_optimization(cfg.model.optim)
    trainer.fit(model)
    return model


if __name__ == "__main__":
    main()

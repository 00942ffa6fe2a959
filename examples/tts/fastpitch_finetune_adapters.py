"""Adapt FastPitch to a new speaker with adapters: the base model is frozen, small residual adapters are added to every layer of the text encoder
and / or the mel decoder, and only they are trained; the result is a few-MB adapter file next to the unchanged base checkpoint.

python examples/tts/fastpitch_finetune_adapters.py +init_from_nemo_model=base.nemo model.train_ds.manifest_filepath=new_speaker.json \
    +model.adapter.modules='[encoder,decoder]' +model.adapter.dim=256 +model.adapter.name=spk1 +model.adapter.save_to=spk1_adapter.pt model.optim.lr=1e-3
Afterwards: ``model = FastPitchModel.restore_from('base.nemo'); model.load_adapters('spk1_adapter.pt')``.
(reference script: ``examples/tts/fastpitch_finetune_adapters.py``)."""
from speech_b200.core.config import OmegaConf, hydra_runner, open_dict, to_container
from speech_b200.tts.classic import FastPitchModel
from speech_b200.utils.exp_manager import exp_manager
from speech_b200.utils.launch import build_trainer
from speech_b200.utils.logging import logging


def add_adapters(model: FastPitchModel, adapter_cfg) -> int:
    """Adds one adapter per requested module, freezes the base, returns the number of trainable parameters."""
    a = dict(adapter_cfg or {})
    name, dim = a.get("name", "adapter"), int(a.get("dim", 256))
    d_model = model.encoder.d_model
    for module in a.get("modules", ["encoder", "decoder"]):
        model.add_adapter(f"{module}:{name}", {"in_features": d_model, "dim": dim, "activation": a.get("activation", "swish"), "norm_position": a.get("norm_position", "pre"),
                                               "dropout": float(a.get("dropout", 0.0))})
    return model.freeze_base_and_train_adapters()


@hydra_runner(config_path="conf", config_name="fastpitch")
def main(cfg):
    if not (cfg.get("init_from_nemo_model") or cfg.get("init_from_pretrained_model") or cfg.get("init_from_ptl_ckpt")):
        raise ValueError("adapter training needs a base model: init_from_nemo_model / init_from_pretrained_model / init_from_ptl_ckpt")
    adapter_cfg = to_container(cfg.model.get("adapter"), resolve=True) if cfg.model.get("adapter") is not None else {}
    with open_dict(cfg):
        cfg.model.pop("adapter", None)
        if cfg.model.get("optim") is not None and cfg.model.optim.get("sched") is not None:
            cfg.model.optim.sched = None
    trainer = build_trainer(cfg)
    exp_manager(trainer, cfg.get("exp_manager", None))
    model = FastPitchModel(cfg=OmegaConf.create(to_container(cfg.model, resolve=True)), trainer=trainer)
    model.maybe_init_from_pretrained_checkpoint(cfg)
    n = add_adapters(model, adapter_cfg)
    logging.info(f"training {n} adapter parameters of {sum(p.numel() for p in model.parameters())} in total")
    trainer.fit(model)
    out = adapter_cfg.get("save_to", "fastpitch_adapters.pt")
    model.save_adapters(out)
    logging.info(f"wrote {out}")
    return model


if __name__ == "__main__":
    main()

"""Fine-tune a pretrained ASR model with an adapter: the base model is frozen, one adapter is added and trained, and the adapter
alone is saved next to the full ``.nemo`` archive.

Usage: python examples/asr/asr_adapters/train_asr_adapter.py model.nemo_model=base.nemo model.train_ds.manifest_filepath=train.json \\
           model.adapter.adapter_name=encoder:domain model.adapter.adapter_type=linear model.adapter.d_model=512
(reference script: ``examples/asr/asr_adapters/train_asr_adapter.py``)."""
import os

from speech_b200.core.config import OmegaConf, hydra_runner, open_dict, to_container
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.exp_manager import exp_manager
from speech_b200.utils.launch import build_trainer
from speech_b200.utils.logging import logging


def load_base_model(cfg):
    if cfg.model.get("nemo_model"):
        return ASRModel.restore_from(cfg.model.nemo_model)
    if cfg.model.get("pretrained_model"):
        return ASRModel.from_pretrained(cfg.model.pretrained_model)
    raise ValueError("set model.nemo_model (a .nemo path) or model.pretrained_model (a registered name)")


def add_and_prepare_adapter(model, acfg):
    """Returns the full adapter name.  Any adapter already present in the base model is disabled, so that only the new one trains."""
    name = acfg.adapter_name
    if acfg.get("adapter_module_name") and ":" not in name:
        name = f"{acfg.adapter_module_name}:{name}"
    spec = to_container(acfg[acfg.adapter_type], resolve=True)
    if model.is_adapter_available():
        model.set_enabled_adapters(enabled=False)
    model.add_adapter(name, spec)
    model.set_enabled_adapters(name, True)
    n = model.freeze_base_and_train_adapters()
    logging.info(f"adapter '{name}' ({acfg.adapter_type}): {n / 1e6:.3f} M trainable of {sum(p.numel() for p in model.parameters()) / 1e6:.1f} M parameters")
    return name


@hydra_runner(config_path="../conf/asr_adapters", config_name="asr_adaptation")
def main(cfg):
    trainer = build_trainer(cfg)
    log_dir = exp_manager(trainer, cfg.get("exp_manager", None))
    model = load_base_model(cfg)
    model.set_trainer(trainer)
    with open_dict(model.cfg):
        model.cfg.log_prediction = cfg.model.get("log_prediction", False)
        model.cfg.optim = cfg.model.optim
    model.setup_training_data(cfg.model.train_ds)
    if cfg.model.validation_ds.get("manifest_filepath"):
        model.setup_multiple_validation_data(cfg.model.validation_ds)
    if hasattr(model, "spec_augmentation") and cfg.model.get("spec_augment") is not None:
        from speech_b200.core.instantiate import from_config_dict

        model.spec_augmentation = from_config_dict(cfg.model.spec_augment)
    name = add_and_prepare_adapter(model, cfg.model.adapter)
    trainer.fit(model)
    out_dir = str(log_dir) if log_dir else "."
    state_name = cfg.model.adapter.get("adapter_state_dict_name") or "adapters.pt"
    model.save_adapters(os.path.join(out_dir, state_name), name=name)
    model.save_to(os.path.join(out_dir, f"{cfg.name}.nemo"))
    logging.info(f"adapter weights: {os.path.join(out_dir, state_name)}")
    return model


if __name__ == "__main__":
    main()

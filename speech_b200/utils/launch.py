"""Shared body of the example training / evaluation scripts.

Every training example does the same five things as the reference's scripts (``examples/asr/asr_ctc/speech_to_text_ctc_bpe.py``
and friends): print the resolved config, build the ``Trainer`` from ``cfg.trainer``, set up the experiment manager from
``cfg.exp_manager``, build the model from ``cfg.model`` (optionally initialising from a checkpoint, ``cfg.init_from_*``) and
call ``fit`` (+ ``test`` when a test set is configured).
"""
from __future__ import annotations

from typing import Any, Optional, Type

from ..core.config import DictConfig, OmegaConf, to_container
from ..core.trainer import Trainer
from .exp_manager import exp_manager
from .logging import logging


def build_trainer(cfg: DictConfig) -> Trainer:
    kw = to_container(cfg.trainer, resolve=True) if cfg.get("trainer") is not None else {}
    st = kw.get("strategy")
    if isinstance(st, dict):
        # ``strategy: {dp_shard_size: 4, tp_size: 2, sequence_parallel: true}`` (optionally with a ``_target_``) builds the device-mesh
        # strategy object; plain strings ("auto", "ddp", "fsdp") pass through
        from ..parallel.strategy import ParallelStrategy

        st = {k: v for k, v in st.items() if k != "_target_"}
        kw["strategy"] = ParallelStrategy(**st)
    return Trainer(**kw)


def run_training(model_cls: Type, cfg: DictConfig, model_key: str = "model", test: bool = True) -> Any:
    logging.info(f"Config:\n{OmegaConf.to_yaml(cfg)}")
    trainer = build_trainer(cfg)
    exp_manager(trainer, cfg.get("exp_manager", None))
    # interpolations such as ${model.sample_rate} or ${trainer.max_steps} refer to the root config: resolve them while the
    # model block is still attached to it
    model_cfg = OmegaConf.create(to_container(cfg[model_key], resolve=True))
    model = model_cls(cfg=model_cfg, trainer=trainer)
    if hasattr(model, "maybe_init_from_pretrained_checkpoint"):
        model.maybe_init_from_pretrained_checkpoint(cfg)
    trainer.fit(model)
    if test and cfg[model_key].get("test_ds") is not None and (cfg[model_key].test_ds.get("manifest_filepath") is not None
                                                                or cfg[model_key].test_ds.get("synthetic") is not None):
        trainer.test(model)
    return model


def restore_model(model_cls: Type, path_or_name: str, map_location: Optional[str] = None):
    """``.nemo`` path → ``restore_from``; anything else → ``from_pretrained``."""
    if str(path_or_name).endswith(".nemo"):
        return model_cls.restore_from(path_or_name, map_location=map_location)
    return model_cls.from_pretrained(path_or_name, map_location=map_location)

"""Typed parameter records for optimizers and learning-rate schedulers, and the top-level config records of a training script
(``NemoConfig`` = name + model + trainer + experiment manager).  A record documents the accepted keys with their defaults, can be
partially filled (``get_scheduler_config('CosineAnnealingParams', min_lr=1e-5)()``) and converts to the plain dictionary the
optimizer / scheduler factories take.  Custom optimizers and schedulers register their record next to their class.
Reference: ``core/config/schedulers.py``, ``core/config/optimizers.py``, ``core/config/modelPT.py``, ``core/config/base_config.py``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, fields, is_dataclass
from functools import partial
from typing import Any, Dict, List, Optional, Tuple

MISSING = "???"


# ------------------------------------------------------------------------------------------------------------- schedulers
@dataclass
class SchedulerParams:
    last_epoch: int = -1


@dataclass
class SquareRootConstantSchedulerParams(SchedulerParams):
    constant_steps: Optional[float] = None
    constant_ratio: Optional[float] = None


@dataclass
class WarmupSchedulerParams(SchedulerParams):
    max_steps: int = 0
    warmup_steps: Optional[float] = None
    warmup_ratio: Optional[float] = None


@dataclass
class WarmupHoldSchedulerParams(WarmupSchedulerParams):
    hold_steps: Optional[float] = None
    hold_ratio: Optional[float] = None
    min_lr: float = 0.0


@dataclass
class WarmupAnnealingHoldSchedulerParams(WarmupSchedulerParams):
    constant_steps: Optional[float] = None
    constant_ratio: Optional[float] = None
    min_lr: float = 0.0


@dataclass
class SquareAnnealingParams(WarmupSchedulerParams):
    min_lr: float = 1e-5


@dataclass
class SquareRootAnnealingParams(WarmupSchedulerParams):
    min_lr: float = 0.0


@dataclass
class CosineAnnealingParams(WarmupAnnealingHoldSchedulerParams):
    min_lr: float = 0.0


@dataclass
class NoamAnnealingParams(WarmupSchedulerParams):
    min_lr: float = 0.0
    d_model: Optional[int] = None


@dataclass
class NoamHoldAnnealingParams(WarmupHoldSchedulerParams):
    decay_rate: float = 0.5


@dataclass
class WarmupAnnealingParams(WarmupSchedulerParams):
    warmup_ratio: Optional[float] = None


@dataclass
class InverseSquareRootAnnealingParams(WarmupSchedulerParams):
    pass


@dataclass
class PolynomialDecayAnnealingParams(WarmupSchedulerParams):
    power: float = 1.0
    cycle: bool = False
    min_lr: float = 0.0


@dataclass
class PolynomialHoldDecayAnnealingParams(WarmupSchedulerParams):
    hold_steps: Optional[float] = None
    hold_ratio: Optional[float] = None
    power: float = 1.0
    cycle: bool = False
    min_lr: float = 0.0


@dataclass
class StepLRParams(SchedulerParams):
    step_size: float = 0.1
    gamma: float = 0.1


@dataclass
class ExponentialLRParams(SchedulerParams):
    gamma: float = 0.9


@dataclass
class ReduceLROnPlateauParams:
    mode: str = "min"
    factor: float = 0.1
    patience: int = 10
    verbose: bool = False
    threshold: float = 1e-4
    threshold_mode: str = "rel"
    cooldown: int = 0
    min_lr: float = 0.0
    eps: float = 1e-8


@dataclass
class CyclicLRParams(SchedulerParams):
    base_lr: float = 0.001
    max_lr: float = 0.1
    step_size_up: int = 2000
    step_size_down: Optional[int] = None
    mode: str = "triangular"
    gamma: float = 1.0
    scale_mode: str = "cycle"
    cycle_momentum: bool = True
    base_momentum: float = 0.8
    max_momentum: float = 0.9


AVAILABLE_SCHEDULER_PARAMS: Dict[str, Any] = {
    "SchedulerParams": SchedulerParams,
    "WarmupPolicyParams": WarmupSchedulerParams,
    "WarmupHoldPolicyParams": WarmupHoldSchedulerParams,
    "WarmupAnnealingHoldSchedulerParams": WarmupAnnealingHoldSchedulerParams,
    "SquareAnnealingParams": SquareAnnealingParams,
    "SquareRootAnnealingParams": SquareRootAnnealingParams,
    "InverseSquareRootAnnealingParams": InverseSquareRootAnnealingParams,
    "SquareRootConstantSchedulerParams": SquareRootConstantSchedulerParams,
    "CosineAnnealingParams": CosineAnnealingParams,
    "NoamAnnealingParams": NoamAnnealingParams,
    "NoamHoldAnnealingParams": NoamHoldAnnealingParams,
    "WarmupAnnealingParams": WarmupAnnealingParams,
    "PolynomialDecayAnnealingParams": PolynomialDecayAnnealingParams,
    "PolynomialHoldDecayAnnealingParams": PolynomialHoldDecayAnnealingParams,
    "StepLRParams": StepLRParams,
    "ExponentialLRParams": ExponentialLRParams,
    "ReduceLROnPlateauParams": ReduceLROnPlateauParams,
    "CyclicLRParams": CyclicLRParams,
}


def register_scheduler_params(name: str, scheduler_params) -> None:
    if name in AVAILABLE_SCHEDULER_PARAMS:
        raise ValueError(f"Cannot register duplicate scheduler params ({name})")
    AVAILABLE_SCHEDULER_PARAMS[name] = scheduler_params


def get_scheduler_config(name: str, **kwargs):
    """The record class registered under ``name`` with ``kwargs`` pre-filled; call the result to get the record."""
    if name not in AVAILABLE_SCHEDULER_PARAMS:
        raise ValueError(f"Cannot resolve scheduler parameters '{name}'. Available: {sorted(AVAILABLE_SCHEDULER_PARAMS)}")
    return partial(AVAILABLE_SCHEDULER_PARAMS[name], **kwargs)


# -------------------------------------------------------------------------------------------------------------- optimizers
@dataclass
class OptimizerParams:
    lr: Optional[float] = MISSING


@dataclass
class SGDParams(OptimizerParams):
    momentum: float = 0
    dampening: float = 0
    weight_decay: float = 0
    nesterov: bool = False


@dataclass
class AdamParams(OptimizerParams):
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-08
    weight_decay: float = 0
    amsgrad: bool = False


@dataclass
class AdamWParams(OptimizerParams):
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-08
    weight_decay: float = 0
    amsgrad: bool = False


@dataclass
class AdadeltaParams(OptimizerParams):
    rho: float = 0.9
    eps: float = 1e-6
    weight_decay: float = 0


@dataclass
class AdamaxParams(OptimizerParams):
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0


@dataclass
class AdagradParams(OptimizerParams):
    lr_decay: float = 0
    weight_decay: float = 0
    initial_accumulator_value: float = 0
    eps: float = 1e-10


@dataclass
class RMSpropParams(OptimizerParams):
    alpha: float = 0.99
    eps: float = 1e-8
    weight_decay: float = 0
    momentum: float = 0
    centered: bool = False


@dataclass
class RpropParams(OptimizerParams):
    etas: Tuple[float, float] = (0.5, 1.2)
    step_sizes: Tuple[float, float] = (1e-6, 50)


@dataclass
class NovogradParams(OptimizerParams):
    lr: float = 1e-3
    betas: Tuple[float, float] = (0.95, 0.98)
    eps: float = 1e-8
    weight_decay: float = 0
    grad_averaging: bool = False
    amsgrad: bool = False
    luc: bool = False
    luc_trust: float = 1e-3
    luc_eps: float = 1e-8


@dataclass
class AdafactorParams(OptimizerParams):
    beta1: Optional[float] = None
    eps: Tuple[float, float] = (1e-30, 1e-3)
    clip_threshold: float = 1.0
    decay_rate: float = 0.8
    weight_decay: float = 0
    scale_parameter: bool = True
    relative_step: bool = False
    warmup_init: bool = False


@dataclass
class AdanParams(OptimizerParams):
    betas: Tuple[float, float, float] = (0.98, 0.92, 0.99)
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 0.0
    no_prox: bool = False


AVAILABLE_OPTIMIZER_PARAMS: Dict[str, Any] = {
    "optim_params": OptimizerParams,
    "adam_params": AdamParams,
    "fused_adamw_params": AdamWParams,
    "novograd_params": NovogradParams,
    "sgd_params": SGDParams,
    "adadelta_params": AdadeltaParams,
    "adamax_params": AdamaxParams,
    "adagrad_params": AdagradParams,
    "adamw_params": AdamWParams,
    "rmsprop_params": RMSpropParams,
    "rprop_params": RpropParams,
    "adafactor_params": AdafactorParams,
    "adan_params": AdanParams,
}


def register_optimizer_params(name: str, optimizer_params) -> None:
    if name in AVAILABLE_OPTIMIZER_PARAMS:
        raise ValueError(f"Cannot register duplicate optimizer params ({name})")
    AVAILABLE_OPTIMIZER_PARAMS[name] = optimizer_params


def get_optimizer_config(name: Optional[str], **kwargs):
    """``name`` may be a registry key (``'adam_params'``), an optimizer name (``'adam'`` → ``'adam_params'``) or ``None`` (the kwargs are
    returned as they are)."""
    if name is None:
        return kwargs
    key = name if name in AVAILABLE_OPTIMIZER_PARAMS else f"{name}_params"
    if key not in AVAILABLE_OPTIMIZER_PARAMS:
        raise ValueError(f"Cannot resolve optimizer parameters '{name}'. Available: {sorted(AVAILABLE_OPTIMIZER_PARAMS)}")
    return partial(AVAILABLE_OPTIMIZER_PARAMS[key], **kwargs)


def params_to_dict(params) -> Dict[str, Any]:
    """A record (or a partial of one) as the keyword dictionary of its optimizer / scheduler; unset mandatory values are left out."""
    if isinstance(params, partial):
        params = params()
    d = asdict(params) if is_dataclass(params) else dict(params)
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in d.items() if v != MISSING}


# ------------------------------------------------------------------------------------------------------- script-level configs
@dataclass
class Config:
    name: Optional[str] = None


@dataclass
class DatasetConfig:
    batch_size: int = 32
    drop_last: bool = False
    shuffle: bool = False
    num_workers: Optional[int] = 0
    pin_memory: bool = True


@dataclass
class SchedConfig:
    name: str = MISSING
    min_lr: float = 0.0
    last_epoch: int = -1


@dataclass
class OptimConfig:
    name: str = MISSING
    sched: Optional[SchedConfig] = None


@dataclass
class ModelConfig:
    train_ds: Optional[DatasetConfig] = None
    validation_ds: Optional[DatasetConfig] = None
    test_ds: Optional[DatasetConfig] = None
    optim: Optional[OptimConfig] = None


@dataclass
class TrainerConfig:
    devices: Any = 1
    num_nodes: int = 1
    accelerator: Optional[str] = "gpu"
    strategy: Any = "ddp"
    precision: Any = "bf16"
    max_epochs: int = 1000
    max_steps: int = -1
    accumulate_grad_batches: int = 1
    gradient_clip_val: float = 0.0
    log_every_n_steps: int = 50
    val_check_interval: Any = 1.0
    check_val_every_n_epoch: int = 1
    num_sanity_val_steps: int = 0
    enable_checkpointing: bool = False
    logger: Any = False
    limit_train_batches: Any = 1.0
    limit_val_batches: Any = 1.0
    sync_batchnorm: bool = False
    benchmark: bool = False


@dataclass
class HydraConfig:
    run: Dict[str, Any] = field(default_factory=lambda: {"dir": "."})
    job_logging: Dict[str, Any] = field(default_factory=lambda: {"root": {"handlers": None}})


@dataclass
class NemoConfig:
    name: str = MISSING
    model: Any = MISSING
    trainer: TrainerConfig = field(default_factory=lambda: TrainerConfig(strategy="ddp", enable_checkpointing=False, logger=False, log_every_n_steps=1))
    exp_manager: Optional[Any] = None
    hydra: HydraConfig = field(default_factory=HydraConfig)


class ModelConfigBuilder:
    """Fills a ``ModelConfig`` step by step (``set_train_ds`` / ``set_validation_ds`` / ``set_test_ds`` / ``set_optim``); ``build()`` runs the
    subclass's ``_finalize_cfg`` (which resolves the values that depend on each other) and returns the finished config."""

    def __init__(self, model_cfg: ModelConfig):
        self.model_cfg = model_cfg
        self.train_ds_cfg = self.validation_ds_cfg = self.test_ds_cfg = self.optim_cfg = None

    def set_train_ds(self, cfg: Optional[DatasetConfig] = None):
        self.model_cfg.train_ds = cfg

    def set_validation_ds(self, cfg: Optional[DatasetConfig] = None):
        self.model_cfg.validation_ds = cfg

    def set_test_ds(self, cfg: Optional[DatasetConfig] = None):
        self.model_cfg.test_ds = cfg

    def set_optim(self, cfg, sched_cfg: Optional[SchedConfig] = None):
        """``cfg``: an optimizer record; its class name without ``Params`` (lower-cased) becomes the optimizer name."""
        @dataclass
        class WrappedOptimConfig(OptimConfig, cfg.__class__):
            pass

        name = cfg.__class__.__name__.replace("Params", "").lower()
        kw = {f.name: getattr(cfg, f.name) for f in fields(cfg)}
        self.model_cfg.optim = WrappedOptimConfig(**{**kw, "name": name, "sched": sched_cfg})

    def _finalize_cfg(self):
        raise NotImplementedError

    def build(self) -> ModelConfig:
        self._finalize_cfg()
        return self.model_cfg


def to_dictconfig(cfg):
    """A (nested) record as the framework's dictionary config."""
    from .config import OmegaConf

    def conv(v):
        if is_dataclass(v) and not isinstance(v, type):
            return {f.name: conv(getattr(v, f.name)) for f in fields(v)}
        if isinstance(v, dict):
            return {k: conv(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [conv(x) for x in v]
        return v

    return OmegaConf.create(conv(cfg))

"""Optimizers and learning-rate schedules."""
from .lr_scheduler import AVAILABLE_SCHEDULERS, prepare_lr_scheduler, register_scheduler  # noqa: F401
from .optimizers import AVAILABLE_OPTIMIZERS, get_optimizer, parse_optimizer_args, register_optimizer  # noqa: F401

"""Learning-rate schedules: warm-up / hold / anneal families.

Closed forms follow the reference (``nemo/core/optim/lr_scheduler.py:39-1067``).  The Noam
schedule is ``lr = base * d_model^-0.5 * min(step^-0.5, step * warmup^-1.5)`` (``:566-575``).
Every scheduler is a ``torch.optim.lr_scheduler.LRScheduler`` stepped once per optimizer
step.  ``prepare_lr_scheduler`` builds ``{"scheduler", "interval", ...}`` from an
``optim.sched`` config block and derives ``max_steps`` from epochs and dataloader length
when it is not given (``:759-1040``).
"""
from __future__ import annotations

import copy
import math
import warnings
from typing import Any, Dict, Optional

from torch.optim import lr_scheduler as _torch_sched
from torch.optim.lr_scheduler import LRScheduler

from ..config import DictConfig, to_container


class WarmupPolicy(LRScheduler):
    """Linear warm-up from ~0 to the base LR, then ``_get_lr(step)`` of the subclass."""

    def __init__(self, optimizer, *, warmup_steps=None, warmup_ratio=None, max_steps=None, min_lr=0.0,
                 last_epoch=-1):
        if warmup_steps is not None and warmup_ratio is not None:
            raise ValueError("Either use particular number of step or ratio")
        if warmup_ratio is not None and max_steps is None:
            raise ValueError("If there is a ratio, there should be a total steps")
        self.max_steps = max_steps
        if warmup_steps is not None:
            self.warmup_steps = warmup_steps
        elif warmup_ratio is not None:
            self.warmup_steps = int(warmup_ratio * max_steps)
        else:
            self.warmup_steps = 0
        self.min_lr = min_lr
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        step = self.last_epoch
        if step <= self.warmup_steps and self.warmup_steps > 0:
            return self._get_warmup_lr(step)
        if self.max_steps is not None and step > self.max_steps:
            return [self.min_lr for _ in self.base_lrs]
        return self._get_lr(step)

    def _get_warmup_lr(self, step):
        lr_val = (step + 1) / (self.warmup_steps + 1)
        return [initial_lr * lr_val for initial_lr in self.base_lrs]

    def _get_lr(self, step):
        return self.base_lrs


class SquareRootConstantPolicy(LRScheduler):
    def __init__(self, optimizer, *, constant_steps=None, constant_ratio=None, max_steps=None, min_lr=0.0,
                 last_epoch=-1):
        self.max_steps = max_steps
        if constant_steps is not None:
            self.constant_steps = constant_steps
        elif constant_ratio is not None:
            self.constant_steps = int(constant_ratio * max_steps)
        else:
            self.constant_steps = 0
        self.constant_lr = 1 / (self.constant_steps ** 0.5) if self.constant_steps else 1.0
        self.min_lr = min_lr
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        step = self.last_epoch
        if step <= self.constant_steps:
            return [self.constant_lr for _ in self.base_lrs]
        if self.max_steps is not None and step > self.max_steps:
            return [self.min_lr for _ in self.base_lrs]
        return [1 / math.sqrt(step) for _ in self.base_lrs]


class WarmupHoldPolicy(WarmupPolicy):
    def __init__(self, optimizer, *, warmup_steps=None, warmup_ratio=None, hold_steps=None, hold_ratio=None,
                 max_steps=None, min_lr=0.0, last_epoch=-1):
        if hold_steps is not None and hold_ratio is not None:
            raise ValueError("Either use particular number of step or ratio")
        if hold_ratio is not None and max_steps is None:
            raise ValueError("If there is a ratio, there should be a total steps")
        self.min_lr = min_lr
        self._last_warmup_lr = 0.0
        self.max_steps = max_steps
        ws = warmup_steps if warmup_steps is not None else (int(warmup_ratio * max_steps) if warmup_ratio else 0)
        if hold_steps is not None:
            self.hold_steps = hold_steps + ws
        elif hold_ratio is not None:
            self.hold_steps = int(hold_ratio * max_steps) + ws
        else:
            self.hold_steps = 0
        super().__init__(optimizer, warmup_steps=warmup_steps, warmup_ratio=warmup_ratio, max_steps=max_steps,
                         last_epoch=last_epoch, min_lr=min_lr)

    def get_lr(self):
        step = self.last_epoch
        if step <= self.warmup_steps and self.warmup_steps > 0:
            return self._get_warmup_lr(step)
        if self.warmup_steps <= step < self.hold_steps:
            return self.base_lrs
        if self.max_steps is not None and step > self.max_steps:
            return [self.min_lr for _ in self.base_lrs]
        return self._get_lr(step)


class WarmupAnnealHoldPolicy(LRScheduler):
    """Warm-up, anneal until ``max_steps - constant_steps``, then hold ``min_lr``."""

    def __init__(self, optimizer, *, warmup_steps=None, warmup_ratio=None, constant_steps=None, constant_ratio=None,
                 max_steps=None, min_lr=0.0, last_epoch=-1):
        if max_steps is None:
            raise ValueError("max_steps is required")
        self.max_steps = max_steps
        self.warmup_steps = warmup_steps if warmup_steps is not None else (
            int(warmup_ratio * max_steps) if warmup_ratio is not None else 0)
        self.constant_steps = constant_steps if constant_steps is not None else (
            int(constant_ratio * max_steps) if constant_ratio is not None else 0)
        self.decay_steps = max_steps - (self.constant_steps + self.warmup_steps)
        self.min_lr = min_lr
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        step = self.last_epoch
        if self.warmup_steps > 0 and step <= self.warmup_steps:
            return [b * (step + 1) / (self.warmup_steps + 1) for b in self.base_lrs]
        if self.constant_steps > 0 and (self.warmup_steps + self.decay_steps) < step <= self.max_steps:
            return [self.min_lr for _ in self.base_lrs]
        if step > self.max_steps:
            return [self.min_lr for _ in self.base_lrs]
        return self._get_lr(step)

    def _get_lr(self, step):
        return self.base_lrs


def _squareroot_annealing(initial_lr, step, max_steps, min_lr):
    mult = ((max_steps - step) / max_steps) ** 0.5
    return max(initial_lr * mult, min_lr)


def _square_annealing(initial_lr, step, max_steps, min_lr):
    mult = ((max_steps - step) / max_steps) ** 2
    return max(initial_lr * mult, min_lr)


def _cosine_annealing(initial_lr, step, max_steps, min_lr):
    mult = 0.5 * (1 + math.cos(math.pi * step / max_steps))
    return (initial_lr - min_lr) * mult + min_lr


def _linear_warmup_with_cosine_annealing(max_lr, warmup_steps, step, decay_steps, min_lr):
    assert max_lr > min_lr
    if warmup_steps > 0 and step <= warmup_steps:
        return max_lr * float(step) / float(warmup_steps)
    if step > warmup_steps + decay_steps:
        return min_lr
    num = step - warmup_steps
    ratio = float(num) / float(decay_steps)
    coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
    return min_lr + coeff * (max_lr - min_lr)


def _poly_decay(initial_lr, step, decay_steps, power, min_lr, cycle):
    if cycle:
        mult = 1.0 if step == 0 else math.ceil(step / decay_steps)
        decay_steps *= mult
    else:
        step = min(step, decay_steps)
    p = step / decay_steps
    lr = (initial_lr - min_lr) * math.pow(1.0 - p, power)
    return lr + min_lr


def _noam_hold_annealing(initial_lr, step, warmup_steps, hold_steps, decay_rate, min_lr):
    T_warmup_decay = max(1, warmup_steps ** decay_rate)
    T_hold_decay = max(1, (step - hold_steps) ** decay_rate)
    lr = (initial_lr * T_warmup_decay) / T_hold_decay
    return max(lr, min_lr)


class SquareAnnealing(WarmupPolicy):
    def __init__(self, optimizer, *, max_steps, min_lr=1e-5, last_epoch=-1, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        return [_square_annealing(b, step - self.warmup_steps, self.max_steps - self.warmup_steps, self.min_lr)
                for b in self.base_lrs]


class SquareRootAnnealing(WarmupPolicy):
    def __init__(self, optimizer, *, max_steps, min_lr=0, last_epoch=-1, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        return [_squareroot_annealing(b, step, self.max_steps, self.min_lr) for b in self.base_lrs]


class CosineAnnealing(WarmupAnnealHoldPolicy):
    def __init__(self, optimizer, *, max_steps, min_lr=0, last_epoch=-1, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        for b in self.base_lrs:
            if b < self.min_lr:
                raise ValueError(f"{self} received an initial learning rate that was lower than the minimum learning rate.")
        if self.constant_steps is None or self.constant_steps == 0:
            return [_cosine_annealing(b, step - self.warmup_steps, self.max_steps - self.warmup_steps, self.min_lr)
                    for b in self.base_lrs]
        return self._get_linear_warmup_with_cosine_annealing_lr(step)

    def _get_warmup_lr(self, step):
        if self.constant_steps is None or self.constant_steps == 0:
            return super()._get_warmup_lr(step)
        return self._get_linear_warmup_with_cosine_annealing_lr(step)

    def _get_linear_warmup_with_cosine_annealing_lr(self, step):
        return [_linear_warmup_with_cosine_annealing(self.base_lrs[0], self.warmup_steps, step, self.decay_steps,
                                                     self.min_lr) for _ in self.base_lrs]


class NoamAnnealing(LRScheduler):
    def __init__(self, optimizer, *, d_model, warmup_steps=None, warmup_ratio=None, max_steps=None, min_lr=0.0,
                 last_epoch=-1):
        self._normalize = d_model ** (-0.5)
        if warmup_steps is not None and warmup_ratio is not None:
            raise ValueError("Either use particular number of step or ratio")
        if warmup_ratio is not None and max_steps is None:
            raise ValueError("If there is a ratio, there should be a total steps")
        self.max_steps = max_steps
        if warmup_steps is not None:
            self.warmup_steps = warmup_steps
        elif warmup_ratio is not None:
            self.warmup_steps = int(warmup_ratio * max_steps)
        else:
            self.warmup_steps = 0
        self.min_lr = min_lr
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        step = max(1, self.last_epoch)
        for b in self.base_lrs:
            if b < self.min_lr:
                raise ValueError(f"{self} received an initial learning rate that was lower than the minimum learning rate.")
        return [self._noam_annealing(initial_lr=b, step=step) for b in self.base_lrs]

    def _noam_annealing(self, initial_lr, step):
        if self.warmup_steps > 0:
            mult = self._normalize * min(step ** (-0.5), step * (self.warmup_steps ** (-1.5)))
        else:
            mult = self._normalize * step ** (-0.5)
        out_lr = initial_lr * mult
        if step > self.warmup_steps:
            out_lr = max(out_lr, self.min_lr)
        return out_lr


class NoamHoldAnnealing(WarmupHoldPolicy):
    def __init__(self, optimizer, *, max_steps, decay_rate=0.5, min_lr=0.0, last_epoch=-1, **kwargs):
        self.decay_rate = decay_rate
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        if self.warmup_steps is None or self.warmup_steps == 0:
            raise ValueError("Noam scheduler cannot be used without warmup steps")
        hold = self.hold_steps - self.warmup_steps if self.hold_steps > 0 else 0
        return [_noam_hold_annealing(b, step=step, warmup_steps=self.warmup_steps, hold_steps=hold,
                                     decay_rate=self.decay_rate, min_lr=self.min_lr) for b in self.base_lrs]

    def set_min_lr(self, min_lr):
        self.min_lr = min_lr


class WarmupAnnealing(WarmupPolicy):
    def __init__(self, optimizer, *, max_steps, last_epoch=-1, min_lr=0.0, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        delta = self.max_steps - self.warmup_steps
        mult = max((self.max_steps - step) / max(delta, 1), 0.0)
        return [max(b * mult, self.min_lr) for b in self.base_lrs]


class InverseSquareRootAnnealing(WarmupPolicy):
    def __init__(self, optimizer, *, max_steps, last_epoch=-1, min_lr=0.0, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        denom = ((step + 1) / (self.warmup_steps + 1)) ** 0.5
        return [max(b / denom, self.min_lr) for b in self.base_lrs]


class T5InverseSquareRootAnnealing(SquareRootConstantPolicy):
    def __init__(self, optimizer, *, max_steps, last_epoch=-1, min_lr=0.0, **kwargs):
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)


class PolynomialDecayAnnealing(WarmupPolicy):
    def __init__(self, optimizer, *, max_steps, min_lr=0.0, power=1.0, cycle=False, last_epoch=-1, **kwargs):
        self.power, self.cycle = power, cycle
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        return [_poly_decay(b, step=step - self.warmup_steps, decay_steps=self.max_steps - self.warmup_steps,
                            power=self.power, min_lr=self.min_lr, cycle=self.cycle) for b in self.base_lrs]


class PolynomialHoldDecayAnnealing(WarmupHoldPolicy):
    def __init__(self, optimizer, *, max_steps, min_lr=0.0, power=1.0, cycle=False, last_epoch=-1, **kwargs):
        self.power, self.cycle = power, cycle
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kwargs)

    def _get_lr(self, step):
        return [_poly_decay(b, step=step - self.hold_steps, decay_steps=self.max_steps - max(self.warmup_steps, self.hold_steps),
                            power=self.power, min_lr=self.min_lr, cycle=self.cycle) for b in self.base_lrs]


class WarmupHoldAnnealOneMinusSquareRoot(WarmupPolicy):
    """Warm-up, hold, then ``lr * (1 - sqrt(progress))`` over the last ``decay_steps``."""

    def __init__(self, optimizer, *, max_steps, decay_steps=None, decay_ratio=None, min_lr=0.0, last_epoch=-1, **kw):
        self.decay_steps = decay_steps if decay_steps is not None else int((decay_ratio or 0.2) * max_steps)
        super().__init__(optimizer=optimizer, max_steps=max_steps, last_epoch=last_epoch, min_lr=min_lr, **kw)

    def _get_lr(self, step):
        start = self.max_steps - self.decay_steps
        if step < start:
            return self.base_lrs
        prog = min(1.0, (step - start) / max(1, self.decay_steps))
        return [max(self.min_lr, b * (1.0 - math.sqrt(prog))) for b in self.base_lrs]


class WarmupHoldAnnealLinear(WarmupHoldAnnealOneMinusSquareRoot):
    def _get_lr(self, step):
        start = self.max_steps - self.decay_steps
        if step < start:
            return self.base_lrs
        prog = min(1.0, (step - start) / max(1, self.decay_steps))
        return [max(self.min_lr, b * (1.0 - prog)) for b in self.base_lrs]


AVAILABLE_SCHEDULERS: Dict[str, Any] = {
    "WarmupPolicy": WarmupPolicy,
    "WarmupHoldPolicy": WarmupHoldPolicy,
    "SquareAnnealing": SquareAnnealing,
    "CosineAnnealing": CosineAnnealing,
    "NoamAnnealing": NoamAnnealing,
    "NoamHoldAnnealing": NoamHoldAnnealing,
    "WarmupHoldAnnealOneMinusSquareRoot": WarmupHoldAnnealOneMinusSquareRoot,
    "WarmupHoldAnnealLinear": WarmupHoldAnnealLinear,
    "WarmupAnnealing": WarmupAnnealing,
    "InverseSquareRootAnnealing": InverseSquareRootAnnealing,
    "T5InverseSquareRootAnnealing": T5InverseSquareRootAnnealing,
    "SquareRootAnnealing": SquareRootAnnealing,
    "PolynomialDecayAnnealing": PolynomialDecayAnnealing,
    "PolynomialHoldDecayAnnealing": PolynomialHoldDecayAnnealing,
    "StepLR": _torch_sched.StepLR,
    "ExponentialLR": _torch_sched.ExponentialLR,
    "ReduceLROnPlateau": _torch_sched.ReduceLROnPlateau,
    "CyclicLR": _torch_sched.CyclicLR,
}


def register_scheduler(name: str, scheduler, scheduler_params=None):
    if name in AVAILABLE_SCHEDULERS:
        raise ValueError(f"Cannot register duplicate scheduler ({name})")
    AVAILABLE_SCHEDULERS[name] = scheduler
    if scheduler_params is not None:                               # the typed record of its arguments, looked up as "<class name>Params"
        from ..config_schemas import register_scheduler_params

        register_scheduler_params(f"{scheduler.__name__}Params", scheduler_params)


def get_scheduler(name: str, **kwargs):
    if name not in AVAILABLE_SCHEDULERS:
        raise ValueError(f"Cannot resolve scheduler '{name}'. Available: {list(AVAILABLE_SCHEDULERS)}")
    import functools

    return functools.partial(AVAILABLE_SCHEDULERS[name], **kwargs)


def compute_max_steps(max_epochs, accumulate_grad_batches, limit_train_batches, num_workers, num_samples,
                      batch_size, drop_last):
    _round = math.floor if drop_last else math.ceil
    sampler_num_samples = math.ceil(num_samples / max(1, num_workers))
    if drop_last and num_workers > 1:
        warnings.warn("Please note that drop_last is broken in pytorch 1.6.0. We will fix when pytorch 1.7.0 is released")
    steps_per_epoch = _round(sampler_num_samples / batch_size)
    if isinstance(limit_train_batches, int) or limit_train_batches == 0.0:
        steps_per_epoch = min(steps_per_epoch, int(limit_train_batches))
    elif steps_per_epoch != float("inf"):
        steps_per_epoch = int(steps_per_epoch * limit_train_batches)
    return math.ceil(steps_per_epoch / accumulate_grad_batches) * max_epochs


def prepare_lr_scheduler(optimizer, scheduler_config, train_dataloader=None) -> Optional[Dict[str, Any]]:
    """``optim.sched`` block -> ``{"scheduler", "interval", "frequency", "monitor", ...}`` or ``None``."""
    if scheduler_config is None:
        return None
    cfg = to_container(scheduler_config, resolve=True) if isinstance(scheduler_config, DictConfig) else copy.deepcopy(
        dict(scheduler_config))
    if "sched" in cfg:
        inner = cfg["sched"]
        for extra in ("max_steps", "t_max_epochs", "t_accumulate_grad_batches", "t_limit_train_batches", "t_num_workers"):
            if extra in cfg and extra not in inner:
                inner[extra] = cfg[extra]
        cfg = inner
    if cfg is None:
        return None
    name = cfg.pop("name", None)
    if name is None:
        return None
    interval = cfg.pop("interval", "step")
    monitor = cfg.pop("monitor", "loss")
    reduce_on_plateau = cfg.pop("reduce_on_plateau", name == "ReduceLROnPlateau")
    frequency = cfg.pop("frequency", 1)
    args = cfg.pop("args", None)
    params = cfg.pop("params", None)
    if params:
        cfg.update(params)
    cfg.pop("_target_", None)
    t = {k: cfg.pop(k, None) for k in ("t_max_epochs", "t_accumulate_grad_batches", "t_limit_train_batches",
                                        "t_num_workers")}
    sched_cls = AVAILABLE_SCHEDULERS.get(name)
    if sched_cls is None:
        raise ValueError(f"Scheduler '{name}' is not registered")
    import inspect

    wants_max_steps = "max_steps" in inspect.signature(sched_cls.__init__).parameters
    max_steps = cfg.get("max_steps", None)
    if wants_max_steps and (max_steps is None or max_steps < 0):
        if t["t_max_epochs"] is None or train_dataloader is None:
            if name in ("NoamAnnealing", "WarmupPolicy", "WarmupHoldPolicy") and cfg.get("warmup_ratio") is None:
                cfg["max_steps"] = None
            else:
                raise ValueError("Scheduler needs `max_steps` (or max_epochs plus a train dataloader) to be set")
        else:
            try:
                n = len(train_dataloader.dataset)
            except Exception:
                n = len(train_dataloader) * (getattr(train_dataloader, "batch_size", 1) or 1)
            bs = getattr(train_dataloader, "batch_size", None) or 1
            cfg["max_steps"] = compute_max_steps(
                t["t_max_epochs"], t["t_accumulate_grad_batches"] or 1, t["t_limit_train_batches"] or 1.0,
                t["t_num_workers"] or 1, n, bs, getattr(train_dataloader, "drop_last", False))
    elif not wants_max_steps:
        cfg.pop("max_steps", None)
    sched = sched_cls(optimizer, **cfg)
    return {"scheduler": sched, "interval": interval, "frequency": frequency, "monitor": monitor,
            "reduce_on_plateau": reduce_on_plateau}

"""Optimizer registry and the extra optimizers the reference ships.

Registry names follow ``nemo/core/optim/optimizers.py:33-75``: ``sgd, adam, adamw, adadelta,
adamax, adagrad, rmsprop, rprop, novograd, adafactor, adan``; ``fused_adam`` / ``fused_adamw``
resolve to this framework's flat-arena AdamW (``speech_b200.core.optim.fused_adamw``) which on
a GPU runs as one hand-written kernel over all parameters.
"""
from __future__ import annotations

import copy
import math
from functools import partial
from typing import Any, Dict, Optional

import torch
from torch import optim
from torch.optim.optimizer import Optimizer

from ..config import DictConfig, to_container


class Novograd(Optimizer):
    """NovoGrad: layer-wise second moments (reference: ``nemo/core/optim/novograd.py``)."""

    def __init__(self, params, lr=1e-3, betas=(0.95, 0.98), eps=1e-8, weight_decay=0, grad_averaging=False,
                 amsgrad=False, luc=False, luc_trust=1e-3, luc_eps=1e-8):
        if lr < 0.0 or eps < 0.0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("Invalid Novograd hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      grad_averaging=grad_averaging, amsgrad=amsgrad))
        self.luc, self.luc_trust, self.luc_eps = luc, luc_trust, luc_eps

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                if grad.is_sparse:
                    raise RuntimeError("Sparse gradients are not supported.")
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p)
                    state["exp_avg_sq"] = torch.zeros([], device=p.device)
                    if group["amsgrad"]:
                        state["max_exp_avg_sq"] = torch.zeros([], device=p.device)
                exp_avg, exp_avg_sq = state["exp_avg"], state["exp_avg_sq"]
                beta1, beta2 = group["betas"]
                state["step"] += 1
                norm = grad.float().norm().pow(2)
                if exp_avg_sq.item() == 0 and state["step"] == 1:
                    exp_avg_sq.copy_(norm)
                else:
                    exp_avg_sq.mul_(beta2).add_(norm, alpha=1.0 - beta2)
                if group["amsgrad"]:
                    torch.max(state["max_exp_avg_sq"], exp_avg_sq, out=state["max_exp_avg_sq"])
                    denom = state["max_exp_avg_sq"].sqrt().add_(group["eps"])
                else:
                    denom = exp_avg_sq.sqrt().add_(group["eps"])
                g = grad / denom
                if group["weight_decay"] != 0:
                    g = g.add(p, alpha=group["weight_decay"])
                if group["grad_averaging"]:
                    g = g * (1 - beta1)
                exp_avg.mul_(beta1).add_(g)
                if self.luc:
                    data_norm, grad_norm = p.norm(), exp_avg.norm()
                    luc_factor = self.luc_trust * data_norm / (grad_norm + self.luc_eps)
                    p.add_(exp_avg, alpha=-float(min(luc_factor, group["lr"])))
                else:
                    p.add_(exp_avg, alpha=-group["lr"])
        return loss


class Adafactor(Optimizer):
    """Adafactor with factored second moments (reference: ``nemo/core/optim/adafactor.py``)."""

    def __init__(self, params, lr=None, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, beta1=None,
                 weight_decay=0.0, scale_parameter=True, relative_step=False, warmup_init=False, min_step=1e-2):
        if lr is not None and relative_step:
            raise ValueError("Cannot combine manual lr and relative_step options")
        if warmup_init and not relative_step:
            raise ValueError("warmup_init requires relative_step=True")
        self.min_step = min_step
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate,
                                      beta1=beta1, weight_decay=weight_decay, scale_parameter=scale_parameter,
                                      relative_step=relative_step, warmup_init=warmup_init, min_step=min_step))

    @staticmethod
    def _rms(t):
        return t.norm(2) / (t.numel() ** 0.5)

    def _get_lr(self, group, state):
        rel = group["lr"]
        if group["relative_step"]:
            min_step = 1e-6 * state["step"] if group["warmup_init"] else self.min_step
            rel = min(min_step, 1.0 / math.sqrt(state["step"]))
        scale = 1.0
        if group["scale_parameter"]:
            scale = max(group["eps"][1], state["RMS"])
        return scale * rel

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                state = self.state[p]
                factored = grad.dim() >= 2
                use_m = group["beta1"] is not None
                if len(state) == 0:
                    state["step"] = 0
                    if use_m:
                        state["exp_avg"] = torch.zeros_like(grad)
                    if factored:
                        state["exp_avg_sq_row"] = torch.zeros(grad.shape[:-1], device=grad.device)
                        state["exp_avg_sq_col"] = torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=grad.device)
                    else:
                        state["exp_avg_sq"] = torch.zeros_like(grad)
                    state["RMS"] = 0
                pf = p.float()
                state["step"] += 1
                state["RMS"] = float(self._rms(pf))
                lr = self._get_lr(group, state)
                beta2t = 1.0 - math.pow(state["step"], group["decay_rate"])
                update = grad ** 2 + group["eps"][0]
                if factored:
                    r, c = state["exp_avg_sq_row"], state["exp_avg_sq_col"]
                    r.mul_(beta2t).add_(update.mean(dim=-1), alpha=1.0 - beta2t)
                    c.mul_(beta2t).add_(update.mean(dim=-2), alpha=1.0 - beta2t)
                    r_factor = (r / r.mean(dim=-1, keepdim=True)).rsqrt_().unsqueeze(-1)
                    c_factor = c.unsqueeze(-2).rsqrt()
                    update = r_factor * c_factor * grad
                else:
                    v = state["exp_avg_sq"]
                    v.mul_(beta2t).add_(update, alpha=1.0 - beta2t)
                    update = v.rsqrt() * grad
                update.div_((self._rms(update) / group["clip_threshold"]).clamp_(min=1.0))
                update.mul_(lr)
                if use_m:
                    m = state["exp_avg"]
                    m.mul_(group["beta1"]).add_(update, alpha=1 - group["beta1"])
                    update = m
                if group["weight_decay"] != 0:
                    pf.add_(pf, alpha=-group["weight_decay"] * lr)
                pf.add_(-update)
                p.copy_(pf)
        return loss


class Adan(Optimizer):
    """Adan: adaptive Nesterov momentum (reference: ``nemo/core/optim/adan.py``)."""

    def __init__(self, params, lr=1e-3, betas=(0.98, 0.92, 0.99), eps=1e-8, weight_decay=0.0, max_grad_norm=0.0,
                 no_prox=False, foreach=True):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      max_grad_norm=max_grad_norm, no_prox=no_prox))

    @torch.no_grad()
    def restart_opt(self):
        for group in self.param_groups:
            group["step"] = 0
            for p in group["params"]:
                if p.requires_grad:
                    st = self.state[p]
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    st["exp_avg_diff"] = torch.zeros_like(p)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        clip = 1.0
        mg = self.defaults["max_grad_norm"]
        if mg > 0:
            sq = sum(float(p.grad.float().pow(2).sum()) for g in self.param_groups for p in g["params"]
                     if p.grad is not None)
            clip = min(1.0, mg / (math.sqrt(sq) + self.defaults["eps"]))
        for group in self.param_groups:
            beta1, beta2, beta3 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            bc1 = 1.0 - beta1 ** group["step"]
            bc2 = 1.0 - beta2 ** group["step"]
            bc3 = 1.0 - beta3 ** group["step"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    st["exp_avg_diff"] = torch.zeros_like(p)
                grad = p.grad * clip
                if "neg_pre_grad" not in st or group["step"] == 1:
                    st["neg_pre_grad"] = -grad.clone()
                neg_pre = st["neg_pre_grad"]
                diff = neg_pre.add_(grad)
                st["exp_avg"].mul_(beta1).add_(grad, alpha=1 - beta1)
                st["exp_avg_diff"].mul_(beta2).add_(diff, alpha=1 - beta2)
                upd = grad + beta2 * diff
                st["exp_avg_sq"].mul_(beta3).addcmul_(upd, upd, value=1 - beta3)
                denom = (st["exp_avg_sq"].sqrt() / math.sqrt(bc3)).add_(group["eps"])
                step_size_diff = group["lr"] * beta2 / bc2
                step_size = group["lr"] / bc1
                if group["no_prox"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                    p.addcdiv_(st["exp_avg"], denom, value=-step_size)
                    p.addcdiv_(st["exp_avg_diff"], denom, value=-step_size_diff)
                else:
                    p.addcdiv_(st["exp_avg"], denom, value=-step_size)
                    p.addcdiv_(st["exp_avg_diff"], denom, value=-step_size_diff)
                    p.div_(1 + group["lr"] * group["weight_decay"])
                st["neg_pre_grad"] = -grad.clone()
        return loss


def _fused_adamw(*args, **kwargs):
    from .fused_adamw import FusedAdamW

    return FusedAdamW(*args, **kwargs)


def _fully_sharded_adamw(params, model=None, **kwargs):
    """ZeRO-3 AdamW (``parallel/fsdp2.py``); needs the model (units are modules), which ``ModelPT.setup_optimization`` passes."""
    from ...parallel.fsdp2 import FullyShardedAdamW

    if model is None:
        raise ValueError("fully_sharded_adamw needs `model=`: construct it through ModelPT.setup_optimization or pass the module")
    kwargs.pop("amsgrad", None)
    return FullyShardedAdamW(model, **kwargs)


def _sharded_adamw(*args, **kwargs):
    from ...parallel.fsdp import ShardedFusedAdamW

    return ShardedFusedAdamW(*args, **kwargs)


AVAILABLE_OPTIMIZERS: Dict[str, Any] = {
    "sgd": optim.SGD,
    "adam": optim.Adam,
    "adamw": optim.AdamW,
    "adadelta": optim.Adadelta,
    "adamax": optim.Adamax,
    "adagrad": optim.Adagrad,
    "rmsprop": optim.RMSprop,
    "rprop": optim.Rprop,
    "novograd": Novograd,
    "adafactor": Adafactor,
    "adan": Adan,
    "fused_adam": _fused_adamw,
    "fused_adamw": _fused_adamw,
    "distributed_fused_adam": _sharded_adamw,
    "sharded_adamw": _sharded_adamw,
    "fully_sharded_adamw": _fully_sharded_adamw,
    "fsdp2_adamw": _fully_sharded_adamw,
}


def register_optimizer(name: str, optimizer, optimizer_params=None):
    if name in AVAILABLE_OPTIMIZERS:
        raise ValueError(f"Cannot register duplicate optimizer ({name})")
    AVAILABLE_OPTIMIZERS[name] = optimizer
    if optimizer_params is not None:                               # the typed record of its arguments, looked up as "<name>_params"
        from ..config_schemas import register_optimizer_params

        register_optimizer_params(f"{name}_params", optimizer_params)


def parse_optimizer_args(optimizer_name: str, optimizer_kwargs: Any) -> Dict[str, Any]:
    """Flatten an ``optim`` block: drops ``name``/``sched``/``_target_`` and merges ``params`` / ``args``."""
    if optimizer_kwargs is None:
        return {}
    kw = to_container(optimizer_kwargs, resolve=True) if isinstance(optimizer_kwargs, DictConfig) else copy.deepcopy(
        dict(optimizer_kwargs))
    for k in ("name", "sched", "_target_", "cls", "lr_mult", "wd_mult"):
        kw.pop(k, None)
    for nested in ("params", "args"):
        if isinstance(kw.get(nested), dict):
            inner = kw.pop(nested)
            inner.pop("name", None)
            kw.update(inner)
    if "betas" in kw and isinstance(kw["betas"], list):
        kw["betas"] = tuple(kw["betas"])
    if "eps" in kw and isinstance(kw["eps"], list):
        kw["eps"] = tuple(kw["eps"])
    return kw


def get_optimizer(name: str, **kwargs):
    if name not in AVAILABLE_OPTIMIZERS:
        raise ValueError(f"Cannot resolve optimizer '{name}'. Available optimizers are : {list(AVAILABLE_OPTIMIZERS)}")
    return partial(AVAILABLE_OPTIMIZERS[name], **kwargs)

"""Optimizer wrappers: exponential moving average of the weights, and fp32 main parameters for low-precision models.

Reference: ``common/callbacks/ema.py:27-350`` (``EMAOptimizer``: wraps any optimizer; after every ``every_n_steps`` updates the
EMA copy is moved towards the weights with a foreach ``lerp`` — on a side stream when the device is a GPU —, ``swap_ema_weights``
context for validation, EMA state saved with the optimizer state), ``core/optim/optimizer_with_main_params.py:124,356``
(``MainParamsOptimizerWrapper``: fp32 copies of bf16 / fp16 parameters are what the inner optimizer updates; gradients are copied
— optionally accumulated in fp32 and all-reduced in buckets — before the update and the result is cast back).
"""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
from torch.optim import Optimizer


class EMAOptimizer(Optimizer):
    def __init__(self, optimizer: Optimizer, device: Optional[torch.device] = None, decay: float = 0.9999, every_n_steps: int = 1,
                 current_step: int = 0):
        if not 0.0 <= decay <= 1.0:
            raise ValueError("EMA decay value must be between 0 and 1")
        self.optimizer, self.decay, self.every_n_steps, self.current_step = optimizer, decay, every_n_steps, current_step
        self.device = device
        self.ema_params: List[torch.Tensor] = []
        self.in_saving_ema_model_context = False
        self._stream = None
        self._event = None

    param_groups = property(lambda self: self.optimizer.param_groups)
    state = property(lambda self: self.optimizer.state)
    defaults = property(lambda self: self.optimizer.defaults)

    def all_parameters(self) -> List[torch.Tensor]:
        return [p for g in self.optimizer.param_groups for p in g["params"]]

    def _ensure(self):
        params = self.all_parameters()
        if len(self.ema_params) < len(params):
            for p in params[len(self.ema_params):]:
                self.ema_params.append(p.detach().clone().to(self.device or p.device))

    def zero_grad(self, set_to_none: bool = True):
        return self.optimizer.zero_grad(set_to_none=set_to_none)

    def step(self, closure=None, **kw):
        self.join()
        loss = self.optimizer.step(closure) if closure is not None else self.optimizer.step(**kw)
        self._ensure()
        self.current_step += 1
        if self.current_step % self.every_n_steps == 0:
            self.update()
        return loss

    @torch.no_grad()
    def update(self):
        params = [p.detach() for p in self.all_parameters()]
        if params and params[0].is_cuda and self.device in (None, params[0].device):
            if self._stream is None:
                self._stream = torch.cuda.Stream(params[0].device)
            self._stream.wait_stream(torch.cuda.current_stream(params[0].device))
            with torch.cuda.stream(self._stream):
                torch._foreach_lerp_(self.ema_params, params, 1.0 - self.decay)
            self._event = self._stream.record_event()
        else:
            for e, p in zip(self.ema_params, params):
                e.lerp_(p.to(e.device, e.dtype), 1.0 - self.decay)

    def join(self):
        """The next weight update must not overtake an EMA update that still reads the weights on the side stream."""
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
            self._event = None

    @torch.no_grad()
    def switch_main_parameter_weights(self):
        self.join()
        self._ensure()
        for p, e in zip(self.all_parameters(), self.ema_params):
            tmp = p.detach().clone()
            p.copy_(e.to(p.device, p.dtype))
            e.copy_(tmp.to(e.device, e.dtype))

    @contextlib.contextmanager
    def swap_ema_weights(self, enabled: bool = True):
        """Inside the block the model holds the averaged weights (validation / export); the originals come back afterwards."""
        if enabled:
            self.switch_main_parameter_weights()
        try:
            yield
        finally:
            if enabled:
                self.switch_main_parameter_weights()

    def state_dict(self) -> Dict[str, Any]:
        self.join()
        return {"opt": self.optimizer.state_dict(), "ema": [e.clone() for e in self.ema_params], "current_step": self.current_step,
                "decay": self.decay, "every_n_steps": self.every_n_steps}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self.join()
        self.optimizer.load_state_dict(state_dict["opt"])
        self.ema_params = [e.clone().to(self.device) if self.device else e.clone() for e in state_dict["ema"]]
        self.current_step, self.decay, self.every_n_steps = state_dict["current_step"], state_dict["decay"], state_dict["every_n_steps"]

    def add_param_group(self, param_group):
        self.optimizer.add_param_group(param_group)


class MainParamsOptimizerWrapper(Optimizer):
    """Keeps an fp32 "main" copy of every low-precision parameter; the inner optimizer (built by ``optimizer_factory`` over the
    main copies) never sees bf16 values.  ``fp32_grad_accum`` accumulates micro-batch gradients in fp32 main gradients;
    ``async_grad_allreduce`` is honoured by reducing the main gradients of the data-parallel group in ``step``."""

    def __init__(self, params: Iterable[torch.nn.Parameter], optimizer_factory, fp32_grad_accum: bool = False, grad_allreduce_group=None,
                 grad_div_factor: Optional[float] = None):
        self.model_params = [p for p in params if p.requires_grad]
        self.main_params = [p.detach().clone().float().requires_grad_(True) for p in self.model_params]
        self.optimizer = optimizer_factory(self.main_params)
        self.fp32_grad_accum, self.group, self.div = fp32_grad_accum, grad_allreduce_group, grad_div_factor
        if fp32_grad_accum:
            for m in self.main_params:
                m.grad = torch.zeros_like(m)
            self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(i)) for i, p in enumerate(self.model_params)]

    param_groups = property(lambda self: self.optimizer.param_groups)
    state = property(lambda self: self.optimizer.state)

    def _make_hook(self, i):
        def hook(p):
            self.main_params[i].grad.add_(p.grad.float())
            p.grad = None

        return hook

    def zero_grad(self, set_to_none: bool = True):
        for p in self.model_params:
            p.grad = None
        for m in self.main_params:
            if self.fp32_grad_accum:
                m.grad.zero_()
            else:
                m.grad = None

    @torch.no_grad()
    def step(self, closure=None, **kw):
        if not self.fp32_grad_accum:
            for p, m in zip(self.model_params, self.main_params):
                m.grad = None if p.grad is None else p.grad.detach().float()
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            ws = dist.get_world_size(self.group)
            for m in self.main_params:
                if m.grad is not None:
                    m.grad.div_(self.div or ws)
                    dist.all_reduce(m.grad, group=self.group)
        loss = self.optimizer.step(closure) if closure is not None else self.optimizer.step()
        for p, m in zip(self.model_params, self.main_params):
            p.copy_(m.to(p.dtype))
        return loss

    def state_dict(self):
        return {"optimizer": self.optimizer.state_dict(), "fp32_from_fp16_params": [m.detach().clone() for m in self.main_params]}

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd["optimizer"])
        with torch.no_grad():
            for m, s in zip(self.main_params, sd["fp32_from_fp16_params"]):
                m.copy_(s)
            for p, m in zip(self.model_params, self.main_params):
                p.copy_(m.to(p.dtype))

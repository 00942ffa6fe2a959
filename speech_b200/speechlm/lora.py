"""Low-rank adapters for the language-model backbone and regex parameter freezing.

``apply_lora`` wraps the linear layers whose names match ``target_modules`` with ``W x + (alpha / r) · B (A x)``; adapter
parameters carry ``.lora_`` in their names, which ``freeze_and_subset`` never freezes (the reference's convention with
HF-PEFT: ``speechlm2/parts/lora.py:22``, ``parts/optim_setup.py:165``).  ``merge_lora`` folds the adapters back into the
base weights for export.
"""
from __future__ import annotations

import math
import re
from typing import Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from .. import ops


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, r: int = 8, lora_alpha: float = 16.0, lora_dropout: float = 0.0):
        super().__init__()
        self.base = base
        self.r, self.scaling = r, lora_alpha / r
        self.lora_A = nn.Linear(base.in_features, r, bias=False)
        self.lora_B = nn.Linear(r, base.out_features, bias=False)
        nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B.weight)
        self.lora_dropout = nn.Dropout(lora_dropout) if lora_dropout > 0 else nn.Identity()
        for p in base.parameters():
            p.requires_grad_(False)

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    @property
    def in_features(self):
        return self.base.in_features

    @property
    def out_features(self):
        return self.base.out_features

    def forward(self, x):
        y = ops.linear(x, self.base.weight, self.base.bias)
        a = ops.linear(self.lora_dropout(x), self.lora_A.weight, None)
        return y + self.scaling * ops.linear(a, self.lora_B.weight, None).to(y.dtype)

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight + self.scaling * (self.lora_B.weight @ self.lora_A.weight).to(self.base.weight.dtype)


def apply_lora(model: nn.Module, r: int = 8, lora_alpha: float = 16.0, lora_dropout: float = 0.0,
               target_modules: Sequence[str] = ("q_proj", "v_proj"), **_) -> List[str]:
    """Replace matching ``nn.Linear`` children in place; returns the names that were wrapped."""
    wrapped = []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if isinstance(child, nn.Linear) and any(child_name == t or re.fullmatch(t, full) for t in target_modules):
                setattr(module, child_name, LoRALinear(child, r, lora_alpha, lora_dropout))
                wrapped.append(full)
    if not wrapped:
        raise ValueError(f"no linear layer matched target_modules={list(target_modules)}")
    return wrapped


def merge_lora(model: nn.Module) -> None:
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            if isinstance(child, LoRALinear):
                with torch.no_grad():
                    child.base.weight.copy_(child.merged_weight())
                setattr(module, child_name, child.base)


def freeze_and_subset(named_parameters: Iterable, freeze_params: Optional[Sequence[str]] = None,
                      prevent_freeze_params: Optional[Sequence[str]] = None, exclude_from_freeze: str = ".lora_"):
    """Set ``requires_grad=False`` on parameters matching any ``freeze_params`` regex unless they match
    ``prevent_freeze_params`` or are adapter weights; returns the trainable ``(name, param)`` list."""
    fr = [re.compile(p) for p in (freeze_params or [])]
    keep = [re.compile(p) for p in (prevent_freeze_params or [])]
    trainable = []
    for n, p in named_parameters:
        frozen = any(r.match(n) for r in fr) and not any(r.match(n) for r in keep) and exclude_from_freeze not in n
        if frozen:
            p.requires_grad_(False)
        if p.requires_grad:
            trainable.append((n, p))
    return trainable

"""Base classes for building blocks: ``NeuralModule``, ``Loss``, ``AccessMixin``, adapters.

``NeuralModule`` is ``torch.nn.Module`` plus typed ports, config (de)serialisation and
freeze / unfreeze helpers (reference: ``nemo/core/classes/module.py:69``,
``common.py:436,749-842``).  ``AccessMixin`` is the tensor registry that lets a model pick
up intermediate activations (inter-CTC, auxiliary losses; reference:
``nemo/core/classes/mixins/access_mixins.py``).  ``AdapterModuleMixin`` adds named residual
adapters to any module (reference: ``nemo/core/classes/mixins/adapter_mixins.py``).
"""
from __future__ import annotations

import contextlib
import inspect
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from .config import DictConfig, OmegaConf, to_container
from .instantiate import from_config_dict as _from_config_dict
from .neural_types import NeuralType


class Typing:
    @property
    def input_types(self) -> Optional[Dict[str, NeuralType]]:
        return None

    @property
    def output_types(self) -> Optional[Dict[str, NeuralType]]:
        return None


class Serialization:
    @classmethod
    def from_config_dict(cls, config: Any, trainer=None):
        if isinstance(config, (dict,)):
            config = OmegaConf.create(config)
        plain = to_container(config, resolve=True) if isinstance(config, DictConfig) else dict(config)
        if any(k in plain for k in ("_target_", "cls", "target")):
            if "target" in plain and "_target_" not in plain:
                from .instantiate import locate

                target_cls = locate(plain["target"])
                kwargs = {"cfg": OmegaConf.create(plain)}
                if trainer is not None:
                    kwargs["trainer"] = trainer
                return target_cls(**kwargs)
            return _from_config_dict(plain)
        # No target: build ``cls`` from the config (model classes take ``cfg=``).
        params = inspect.signature(cls.__init__).parameters
        if "cfg" in params:
            return cls(cfg=OmegaConf.create(plain), trainer=trainer) if "trainer" in params else cls(cfg=OmegaConf.create(plain))
        return cls(**plain)

    def to_config_dict(self) -> DictConfig:
        cfg = getattr(self, "_cfg", None)
        if cfg is not None:
            return OmegaConf.create(to_container(cfg, resolve=True)) if isinstance(cfg, DictConfig) else OmegaConf.create(cfg)
        raise NotImplementedError("to_config_dict() needs a stored _cfg")


class NeuralModule(nn.Module, Typing, Serialization):
    def __init__(self):
        super().__init__()
        self._frozen_grad_map: Optional[Dict[str, bool]] = None

    @property
    def num_weights(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    def input_example(self, max_batch=None, max_dim=None):
        return None

    def freeze(self) -> None:
        """Stop gradients for every parameter and switch to eval mode; remembers prior flags."""
        grad_map = {}
        for n, p in self.named_parameters():
            grad_map[n] = p.requires_grad
            p.requires_grad = False
        if self._frozen_grad_map is None:
            self._frozen_grad_map = grad_map
        else:
            self._frozen_grad_map.update({k: v for k, v in grad_map.items() if k not in self._frozen_grad_map})
        self.eval()

    def unfreeze(self, partial: bool = False) -> None:
        """Re-enable gradients; with ``partial=True`` only those that were trainable before ``freeze``."""
        if partial and self._frozen_grad_map is None:
            raise ValueError("Cannot unfreeze partially without first freezing the module with `freeze()`")
        for n, p in self.named_parameters():
            if partial and self._frozen_grad_map is not None and n in self._frozen_grad_map:
                p.requires_grad = self._frozen_grad_map[n]
            else:
                p.requires_grad = True
        self._frozen_grad_map = None
        self.train()

    @contextlib.contextmanager
    def as_frozen(self):
        training = self.training
        self.freeze()
        try:
            yield
        finally:
            self.unfreeze(partial=True)
            self.train(training)


class Loss(nn.modules.loss._Loss, Typing, Serialization):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)


class AccessMixin:
    """Module-level tensor registry with a global on/off switch keyed by model GUID."""

    _GLOBAL: Dict[Any, Dict[str, Any]] = {}

    def register_accessible_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if not hasattr(self, "_registry"):
            self._registry: Dict[str, List[torch.Tensor]] = {}
        cfg = self.access_cfg
        if cfg.get("detach", False):
            tensor = tensor.detach()
        if cfg.get("convert_to_cpu", False):
            tensor = tensor.cpu()
        self._registry.setdefault(name, []).append(tensor)

    @classmethod
    def get_module_registry(cls, module: nn.Module) -> Dict[str, Dict[str, List[torch.Tensor]]]:
        out = {}
        for name, m in module.named_modules():
            reg = getattr(m, "_registry", None)
            if reg:
                out[name] = reg
        return out

    def reset_registry(self, registry_key: Optional[str] = None) -> None:
        mods = self.modules() if isinstance(self, nn.Module) else [self]
        for m in mods:
            reg = getattr(m, "_registry", None)
            if reg is None:
                continue
            if registry_key is None:
                reg.clear()
            else:
                reg.pop(registry_key, None)

    @property
    def access_cfg(self) -> Dict[str, Any]:
        guid = getattr(self, "model_guid", None)
        return AccessMixin._GLOBAL.setdefault(guid, {"enabled": False, "detach": False, "convert_to_cpu": False,
                                                     "save_encoder_tensors": False})

    @classmethod
    def update_access_cfg(cls, cfg: dict, guid=None):
        cls._GLOBAL.setdefault(guid, {"enabled": False, "detach": False, "convert_to_cpu": False,
                                      "save_encoder_tensors": False}).update(cfg)

    @classmethod
    def is_access_enabled(cls, guid=None) -> bool:
        return cls._GLOBAL.get(guid, {}).get("enabled", False)

    @classmethod
    def set_access_enabled(cls, access_enabled: bool, guid=None):
        cls.update_access_cfg({"enabled": access_enabled}, guid)


class LinearAdapter(nn.Module):
    """Bottleneck residual adapter: ``LN? -> Linear(d, r) -> act -> Linear(r, d)`` (zero-init output).

    Reference: ``nemo/collections/common/parts/adapter_modules.py``.
    """

    def __init__(self, in_features: int, dim: int, activation: str = "swish", norm_position: str = "pre",
                 dropout: float = 0.0, **_):
        super().__init__()
        act = {"swish": nn.SiLU, "silu": nn.SiLU, "relu": nn.ReLU, "gelu": nn.GELU, "tanh": nn.Tanh}[activation]
        self.norm_position = norm_position
        layers: List[nn.Module] = []
        if norm_position == "pre":
            layers.append(nn.LayerNorm(in_features))
        layers += [nn.Linear(in_features, dim, bias=False), act(), nn.Linear(dim, in_features, bias=False)]
        if norm_position == "post":
            layers.append(nn.LayerNorm(in_features))
        self.module = nn.Sequential(*layers)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        last_linear = [m for m in self.module if isinstance(m, nn.Linear)][-1]
        nn.init.zeros_(last_linear.weight)
        if norm_position == "post":
            nn.init.zeros_(self.module[-1].weight)
            nn.init.zeros_(self.module[-1].bias)

    def forward(self, x):
        y = self.module(x)
        return self.dropout(y) if self.dropout is not None else y


class AdapterModuleMixin:
    """Adds named adapters to a module; the host calls ``forward_enabled_adapters(x)``."""

    adapter_global_cfg_key = "global_cfg"

    def add_adapter(self, name: str, cfg: Any, **kwargs) -> None:
        if not hasattr(self, "adapter_layer"):
            self.adapter_layer = nn.ModuleDict()
            self.adapter_cfg: Dict[str, Any] = {}
        if name in self.adapter_layer:
            raise ValueError(f"Adapter with name `{name}` already exists")
        plain = to_container(cfg, resolve=True) if isinstance(cfg, DictConfig) else dict(cfg)
        from .adapters import ADAPTER_CLASSES, build_strategy

        strategy_cfg = plain.pop("adapter_strategy", None)
        short = str(plain.get("_target_", "")).rsplit(".", 1)[-1]
        if short in ADAPTER_CLASSES:
            kw = {k: v for k, v in plain.items() if k != "_target_"}
            module = ADAPTER_CLASSES[short](adapter_strategy=strategy_cfg, **kw)
        elif "_target_" in plain:
            from .instantiate import TARGET_ALIASES

            TARGET_ALIASES.setdefault("nemo.collections.common.parts.adapter_modules.LinearAdapter",
                                      "speech_b200.core.module.LinearAdapter")
            module = _from_config_dict(plain)
        else:
            module = LinearAdapter(**plain)
        if not hasattr(module, "adapter_strategy"):
            module.adapter_strategy = build_strategy(strategy_cfg)
        plain = {**plain, **({"adapter_strategy": strategy_cfg} if strategy_cfg is not None else {})}
        dev = next((p.device for p in self.parameters()), None) if isinstance(self, nn.Module) else None
        if dev is not None:
            module = module.to(dev)
        self.adapter_layer[name] = module
        self.adapter_cfg[name] = {"enabled": True, "cfg": plain}

    def is_adapter_available(self) -> bool:
        return hasattr(self, "adapter_layer") and len(self.adapter_layer) > 0

    def set_enabled_adapters(self, name: Optional[str] = None, enabled: bool = True) -> None:
        if not self.is_adapter_available():
            raise ValueError("No adapter is available to enable/disable")
        for k in self.adapter_cfg:
            if name is None or k == name:
                self.adapter_cfg[k]["enabled"] = enabled

    def get_enabled_adapters(self) -> List[str]:
        if not self.is_adapter_available():
            return []
        return [k for k, v in self.adapter_cfg.items() if v["enabled"]]

    def unfreeze_enabled_adapters(self, freeze_batchnorm: bool = True) -> None:
        for k in self.get_enabled_adapters():
            for p in self.adapter_layer[k].parameters():
                p.requires_grad = True
            self.adapter_layer[k].train()

    def forward_enabled_adapters(self, x: torch.Tensor) -> torch.Tensor:
        """Apply the enabled adapters in the order they were added, each merged by its strategy (residual add by default)."""
        for k in self.get_enabled_adapters():
            ad = self.adapter_layer[k]
            strategy = getattr(ad, "adapter_strategy", None)
            x = strategy(x, ad, module=self) if strategy is not None else x + ad(x)
        return x

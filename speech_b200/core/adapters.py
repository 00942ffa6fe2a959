"""Adapters: strategies that merge an adapter's output into the host's activations, attention-type adapters, and the
model-level mixin that routes ``add_adapter("encoder:name", cfg)`` to sub-modules and saves / restores adapters on their own.

Module-level hosting (``add_adapter`` / ``forward_enabled_adapters`` on a layer) is :class:`speech_b200.core.module.AdapterModuleMixin`.
Reference: ``core/classes/mixins/adapter_mixins.py`` (``AdapterModelPTMixin`` :550-1000, module mixin :120-540),
``core/classes/mixins/adapter_mixin_strategies.py`` (``ResidualAddAdapterStrategy``, ``ReturnResultAdapterStrategy``),
``collections/asr/parts/submodules/adapters/multi_head_attention_adapter_module.py`` (attention / positional-encoding adapters),
``collections/asr/parts/mixins/asr_adapter_mixins.py`` (``ASRAdapterModelMixin``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from .config import DictConfig, OmegaConf, open_dict, to_container


# ------------------------------------------------------------------------------------------------ strategies
class ResidualAddAdapterStrategy:
    """``x + adapter(x)``.  ``stochastic_depth``: during training the adapter's contribution of a whole batch is dropped with
    that probability.  ``l2_lambda`` > 0 records ``l2_lambda * mean((adapter(x))^2)`` on the host as an auxiliary loss (the
    model adds ``adapter_auxiliary_loss()`` to its training loss) so that the adapter stays close to the identity."""

    def __init__(self, stochastic_depth: float = 0.0, l2_lambda: float = 0.0):
        self.stochastic_depth, self.l2_lambda = float(stochastic_depth), float(l2_lambda)

    def __call__(self, x: torch.Tensor, adapter: nn.Module, *, module: nn.Module) -> torch.Tensor:
        out = adapter(x)
        if module.training and self.stochastic_depth > 0.0:
            if float(torch.rand(())) < self.stochastic_depth:
                out = out * 0.0
        if module.training and self.l2_lambda > 0.0 and any(p.requires_grad for p in adapter.parameters()):
            aux = getattr(module, "_adapter_aux_losses", None)
            if aux is None:
                aux = module._adapter_aux_losses = []
            aux.append(self.l2_lambda * out.float().pow(2).mean())
        return x + out


class ReturnResultAdapterStrategy:
    """The adapter's output replaces the input (adapters that already contain their own residual path, e.g. attention adapters
    that update positional encodings)."""

    def __call__(self, x: torch.Tensor, adapter: nn.Module, *, module: nn.Module) -> torch.Tensor:
        return adapter(x)


def build_strategy(cfg: Optional[Dict[str, Any]]):
    if cfg is None:
        return ResidualAddAdapterStrategy()
    cfg = dict(cfg)
    target = str(cfg.pop("_target_", "ResidualAddAdapterStrategy")).rsplit(".", 1)[-1]
    if target == "ResidualAddAdapterStrategy":
        return ResidualAddAdapterStrategy(**{k: v for k, v in cfg.items() if k in ("stochastic_depth", "l2_lambda")})
    if target == "ReturnResultAdapterStrategy":
        return ReturnResultAdapterStrategy()
    raise ValueError(f"unknown adapter strategy '{target}'")


def adapter_auxiliary_loss(model: nn.Module) -> Optional[torch.Tensor]:
    """Sum (and clear) the auxiliary losses recorded by residual strategies with ``l2_lambda`` during the last forward."""
    terms = []
    for m in model.modules():
        aux = getattr(m, "_adapter_aux_losses", None)
        if aux:
            terms += aux
            m._adapter_aux_losses = []
    return torch.stack(terms).sum() if terms else None


# ------------------------------------------------------------------------------------------------ attention adapters
class MultiHeadAttentionAdapter(nn.Module):
    """Self-attention adapter: ``LayerNorm -> multi-head attention (absolute positions) -> dropout``, output projection
    zero-initialised so that the adapter starts as a no-op under the residual strategy.  ``forward(x, mask=None)``."""

    def __init__(self, n_head: int, n_feat: int, dropout_rate: float = 0.0, proj_dim: Optional[int] = None, adapter_strategy: Any = None, **_):
        super().__init__()
        d = n_feat if not proj_dim or proj_dim < 1 else proj_dim * n_head
        if d % n_head:
            raise ValueError("projection width must be divisible by the number of heads")
        self.h, self.dk = n_head, d // n_head
        self.pre_norm = nn.LayerNorm(n_feat)
        self.linear_q, self.linear_k, self.linear_v = nn.Linear(n_feat, d), nn.Linear(n_feat, d), nn.Linear(n_feat, d)
        self.linear_out = nn.Linear(d, n_feat)
        self.dropout = nn.Dropout(dropout_rate)
        nn.init.zeros_(self.linear_out.weight)
        nn.init.zeros_(self.linear_out.bias)
        self.adapter_strategy = build_strategy(adapter_strategy)

    def _scores_extra(self, q: torch.Tensor) -> Optional[torch.Tensor]:
        return None

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, T, _ = x.shape
        h = self.pre_norm(x)
        q = self.linear_q(h).view(B, T, self.h, self.dk).transpose(1, 2)
        k = self.linear_k(h).view(B, T, self.h, self.dk).transpose(1, 2)
        v = self.linear_v(h).view(B, T, self.h, self.dk).transpose(1, 2)
        s = torch.matmul(q, k.transpose(-1, -2))
        extra = self._scores_extra(q)
        if extra is not None:
            s = s + extra
        s = s / self.dk ** 0.5
        if mask is not None:
            s = s.masked_fill(mask.unsqueeze(1), -1e4)
        p = torch.softmax(s, dim=-1)
        if mask is not None:
            p = p.masked_fill(mask.unsqueeze(1), 0.0)
        y = torch.matmul(self.dropout(p), v).transpose(1, 2).reshape(B, T, -1)
        return self.linear_out(y)


class RelPositionMultiHeadAttentionAdapter(MultiHeadAttentionAdapter):
    """As above with a learned relative-position bias per head over offsets ``[-max_rel, max_rel]`` (clamped beyond)."""

    def __init__(self, n_head: int, n_feat: int, dropout_rate: float = 0.0, proj_dim: Optional[int] = None, max_rel: int = 64,
                 adapter_strategy: Any = None, **_):
        super().__init__(n_head, n_feat, dropout_rate, proj_dim, adapter_strategy)
        self.max_rel = max_rel
        self.rel_emb = nn.Parameter(torch.zeros(2 * max_rel + 1, n_head, self.dk))
        nn.init.normal_(self.rel_emb, std=0.02)

    def _scores_extra(self, q: torch.Tensor) -> torch.Tensor:
        T = q.shape[2]
        idx = torch.arange(T, device=q.device)
        rel = (idx[:, None] - idx[None, :]).clamp(-self.max_rel, self.max_rel) + self.max_rel          # [T, T]
        table = torch.einsum("bhtd,rhd->bhtr", q, self.rel_emb.to(q.dtype))                                # [B, H, T, 2R+1]
        return table.gather(3, rel[None, None].expand(q.shape[0], q.shape[1], T, T))


class PositionalEncodingAdapter(nn.Module):
    """Adds a learned correction to the features as a function of absolute position (up to ``max_len`` frames); zero at start."""

    def __init__(self, d_model: int, max_len: int = 5000, xscale: float = 1.0, adapter_strategy: Any = None, **_):
        super().__init__()
        self.pe = nn.Parameter(torch.zeros(max_len, d_model))
        self.xscale = xscale
        self.adapter_strategy = build_strategy(adapter_strategy or {"_target_": "ReturnResultAdapterStrategy"})

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[1]
        if T > self.pe.shape[0]:
            raise ValueError(f"sequence of {T} frames exceeds the adapter's max_len {self.pe.shape[0]}")
        return x * self.xscale + self.pe[:T].unsqueeze(0).to(x.dtype)


ADAPTER_CLASSES = {"MultiHeadAttentionAdapter": MultiHeadAttentionAdapter, "RelPositionMultiHeadAttentionAdapter": RelPositionMultiHeadAttentionAdapter,
                   "PositionalEncodingAdapter": PositionalEncodingAdapter}


# ------------------------------------------------------------------------------------------------ model-level mixin
class AdapterModelPTMixin:
    """Model-level adapter management.  Adapter names may carry a module prefix, ``"encoder:ad1"`` / ``"decoder:ad1"`` /
    ``"joint:ad1"``; without a prefix the default module (the encoder) hosts the adapter.  The model config keeps every adapter's
    config under ``cfg.adapters`` so that a restored model rebuilds its adapters before loading weights."""

    adapter_module_names: Tuple[str, ...] = ("encoder", "decoder", "joint")
    default_adapter_module_name: str = "encoder"

    # ---- routing
    def resolve_adapter_module_name_(self, name: str) -> Tuple[str, str]:
        if ":" in name:
            module, adapter = name.split(":", 1)
            if module not in self.adapter_module_names:
                raise ValueError(f"adapter module '{module}' is not one of {self.adapter_module_names}")
            return module, adapter
        return self.default_adapter_module_name, name

    def _adapter_hosts(self, module_name: Optional[str] = None) -> List[Tuple[str, nn.Module]]:
        names = [module_name] if module_name else list(self.adapter_module_names)
        return [(n, getattr(self, n)) for n in names if getattr(self, n, None) is not None and hasattr(getattr(self, n), "add_adapter")]

    # ---- API
    def add_adapter(self, name: str, cfg: Any) -> None:
        module_name, adapter_name = self.resolve_adapter_module_name_(name)
        hosts = self._adapter_hosts(module_name)
        if not hosts:
            raise ValueError(f"module '{module_name}' of {type(self).__name__} does not support adapters")
        plain = to_container(cfg, resolve=True) if isinstance(cfg, DictConfig) else dict(cfg)
        hosts[0][1].add_adapter(adapter_name, plain)
        with open_dict(self.cfg):
            if self.cfg.get("adapters", None) is None:
                self.cfg.adapters = OmegaConf.create({})
            self.cfg.adapters[f"{module_name}:{adapter_name}"] = OmegaConf.create({**plain, "enabled": True})

    def is_adapter_available(self) -> bool:
        return any(h.is_adapter_available() for _, h in self._adapter_hosts())

    def get_enabled_adapters(self) -> List[str]:
        return [f"{n}:{a}" for n, h in self._adapter_hosts() if h.is_adapter_available() for a in h.get_enabled_adapters()]

    def set_enabled_adapters(self, name: Optional[str] = None, enabled: bool = True) -> None:
        if name is None:
            for _, h in self._adapter_hosts():
                if h.is_adapter_available():
                    h.set_enabled_adapters(None, enabled)
        else:
            module_name, adapter_name = self.resolve_adapter_module_name_(name)
            for _, h in self._adapter_hosts(module_name):
                h.set_enabled_adapters(adapter_name, enabled)
        if self.cfg.get("adapters", None) is not None:
            with open_dict(self.cfg):
                for key in self.cfg.adapters:
                    if name is None or key == "%s:%s" % self.resolve_adapter_module_name_(name):
                        self.cfg.adapters[key].enabled = enabled

    def unfreeze_enabled_adapters(self, freeze_batchnorm: bool = True) -> None:
        for _, h in self._adapter_hosts():
            if h.is_adapter_available():
                h.unfreeze_enabled_adapters(freeze_batchnorm)

    def adapter_parameters(self, name: Optional[str] = None) -> Dict[str, torch.Tensor]:
        """``{state-dict key: tensor}`` of the adapters' weights (all, or the named one)."""
        want = None if name is None else "%s:%s" % self.resolve_adapter_module_name_(name)
        out = {}
        for k, v in self.state_dict().items():
            if ".adapter_layer." not in k and not k.startswith("adapter_layer."):
                continue
            head, _, rest = k.partition("adapter_layer.")
            adapter = rest.split(".", 1)[0]
            module = head.split(".", 1)[0] if head else self.default_adapter_module_name
            if want is None or want == f"{module}:{adapter}":
                out[k] = v
        return out

    def save_adapters(self, filepath: str, name: Optional[str] = None) -> None:
        """Write the adapters' weights and configs only (a few MB next to a multi-GB base model)."""
        keys = None if name is None else {"%s:%s" % self.resolve_adapter_module_name_(name)}
        cfgs = {k: to_container(v, resolve=True) for k, v in (self.cfg.get("adapters", None) or {}).items() if keys is None or k in keys}
        if not cfgs:
            raise ValueError("no adapter to save" + (f" under the name '{name}'" if name else ""))
        torch.save({"__cfg__": cfgs, "state_dict": {k: v.detach().cpu() for k, v in self.adapter_parameters(name).items()}}, filepath)

    def load_adapters(self, filepath: str, name: Optional[str] = None, map_location: Any = "cpu", strict: bool = True) -> None:
        """Add the adapters of ``filepath`` that this model does not have yet (all, or the named one) and load their weights."""
        blob = torch.load(filepath, map_location=map_location, weights_only=False)
        want = None if name is None else "%s:%s" % self.resolve_adapter_module_name_(name)
        have = set((self.cfg.get("adapters", None) or {}).keys())
        loaded = []
        for key, cfg in blob["__cfg__"].items():
            if want is not None and key != want:
                continue
            cfg = dict(cfg)
            enabled = cfg.pop("enabled", True)
            if key not in have:
                self.add_adapter(key, cfg)
            self.set_enabled_adapters(key, enabled)
            loaded.append(key)
        if want is not None and not loaded:
            raise KeyError(f"adapter '{name}' is not in {filepath}")
        sd = {k: v for k, v in blob["state_dict"].items()
              if any(f".adapter_layer.{key.split(':', 1)[1]}." in k or k.startswith(f"adapter_layer.{key.split(':', 1)[1]}.") for key in loaded)}
        missing, unexpected = self.load_state_dict(sd, strict=False)
        if strict and unexpected:
            raise KeyError(f"adapter weights without a home in this model: {unexpected[:5]}")

    def restore_adapters_from_cfg(self) -> None:
        """Called by constructors after the base modules exist: rebuild the adapters listed under ``cfg.adapters``."""
        for key, cfg in list((self.cfg.get("adapters", None) or {}).items()):
            module_name, adapter_name = self.resolve_adapter_module_name_(key)
            hosts = self._adapter_hosts(module_name)
            plain = to_container(cfg, resolve=True)
            enabled = plain.pop("enabled", True)
            if hosts and not (hosts[0][1].is_adapter_available() and adapter_name in getattr(hosts[0][1], "adapter_cfg", {})):
                hosts[0][1].add_adapter(adapter_name, plain)
                hosts[0][1].set_enabled_adapters(adapter_name, enabled)

    def freeze_base_and_train_adapters(self) -> int:
        """The usual recipe: freeze everything, then unfreeze the enabled adapters; returns the number of trainable parameters."""
        for p in self.parameters():
            p.requires_grad = False
        self.unfreeze_enabled_adapters()
        return sum(p.numel() for p in self.parameters() if p.requires_grad)


class ASRAdapterModelMixin(AdapterModelPTMixin):
    """ASR models host adapters in the encoder (every Conformer layer), the prediction / CTC decoder and the joint network."""

    def add_adapter(self, name: str, cfg: Any) -> None:
        module_name, _ = self.resolve_adapter_module_name_(name)
        plain = to_container(cfg, resolve=True) if isinstance(cfg, DictConfig) else dict(cfg)
        host = getattr(self, module_name, None)
        d = getattr(host, "d_model", None) or getattr(host, "_feat_out", None)
        if module_name == "encoder" and d is not None:
            for key in ("in_features", "n_feat", "d_model"):
                if key in plain and plain[key] != d:
                    raise ValueError(f"adapter {key}={plain[key]} does not match the encoder width {d}")
        super().add_adapter(name, plain)

"""Post-training quantisation of the linear layers of a trained model to FP8 (e4m3), with calibration.

The reference quantises ASR encoders to INT8 through an external optimiser package (``examples/asr/quantization``:
``speech_to_text_calibrate.py`` collects activation ranges on a calibration manifest, ``speech_to_text_quant_infer.py`` evaluates
WER of the quantised model).  On Blackwell the tensor cores take FP8 operands natively, so the scheme here is FP8:

* weights: per-output-channel scale ``s_w[o] = max|W[o, :]| / 448`` (448 = largest e4m3 value), stored as e4m3 + fp32 scales;
* activations: one static per-tensor scale per layer from calibration — the ``percentile`` of the observed ``max|x|`` over the
  calibration batches (``max`` for 100) — so inference needs no run-time reduction.

``calibrate`` runs user batches through the model with observers on every selected ``nn.Linear`` input.  ``quantize_model``
replaces those layers by ``QuantLinear``, which computes ``(q(x) q(W)^T) * s_x * s_w + b``: the operands are rounded to e4m3
exactly as the tensor core would see them and multiplied in the compute dtype (the arithmetic of an FP8 GEMM with fp32
accumulation, evaluated with the bf16 / fp32 kernels that exist).  ``quantization_report`` lists per-layer signal-to-quantisation-noise
ratios so that sensitive layers can be kept in bf16 (``skip`` patterns).  ``save_quantized`` / ``load_quantized`` store the e4m3
weights and scales (half the bytes of bf16).
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

E4M3_MAX = 448.0
_FP8 = getattr(torch, "float8_e4m3fn", None)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Round to the e4m3 grid (values beyond +-448 saturate); returned in the input dtype."""
    x = x.clamp(-E4M3_MAX, E4M3_MAX)
    if _FP8 is not None:
        return x.to(_FP8).to(x.dtype)
    # emulation: 3 mantissa bits, exponent range of e4m3 (smallest normal 2^-6, subnormal step 2^-9)
    xf = x.float()
    e = torch.floor(torch.log2(xf.abs().clamp(min=2.0 ** -9))).clamp(min=-6.0)
    step = torch.pow(2.0, e - 3)
    return (torch.round(xf / step) * step).to(x.dtype)


class _Observer:
    def __init__(self):
        self.maxima: List[float] = []

    def __call__(self, module, inputs):
        self.maxima.append(float(inputs[0].detach().abs().max()))

    def amax(self, percentile: float = 100.0) -> float:
        if not self.maxima:
            return 0.0
        t = torch.tensor(self.maxima)
        return float(t.max() if percentile >= 100.0 else torch.quantile(t, percentile / 100.0))


def _selected(model: nn.Module, include: Optional[Sequence[str]], skip: Optional[Sequence[str]]):
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or isinstance(m, QuantLinear):
            continue
        if include and not any(re.search(p, name) for p in include):
            continue
        if skip and any(re.search(p, name) for p in skip):
            continue
        yield name, m


@torch.no_grad()
def calibrate(model: nn.Module, batches: Iterable, forward: Optional[Callable] = None, include: Optional[Sequence[str]] = None,
              skip: Optional[Sequence[str]] = None, percentile: float = 99.9) -> Dict[str, float]:
    """Returns ``{layer name: activation amax}`` after running ``forward(model, batch)`` (default ``model(*batch)``) over the batches."""
    obs, handles = {}, []
    for name, m in _selected(model, include, skip):
        obs[name] = _Observer()
        handles.append(m.register_forward_pre_hook(obs[name]))
    was_training = model.training
    model.eval()
    try:
        for b in batches:
            forward(model, b) if forward is not None else model(*b)
    finally:
        for h in handles:
            h.remove()
        model.train(was_training)
    return {n: o.amax(percentile) for n, o in obs.items()}


class QuantLinear(nn.Module):
    def __init__(self, lin: nn.Linear, act_amax: float):
        super().__init__()
        w = lin.weight.detach().float()
        s_w = (w.abs().amax(dim=1, keepdim=True) / E4M3_MAX).clamp(min=1e-12)
        q = to_e4m3(w / s_w)
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.register_buffer("weight_q", q.to(_FP8) if _FP8 is not None else q)
        self.register_buffer("weight_scale", s_w.squeeze(1))
        self.register_buffer("act_scale", torch.tensor(max(act_amax, 1e-12) / E4M3_MAX))
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def dequantized_weight(self, dtype=torch.float32) -> torch.Tensor:
        return (self.weight_q.to(torch.float32) * self.weight_scale.unsqueeze(1)).to(dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xq = to_e4m3(x / self.act_scale.to(x.dtype))
        y = torch.nn.functional.linear(xq, self.weight_q.to(x.dtype))
        y = y * (self.act_scale * self.weight_scale).to(y.dtype)
        return y if self.bias is None else y + self.bias.to(y.dtype)


def quantize_model(model: nn.Module, amax: Dict[str, float]) -> List[str]:
    """Replace every calibrated ``nn.Linear`` in place; returns the replaced names."""
    done = []
    for name, act in amax.items():
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        lin = getattr(parent, leaf)
        if isinstance(lin, nn.Linear) and not isinstance(lin, QuantLinear):
            setattr(parent, leaf, QuantLinear(lin, act))
            done.append(name)
    return done


@torch.no_grad()
def quantization_report(model: nn.Module, amax: Dict[str, float]) -> List[Dict[str, float]]:
    """Weight SQNR (dB) per layer for the per-channel e4m3 scheme, most sensitive first."""
    rows = []
    for name in amax:
        lin = model.get_submodule(name)
        if not isinstance(lin, nn.Linear):
            continue
        w = lin.weight.detach().float()
        s = (w.abs().amax(dim=1, keepdim=True) / E4M3_MAX).clamp(min=1e-12)
        err = to_e4m3(w / s) * s - w
        sqnr = 10.0 * torch.log10(w.pow(2).sum() / err.pow(2).sum().clamp(min=1e-30))
        rows.append({"layer": name, "weight_sqnr_db": float(sqnr), "act_amax": float(amax[name]), "params": w.numel()})
    return sorted(rows, key=lambda r: r["weight_sqnr_db"])


def save_quantized(model: nn.Module, path: str) -> None:
    state = {}
    for k, v in model.state_dict().items():
        state[k] = v.view(torch.uint8) if _FP8 is not None and v.dtype == _FP8 else v
    torch.save({"state": state, "quantized": [n for n, m in model.named_modules() if isinstance(m, QuantLinear)]}, path)


def load_quantized(model: nn.Module, path: str) -> nn.Module:
    """``model`` is the float architecture; its listed layers are replaced and the stored tensors loaded."""
    blob = torch.load(path, map_location="cpu")
    quantize_model(model, {n: 1.0 for n in blob["quantized"]})
    state = {}
    ref = model.state_dict()
    for k, v in blob["state"].items():
        state[k] = v.view(_FP8) if _FP8 is not None and k in ref and ref[k].dtype == _FP8 else v
    model.load_state_dict(state)
    return model

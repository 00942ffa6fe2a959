"""Confidence estimation for recognition hypotheses (reference: ``parts/utils/asr_confidence_utils.py``).

Frame confidence comes from the output distribution (maximum probability or a normalised entropy: Gibbs, Tsallis or Renyi
with temperature ``alpha``, linear or exponential normalisation); token confidence aggregates the frames a token spans; word
confidence aggregates its tokens (``mean`` / ``min`` / ``max`` / ``prod``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


@dataclass
class ConfidenceMethodConfig:
    name: str = "entropy"                  # "max_prob" | "entropy"
    entropy_type: str = "tsallis"          # "gibbs" | "tsallis" | "renyi"
    alpha: float = 0.33
    entropy_norm: str = "exp"              # "lin" | "exp"


@dataclass
class ConfidenceConfig:
    preserve_frame_confidence: bool = False
    preserve_token_confidence: bool = False
    preserve_word_confidence: bool = False
    exclude_blank: bool = True
    aggregation: str = "min"
    tdt_include_duration: bool = False
    method_cfg: ConfidenceMethodConfig = field(default_factory=ConfidenceMethodConfig)


def get_confidence_aggregation_bank() -> dict:
    return {"mean": lambda x: sum(x) / max(len(x), 1), "min": min, "max": max, "prod": lambda x: math.prod(x)}


def frame_confidence(log_probs: torch.Tensor, cfg: Optional[ConfidenceMethodConfig] = None) -> torch.Tensor:
    """log_probs [..., V] → confidence in [0, 1] per frame."""
    cfg = cfg or ConfidenceMethodConfig()
    lp = log_probs.float()
    V = lp.shape[-1]
    if cfg.name == "max_prob":
        return (lp.max(-1).values.exp() * V - 1) / (V - 1)
    a = float(cfg.alpha)
    p = lp.exp()
    if cfg.entropy_type == "gibbs":
        ent = -(p.pow(a) * lp * a).sum(-1) / p.pow(a).sum(-1).clamp(min=1e-30) if abs(a - 1) > 1e-6 else -(p * lp).sum(-1)
        ent_max = math.log(V)
        if abs(a - 1) > 1e-6:
            # Gibbs entropy of the tempered distribution p^a / Z
            q = torch.softmax(a * lp, -1)
            ent = -(q * torch.log(q.clamp(min=1e-30))).sum(-1)
        if cfg.entropy_norm == "exp":
            return ((-ent).exp() * V - 1) / (V - 1)
        return 1 - ent / ent_max
    s = p.pow(a).sum(-1)
    if cfg.entropy_type == "tsallis":
        ent = (s - 1) / (1 - a)
        ent_max = (V ** (1 - a) - 1) / (1 - a)
        if cfg.entropy_norm == "exp":
            return ((-ent).exp() - math.exp(-ent_max)) / (1 - math.exp(-ent_max))
        return 1 - ent / ent_max
    if cfg.entropy_type == "renyi":
        ent = torch.log2(s) / (1 - a)
        ent_max = math.log2(V)
        if cfg.entropy_norm == "exp":
            return (torch.pow(2.0, -ent) * V - 1) / (V - 1)
        return 1 - ent / ent_max
    raise ValueError(f"unknown entropy type {cfg.entropy_type}")


def ctc_token_confidence(log_probs: torch.Tensor, length: int, blank: int, cfg: Optional[ConfidenceConfig] = None):
    """Greedy CTC path of one utterance → (tokens, per-token confidence, per-frame confidence)."""
    cfg = cfg or ConfidenceConfig()
    agg = get_confidence_aggregation_bank()[cfg.aggregation]
    lp = log_probs[:length]
    fc = frame_confidence(lp, cfg.method_cfg)
    path = lp.argmax(-1).tolist()
    toks, confs, cur, prev = [], [], [], blank
    for t, p in enumerate(path):
        if p != prev:
            if cur:
                confs.append(float(agg(cur)))
                cur = []
            if p != blank:
                toks.append(p)
        if p != blank:
            cur.append(float(fc[t]))
        elif not cfg.exclude_blank and cur:
            cur.append(float(fc[t]))
        prev = p
    if cur:
        confs.append(float(agg(cur)))
    return toks, confs[: len(toks)], fc


def word_confidence(token_conf: Sequence[float], tokens_per_word: Sequence[int], aggregation: str = "min") -> List[float]:
    agg = get_confidence_aggregation_bank()[aggregation]
    out, k = [], 0
    for n in tokens_per_word:
        out.append(float(agg(list(token_conf[k:k + n]))) if n else 1.0)
        k += n
    return out

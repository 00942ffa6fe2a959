"""Online classifier-free-guidance distillation for MagpieTTS.

Guided sampling runs the decoder twice per step (with and without the text condition) and mixes the logits:
``l = l_uncond + s (l_cond - l_uncond)``.  Distillation trains a student that reproduces the guided distribution in ONE
conditional pass: on every batch the frozen teacher is run both ways under teacher forcing, the student once, and the loss is
``KL(softmax(l_teacher_guided / T) || softmax(l_student / T)) T^2`` over the valid frames and all codebooks, optionally mixed
with the ordinary cross-entropy on the data (``ce_weight``).  The guidance scale is either fixed or drawn per batch from
``cfg_scale_range``; in the second case the student receives the scale as an extra embedding added to its decoder input (a
two-layer MLP of the scalar), so one student serves every scale.

Reference: ``tts/models/magpietts_cfg_distillation.py`` (teacher / student set-up, guided-logit target, KL objective).
"""
from __future__ import annotations

import copy
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from .magpietts import MagpieTTSModel


def guided_logits(cond: torch.Tensor, uncond: torch.Tensor, scale) -> torch.Tensor:
    scale = torch.as_tensor(scale, dtype=cond.dtype, device=cond.device)
    while scale.dim() and scale.dim() < cond.dim():
        scale = scale.unsqueeze(-1)
    return uncond + scale * (cond - uncond)


def distillation_kl(student_logits: torch.Tensor, teacher_logits: torch.Tensor, mask: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Mean over the masked positions (and codebooks) of ``KL(teacher || student)`` at ``temperature``."""
    t = F.log_softmax(teacher_logits.float() / temperature, dim=-1)
    s = F.log_softmax(student_logits.float() / temperature, dim=-1)
    kl = (t.exp() * (t - s)).sum(-1)                                                         # [B, T, C]
    m = mask.unsqueeze(-1).to(kl.dtype)
    return (kl * m).sum() / (m.sum() * kl.shape[-1]).clamp(min=1) * temperature ** 2


class MagpieTTSModelOnlineCFGDistillation(MagpieTTSModel):
    def __init__(self, cfg: DictConfig, trainer=None, codec=None, tokenizer=None, teacher: Optional[MagpieTTSModel] = None):
        super().__init__(cfg=cfg, trainer=trainer, codec=codec, tokenizer=tokenizer)
        cfg = self._cfg
        self.kd_temperature = float(cfg_get(cfg, "distillation_temperature", 1.0))
        self.ce_weight = float(cfg_get(cfg, "ce_weight", 0.0))
        rng = cfg_get(cfg, "cfg_scale_range", None)
        self.cfg_scale_range: Optional[Tuple[float, float]] = tuple(float(v) for v in rng) if rng else None
        self.cfg_scale = float(cfg_get(cfg, "cfg_scale", 2.5))
        if self.cfg_scale_range is not None:
            self.scale_embedding = nn.Sequential(nn.Linear(1, self.d_model), nn.SiLU(), nn.Linear(self.d_model, self.d_model))
            nn.init.zeros_(self.scale_embedding[-1].weight)
            nn.init.zeros_(self.scale_embedding[-1].bias)
        if teacher is None:
            teacher = copy.deepcopy(self) if not cfg_get(cfg, "teacher_path", None) else MagpieTTSModel.restore_from(cfg.teacher_path)
            if hasattr(teacher, "scale_embedding"):
                del teacher.scale_embedding
        object.__setattr__(self, "_teacher", teacher)                # frozen, not a sub-module: never trained or check-pointed
        teacher.eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        self._scale_now: Optional[torch.Tensor] = None

    def embed_audio_tokens(self, codes):
        x = super().embed_audio_tokens(codes)
        if self._scale_now is not None and self.cfg_scale_range is not None:
            x = x + self.scale_embedding(self._scale_now.view(1, 1, 1).to(x.dtype)).to(x.dtype)
        return x

    def _loss(self, batch):
        text, text_len, audio, audio_len = batch[:4]
        codes, codes_len = self.audio_to_codes(audio, audio_len)
        codes, codes_len = self.stack_codes(codes, codes_len)
        dev = codes.device
        if self.cfg_scale_range is not None:
            lo, hi = self.cfg_scale_range
            scale = torch.rand((), device=dev) * (hi - lo) + lo
        else:
            scale = torch.tensor(self.cfg_scale, device=dev)
        teacher: MagpieTTSModel = self._teacher
        with torch.no_grad():
            t_cond = teacher.forward(text, text_len, codes, codes_len, drop_condition=False)[0]
            t_unc = teacher.forward(text, text_len, codes, codes_len, drop_condition=True)[0]
            target = guided_logits(t_cond, t_unc, scale)
        self._scale_now = scale
        try:
            logits, _, _, xmask = self.forward(text, text_len, codes, codes_len, drop_condition=False)
        finally:
            self._scale_now = None
        kd = distillation_kl(logits, target, xmask, self.kd_temperature)
        loss, logs = kd, {"distillation_loss": kd.detach(), "cfg_scale": scale.detach()}
        if self.ce_weight > 0:
            tgt = codes[:, :, 1:].permute(0, 2, 1)
            ce = F.cross_entropy(logits[xmask].reshape(-1, logits.shape[-1]), tgt[xmask].reshape(-1))
            loss = loss + self.ce_weight * ce
            logs["codebook_loss"] = ce.detach()
        return loss, logs

    @torch.no_grad()
    def infer_batch(self, text, text_len, cfg_scale: Optional[float] = None, **kw):
        """One conditional pass per step: the guidance is in the weights (and in the scale embedding)."""
        kw.pop("use_cfg", None)
        if self.cfg_scale_range is not None:
            s = self.cfg_scale if cfg_scale is None else cfg_scale
            self._scale_now = torch.tensor(float(s), device=text.device)
        try:
            return super().infer_batch(text, text_len, use_cfg=False, **kw)
        finally:
            self._scale_now = None

"""Losses beyond CTC / transducer / cross-entropy: additive-margin angular softmax (speaker models), multi-label BCE with
length masks (diarization), and the self-supervised objectives (contrastive with quantised targets, masked-token
prediction, multi-decoder MLM).
Reference: ``losses/angularloss.py``, ``losses/bce_loss.py``, ``losses/ssl_losses/{contrastive,mlm,ctc,rnnt}.py``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.module import Loss


class AngularSoftmaxLoss(Loss):
    """Additive angular margin on cosine logits: the target logit becomes ``s * cos(theta + m)``, the others ``s * cos``
    (``angularloss.py:24-69``)."""

    def __init__(self, scale: float = 20.0, margin: float = 1.35):
        super().__init__()
        self.eps = 1e-7
        self.scale, self.margin = scale, margin

    def forward(self, logits, labels):
        target_cos = torch.clamp(logits.gather(1, labels.view(-1, 1)).squeeze(1), -1.0 + self.eps, 1 - self.eps)
        num = self.scale * torch.cos(torch.acos(target_cos) + self.margin)
        mask = torch.ones_like(logits, dtype=torch.bool).scatter_(1, labels.view(-1, 1), False)
        excl = (logits * self.scale).masked_fill(~mask, float("-inf"))
        denom = torch.logaddexp(num, torch.logsumexp(excl, dim=1))
        return -(num - denom).mean()


class BCELoss(Loss):
    """Frame-level multi-speaker binary cross entropy with per-sample target lengths (``bce_loss.py:27-144``)."""

    def __init__(self, reduction: str = "mean", alpha: float = 1.0, weight=None, sorted_preds: bool = False,
                 sorted_loss: bool = False, class_normalization: bool = False):
        super().__init__()
        self.reduction, self.alpha = reduction, alpha
        self.register_buffer("weight", torch.as_tensor(weight, dtype=torch.float32) if weight is not None else torch.tensor([0.5, 0.5]))
        self.class_normalization = class_normalization

    def forward(self, probs, labels, target_lens=None, signal_lengths=None, enable_autocast=False):
        lens = target_lens if target_lens is not None else signal_lengths
        probs = probs.float().clamp(1e-6, 1 - 1e-6)
        labels = labels.float()
        T = probs.shape[1]
        mask = torch.ones(probs.shape[:2], device=probs.device, dtype=torch.bool) if lens is None else \
            (torch.arange(T, device=probs.device)[None] < lens[:, None])
        w = torch.where(labels > 0.5, self.weight[1], self.weight[0]) * 2.0
        bce = -(labels * probs.log() + (1 - labels) * (1 - probs).log()) * w
        bce = bce * mask.unsqueeze(-1)
        if self.reduction == "sum":
            return bce.sum()
        return bce.sum() / (mask.sum() * probs.shape[-1]).clamp(min=1)


class ContrastiveLoss(Loss):
    """wav2vec-2.0 style: for every masked step the (optionally quantised) target must be picked among ``num_negatives``
    distractors sampled from other masked steps of the same utterance (``ssl_losses/contrastive.py:27-300``)."""

    def __init__(self, in_dim: int, proj_dim: int = 128, combine_time_steps: int = 1, num_negatives: int = 100,
                 quantized_targets: bool = False, codebook_size: int = 320, prob_ppl_weight: float = 0.1,
                 logit_temp: float = 0.1, reduce: str = "sum", sample_from_same_utterance_only: bool = True,
                 sample_from_non_masked: bool = False, sample_from_codebook: bool = False, group_loss: bool = False,
                 num_groups: int = 2, quantizer_temp_start: float = 2.0, quantizer_temp_min: float = 0.5,
                 quantizer_temp_decay: float = 0.999995, mask_threshold: float = 0.8, store_ids: bool = True,
                 reduce_ids: bool = False, multiplier: int = 16):
        super().__init__()
        self.combine_time_steps, self.num_negatives = combine_time_steps, num_negatives
        self.quantized_targets, self.prob_ppl_weight = quantized_targets, prob_ppl_weight
        self.logit_temp, self.reduce, self.mask_threshold = logit_temp, reduce, mask_threshold
        self.sample_from_non_masked = sample_from_non_masked
        d = in_dim * combine_time_steps
        if quantized_targets:
            self.num_groups, self.codebook_size = num_groups, codebook_size
            self.q_proj = nn.Linear(d, num_groups * codebook_size)
            self.codebook = nn.Parameter(torch.randn(num_groups, codebook_size, proj_dim // num_groups))
            self.temp, self.temp_min, self.temp_decay = quantizer_temp_start, quantizer_temp_min, quantizer_temp_decay
        else:
            self.target_proj = nn.Linear(d, proj_dim)
        self.prob_ppl = None

    def _targets(self, spec):
        B, T, D = spec.shape
        if not self.quantized_targets:
            return self.target_proj(spec), spec.new_zeros(())
        logits = self.q_proj(spec).view(B * T, self.num_groups, self.codebook_size)
        if self.training:
            y = F.gumbel_softmax(logits.float(), tau=self.temp, hard=True, dim=-1)
            self.temp = max(self.temp * self.temp_decay, self.temp_min)
        else:
            y = F.one_hot(logits.argmax(-1), self.codebook_size).float()
        avg = torch.softmax(logits.float(), dim=-1).mean(0)
        ppl = torch.exp(-(avg * (avg + 1e-7).log()).sum(-1)).sum()
        q = torch.einsum("ngc,gcd->ngd", y, self.codebook).reshape(B, T, -1)
        total = self.num_groups * self.codebook_size
        return q, (total - ppl) / total

    def forward(self, spectrograms, spec_masks, decoder_outputs, decoder_lengths=None):
        """spectrograms / spec_masks: [B, D, T] (mask = 1 where the input was masked); decoder_outputs: [B, T', proj]."""
        spec = spectrograms.transpose(1, 2)
        masks = spec_masks.transpose(1, 2)
        B, T, D = spec.shape
        c = self.combine_time_steps
        T2 = min(T // c, decoder_outputs.shape[1])
        spec = spec[:, : T2 * c].reshape(B, T2, c * D)
        masked = masks[:, : T2 * c].reshape(B, T2, c * D).float().mean(-1) > self.mask_threshold
        out = decoder_outputs[:, :T2]
        targets, ppl_pen = self._targets(spec)
        loss = out.new_zeros((), dtype=torch.float32)
        count = 0
        for b in range(B):
            idx = masked[b].nonzero().squeeze(-1)
            if decoder_lengths is not None:
                idx = idx[idx < decoder_lengths[b]]
            if idx.numel() < 2:
                continue
            pool = torch.arange(T2, device=spec.device) if self.sample_from_non_masked else idx
            n = idx.numel()
            k = min(self.num_negatives, pool.numel() - 1)
            neg = pool[torch.randint(0, pool.numel(), (n, k), device=spec.device)]
            cand = torch.cat([idx.view(n, 1), neg], dim=1)
            sims = F.cosine_similarity(out[b, idx].unsqueeze(1).float(), targets[b, cand].float(), dim=-1) / self.logit_temp
            dup = (cand[:, 1:] == idx.view(n, 1))
            sims[:, 1:] = sims[:, 1:].masked_fill(dup, float("-inf"))
            loss = loss + F.cross_entropy(sims, torch.zeros(n, dtype=torch.long, device=spec.device), reduction="sum")
            count += n
        if self.reduce == "mean" and count:
            loss = loss / count
        if self.quantized_targets:
            loss = loss + self.prob_ppl_weight * ppl_pen * max(count, 1)
        return loss


class MLMLoss(Loss):
    """Masked-token prediction: NLL of the target token at masked steps (``ssl_losses/mlm.py:24-140``)."""

    def __init__(self, combine_time_steps: int = 1, mask_threshold: float = 0.8):
        super().__init__()
        self.combine_time_steps, self.mask_threshold = combine_time_steps, mask_threshold

    def forward(self, decoder_outputs, targets, decoder_lengths=None, target_lengths=None, spec_masks=None, masks=None):
        """decoder_outputs: log-probs [B, T, V]; targets: [B, T]; masks: [B, D, T*c] or [B, T] (1 = masked)."""
        m = masks if masks is not None else spec_masks
        B, T, V = decoder_outputs.shape
        T = min(T, targets.shape[1])          # the quantiser floors T / combine_time_steps, the encoder may round up
        decoder_outputs = decoder_outputs[:, :T]
        if m is None:
            sel = torch.ones((B, T), dtype=torch.bool, device=decoder_outputs.device)
        elif m.dim() == 3:
            c = self.combine_time_steps
            mm = m.transpose(1, 2)[:, : T * c]
            mm = torch.nn.functional.pad(mm, (0, 0, 0, T * c - mm.shape[1])).reshape(B, T, -1)
            sel = mm.float().mean(-1) > self.mask_threshold
        else:
            sel = m[:, :T] > 0.5
        if decoder_lengths is not None:
            sel = sel & (torch.arange(T, device=sel.device)[None] < decoder_lengths[:, None])
        nll = -decoder_outputs.float().gather(-1, targets[:, :T].unsqueeze(-1)).squeeze(-1)
        return (nll * sel).sum() / sel.sum().clamp(min=1)


class MultiMLMLoss(Loss):
    """Sum of MLM losses over several codebooks: outputs [B, T, V, H] (or [B, T, V*H]), targets [B, T*H] or [B, T, H]."""

    def __init__(self, combine_time_steps: int = 1, mask_threshold: float = 0.8, num_decoders: int = 1, squeeze_single: bool = False):
        super().__init__()
        self.num_decoders, self.squeeze_single = num_decoders, squeeze_single
        self.mlm_loss = MLMLoss(combine_time_steps, mask_threshold)

    def forward(self, masks, decoder_outputs, targets, decoder_lengths=None, target_lengths=None):
        H = self.num_decoders
        if decoder_outputs.dim() == 3:
            B, T, VH = decoder_outputs.shape
            decoder_outputs = decoder_outputs.view(B, T, VH // H, H)
        B, T = decoder_outputs.shape[:2]
        targets = targets.reshape(B, -1, H)
        loss = 0.0
        for h in range(H):
            loss = loss + self.mlm_loss(decoder_outputs=decoder_outputs[..., h], targets=targets[..., h],
                                        decoder_lengths=decoder_lengths, masks=masks)
        return loss / H

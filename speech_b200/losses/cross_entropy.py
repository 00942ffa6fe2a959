"""Token-level losses shared by the AED, speech-LLM and TTS models.

``SmoothedCrossEntropyLoss`` takes *log-probabilities*, smooths over the non-target vocabulary and
averages over non-pad tokens (reference: ``nemo/collections/common/losses/smoothed_cross_entropy.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from ..core.module import Loss

__all__ = ["SmoothedCrossEntropyLoss", "CrossEntropyLoss", "BCEWithLogitsLoss", "MSELoss", "AggregatorLoss"]


class SmoothedCrossEntropyLoss(Loss):
    def __init__(self, pad_id: Optional[int] = None, label_smoothing: float = 0.0, predict_last_k: int = 0,
                 eps: float = 1e-6, per_token_reduction: bool = True):
        super().__init__()
        self._pad_id, self._eps, self._predict_last_k = pad_id, eps, predict_last_k
        self._label_smoothing, self._per_token_reduction = label_smoothing, per_token_reduction

    def forward(self, log_probs, labels, output_mask=None):
        if output_mask is None and self._pad_id is None:
            raise ValueError("Both output_mask and pad_id are None")
        if output_mask is None:
            output_mask = (labels != self._pad_id)
        output_mask = output_mask.to(log_probs.dtype)
        if output_mask.dim() != labels.dim():
            raise ValueError("output_mask and labels must have the same rank")
        bsz, length, vocab = log_probs.shape
        smoothing = vocab * self._label_smoothing / (vocab - 1)
        target_lp = log_probs.gather(2, labels.unsqueeze(2).long()).squeeze(2)
        smoothing_lp = log_probs.mean(dim=-1)
        nll = (1.0 - smoothing) * target_lp + smoothing * smoothing_lp
        nll = nll[:, -self._predict_last_k:]
        mask = output_mask[:, -self._predict_last_k:]
        if self._per_token_reduction:
            return -torch.sum(nll * mask) / (mask.sum() + self._eps)
        return -torch.sum(nll * mask, dim=-1)


class CrossEntropyLoss(torch.nn.CrossEntropyLoss):
    def __init__(self, logits_ndim=2, weight=None, reduction="mean", ignore_index=-100):
        if weight is not None and not torch.is_tensor(weight):
            weight = torch.FloatTensor(weight)
        super().__init__(weight=weight, reduction=reduction, ignore_index=ignore_index)
        self._logits_dim = logits_ndim

    def forward(self, logits, labels, loss_mask=None):
        logits_flat = logits.reshape(-1, logits.shape[-1])
        labels_flat = labels.reshape(-1)
        if loss_mask is not None:
            keep = loss_mask.reshape(-1) > 0.5
            logits_flat, labels_flat = logits_flat[keep], labels_flat[keep]
        if len(labels_flat) == 0:
            return super().forward(logits, torch.argmax(logits, dim=-1))
        return super().forward(logits_flat, labels_flat)


class BCEWithLogitsLoss(torch.nn.BCEWithLogitsLoss):
    def forward(self, logits, labels, loss_mask=None):
        labels = torch.stack(labels).transpose(0, 1) if isinstance(labels, (list, tuple)) else labels
        return super().forward(logits, labels.float())


class MSELoss(torch.nn.MSELoss):
    def forward(self, preds, labels):
        return super().forward(preds, labels)


class AggregatorLoss(Loss):
    def __init__(self, num_inputs: int = 2, weights=None):
        super().__init__()
        self._num_losses = num_inputs
        if weights is not None and len(weights) != num_inputs:
            raise ValueError("Length of weights should be equal to the number of inputs (num_inputs)")
        self._weights = weights

    def forward(self, **kwargs):
        values = [kwargs[k] for k in sorted(kwargs.keys())]
        loss = torch.zeros_like(values[0])
        for i, v in enumerate(values):
            loss = loss + (v * self._weights[i] if self._weights is not None else v)
        return loss

"""CTC loss wrapper: blank is the last class, input [B,T,V+1] log-probs, ``mean_batch`` / ``mean_volume``
reductions (reference: ``nemo/collections/asr/losses/ctc.py:24-80``).  The lattice recursion itself is
``ops.ctc_loss`` — a hand-written kernel on GPUs, ``torch.nn.functional.ctc_loss`` on the CPU."""
from __future__ import annotations

import torch

from .. import ops
from ..core.module import Loss
from ..core.neural_types import LabelsType, LengthsType, LogprobsType, LossType, NeuralType, typecheck

__all__ = ["CTCLoss"]


class CTCLoss(Loss):
    def __init__(self, num_classes: int, zero_infinity: bool = False, reduction: str = "mean_batch"):
        super().__init__()
        self._blank = num_classes
        if reduction not in ("none", "mean", "sum", "mean_batch", "mean_volume"):
            raise ValueError("`reduction` must be one of [mean, sum, mean_batch, mean_volume]")
        self.config_reduction = reduction
        self.zero_infinity = zero_infinity
        self._apply_reduction = reduction in ("mean_batch", "mean_volume")

    @property
    def input_types(self):
        return {"log_probs": NeuralType(("B", "T", "D"), LogprobsType()), "targets": NeuralType(("B", "T"), LabelsType()),
                "input_lengths": NeuralType(("B",), LengthsType()), "target_lengths": NeuralType(("B",), LengthsType())}

    @property
    def output_types(self):
        return {"loss": NeuralType(elements_type=LossType())}

    def reduce(self, losses, target_lengths):
        if self.config_reduction == "mean_batch":
            return losses.mean()
        if self.config_reduction == "mean_volume":
            return losses.sum() / target_lengths.sum()
        if self.config_reduction == "mean":
            return (losses / target_lengths.clamp(min=1)).mean()
        if self.config_reduction == "sum":
            return losses.sum()
        return losses

    @typecheck()
    def forward(self, log_probs, targets, input_lengths, target_lengths):
        input_lengths = input_lengths.long()
        target_lengths = target_lengths.long()
        targets = targets.long()
        loss = ops.ctc_loss(log_probs, targets, input_lengths, target_lengths, blank=self._blank,
                            zero_infinity=self.zero_infinity)
        return self.reduce(loss, target_lengths)

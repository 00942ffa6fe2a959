"""Transducer loss front-end: RNNT, TDT and multi-blank RNNT behind one resolver.

Loss names accepted by ``RNNTLoss(loss_name=...)`` follow the reference resolver
(``nemo/collections/asr/losses/rnnt.py:88-158,206-330``): ``default`` / ``warprnnt_numba`` / ``warprnnt`` /
``pytorch`` (RNNT), ``tdt`` / ``tdt_pytorch`` (token-and-duration transducer with ``durations``, ``sigma``,
``omega``), ``multiblank_rnnt`` / ``multiblank_rnnt_pytorch``.  Reductions ``mean_batch | mean | sum |
mean_volume`` (``:421-436``).  T and U axes are trimmed to the batch maxima (``:472-481``).

All variants are served by one implementation: the lattice recursion of ``speech_b200.ops`` (hand-written
kernels on GPUs).  With a fused joint (``forward_fused``) the logits tensor is never built.
"""
from __future__ import annotations

import random
from typing import Any, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..ops import reference as _ref
from ..core.module import Loss
from ..core.neural_types import LabelsType, LengthsType, LogprobsType, LossType, NeuralType, typecheck

RNNT_LOSS_RESOLVER = {
    "default": "rnnt", "warprnnt": "rnnt", "warprnnt_numba": "rnnt", "pytorch": "rnnt", "rnnt": "rnnt",
    "tdt": "tdt", "tdt_pytorch": "tdt",
    "multiblank_rnnt": "multiblank", "multiblank_rnnt_pytorch": "multiblank",
    "graph_rnnt": "graph_rnnt", "graph_w_transducer": "graph_w",
}


def resolve_rnnt_default_loss_name() -> str:
    return "warprnnt_numba"


class RNNTLoss(Loss):
    def __init__(self, num_classes: int, reduction: str = "mean_batch", loss_name: str = "default",
                 loss_kwargs: Optional[Dict[str, Any]] = None):
        super().__init__()
        if reduction not in (None, "none", "mean", "sum", "mean_batch", "mean_volume"):
            raise ValueError("`reduction` must be one of [mean, sum, mean_batch, mean_volume]")
        if loss_name not in RNNT_LOSS_RESOLVER:
            raise ValueError(f"Provided `loss_name` {loss_name} not in list of available RNNT losses \n "
                             f"{list(RNNT_LOSS_RESOLVER)}")
        self._blank = num_classes
        self.reduction = reduction
        self.kind = RNNT_LOSS_RESOLVER[loss_name]
        kw = dict(loss_kwargs or {})
        self.fastemit_lambda = float(kw.get("fastemit_lambda", 0.0))
        self.clamp = float(kw.get("clamp", -1.0))
        self.durations: List[int] = list(kw.get("durations", [])) if self.kind == "tdt" else []
        self.sigma = float(kw.get("sigma", 0.0))
        self.omega = float(kw.get("omega", 0.0))
        self.big_blank_durations: List[int] = list(kw.get("big_blank_durations", [])) if self.kind == "multiblank" else []
        self._graph_loss = None
        if self.kind in ("graph_rnnt", "graph_w"):
            from .graph_transducer import GraphRnntLoss, GraphWTransducerLoss

            gk = {k: v for k, v in kw.items() if k in ("double_scores", "cast_to_float32", "use_grid_implementation", "connect_composed")}
            if self.kind == "graph_w":
                self._graph_loss = GraphWTransducerLoss(num_classes, eps_weight=float(kw.get("eps_weight", 0.0)),
                                                        last_blank_mode=str(kw.get("last_blank_mode", "force_final")), **gk)
            else:
                self._graph_loss = GraphRnntLoss(num_classes, **gk)
        if self.kind == "tdt" and not self.durations:
            raise ValueError("TDT loss needs `durations` in loss_kwargs")
        if self.kind == "multiblank" and not self.big_blank_durations:
            raise ValueError("multi-blank RNNT loss needs `big_blank_durations` in loss_kwargs")
        self._fp16_numba = False

    @property
    def input_types(self):
        return {"log_probs": NeuralType(("B", "T", "T", "D"), LogprobsType()),
                "targets": NeuralType(("B", "T"), LabelsType()),
                "input_lengths": NeuralType(("B",), LengthsType()),
                "target_lengths": NeuralType(("B",), LengthsType())}

    @property
    def output_types(self):
        return {"loss": NeuralType(elements_type=LossType())}

    def reduce(self, losses, target_lengths):
        if isinstance(losses, list):
            losses = torch.cat(losses, 0)
            target_lengths = torch.cat(target_lengths, 0) if isinstance(target_lengths, list) else target_lengths
        if self.reduction == "mean_batch":
            return losses.mean()
        if self.reduction == "mean":
            return torch.div(losses, target_lengths).mean()
        if self.reduction == "sum":
            return losses.sum()
        if self.reduction == "mean_volume":
            return losses.sum() / target_lengths.sum()
        return losses

    def _use_plain_rnnt_this_call(self) -> bool:
        """TDT ``omega``: with this probability a call trains with the plain RNNT lattice on the token logits."""
        return self.kind == "tdt" and self.omega > 0 and self.training and random.random() < self.omega

    # ------------------------------------------------------------------ from logits
    def per_utterance_from_logits(self, acts, labels, act_lens, label_lens):
        max_t, max_u = int(act_lens.max()), int(label_lens.max())
        if acts.shape[1] != max_t:
            acts = acts.narrow(1, 0, max_t)
        if acts.shape[2] != max_u + 1:
            acts = acts.narrow(2, 0, max_u + 1)
        labels = labels[:, :max_u]
        act_lens, label_lens = act_lens.long(), label_lens.long()
        if self._graph_loss is not None:
            return self._graph_loss(acts, labels, act_lens, label_lens)
        if self.kind == "tdt":
            if self._use_plain_rnnt_this_call():
                loss = ops.transducer_loss_from_logits(acts[..., : -len(self.durations)].contiguous(), labels, act_lens,
                                                       label_lens, self._blank, [], 0.0)
            else:
                loss = ops.transducer_loss_from_logits(acts.contiguous(), labels, act_lens, label_lens, self._blank,
                                                       self.durations, self.sigma)
        elif self.kind == "multiblank":
            if acts.is_cuda and ops._use_native(acts):
                from ..ops import native_transducer as _nt

                loss = _nt.multiblank_loss_from_logits(acts, labels, act_lens, label_lens, self._blank,
                                                       self.big_blank_durations, self.sigma)
            else:
                loss = _ref.multiblank_loss_from_logits(acts, labels, act_lens, label_lens, self._blank,
                                                        self.big_blank_durations, self.sigma)
        else:
            loss = ops.transducer_loss_from_logits(acts.contiguous(), labels, act_lens, label_lens, self._blank, [], 0.0)
        if self.fastemit_lambda:
            loss = loss * (1.0 + self.fastemit_lambda)
        return loss

    @typecheck()
    def forward(self, log_probs, targets, input_lengths, target_lengths):
        loss = self.per_utterance_from_logits(log_probs, targets.long(), input_lengths, target_lengths)
        return self.reduce(loss, target_lengths)

    # ------------------------------------------------------------------ fused with the joint
    def forward_fused(self, f, g, weight, bias, transcripts, encoder_lengths, transcript_lengths, act: str = "relu",
                      fused_batch_size: Optional[int] = None, dropout_p: float = 0.0):
        """f: [B,T,H] and g: [B,U+1,H] projected encoder / prediction outputs; returns per-utterance losses.  ``dropout_p`` is
        the joint network's dropout, applied inside the fused kernels on GPUs."""
        f_len, y_len = encoder_lengths.long(), transcript_lengths.long()
        transcripts = transcripts.long()
        if self.kind == "multiblank":
            return self.forward_from_joint_fn(None, f, g, transcripts, f_len, y_len, fused_batch_size,
                                              w=weight, b=bias, act=act)
        durations, sigma, w, b = self.durations, self.sigma, weight, bias
        if self._use_plain_rnnt_this_call():
            nd = len(self.durations)
            durations, sigma, w, b = [], 0.0, weight[:-nd], (bias[:-nd] if bias is not None else None)
        return ops.transducer_joint_loss(f, g, w, b, transcripts, f_len, y_len, self._blank, durations, sigma, act,
                                         self.fastemit_lambda, fused_batch_size or 0, dropout_p=dropout_p)

    def forward_from_joint_fn(self, joint, f, g, transcripts, f_len, y_len, fused_batch_size, w=None, b=None, act="relu"):
        """Generic sub-batched path: build logits for ``fused_batch_size`` utterances at a time."""
        B = f.shape[0]
        sb = fused_batch_size or B
        out = []
        for s in range(0, B, sb):
            e = min(B, s + sb)
            tl, ul = int(f_len[s:e].max()), int(y_len[s:e].max())
            fs, gs = f[s:e, :tl], g[s:e, : ul + 1]
            if joint is not None:
                prev = joint.log_softmax
                joint.log_softmax = False
                try:
                    logits = joint.joint_after_projection(fs, gs)
                finally:
                    joint.log_softmax = prev
            else:
                logits = _ref.joint_logits(fs.float(), gs.float(), w.float(), None if b is None else b.float(), act)
            out.append(self.per_utterance_from_logits(logits, transcripts[s:e], f_len[s:e], y_len[s:e]))
        return torch.cat(out)

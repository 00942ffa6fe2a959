"""Word / character error rate with distributed accumulation.

``word_error_rate`` and the ``WER`` metric object (update / compute / reset, numerator and denominator summed
across ranks) follow ``nemo/collections/asr/metrics/wer.py:187``.  The edit distance is a plain
dynamic-programming Levenshtein distance over word or character lists.
"""
from __future__ import annotations

from typing import Sequence, List, Optional, Tuple

import torch
import torch.distributed as dist


def edit_distance(a: List, b: List) -> int:
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


def word_error_rate(hypotheses: List[str], references: List[str], use_cer: bool = False) -> float:
    if len(hypotheses) != len(references):
        raise ValueError(f"In word error rate calculation, hypotheses and reference lists must have the same number "
                         f"of elements. But I got:{len(hypotheses)} and {len(references)} correspondingly")
    scores = words = 0
    for h, r in zip(hypotheses, references):
        hl, rl = (list(h), list(r)) if use_cer else (h.split(), r.split())
        words += len(rl)
        scores += edit_distance(hl, rl)
    return scores / words if words != 0 else float("inf")


def edit_operations(hyp: Sequence, ref: Sequence) -> Tuple[int, int, int]:
    """(insertions, deletions, substitutions) of one minimum-cost alignment of ``hyp`` against ``ref``."""
    R, H = len(ref), len(hyp)
    d = [[0] * (H + 1) for _ in range(R + 1)]
    for i in range(R + 1):
        d[i][0] = i
    for j in range(H + 1):
        d[0][j] = j
    for i in range(1, R + 1):
        ri, row, up = ref[i - 1], d[i], d[i - 1]
        for j in range(1, H + 1):
            row[j] = min(up[j - 1] + (ri != hyp[j - 1]), up[j] + 1, row[j - 1] + 1)
    ins = dele = sub = 0
    i, j = R, H
    while i > 0 or j > 0:
        if i > 0 and j > 0 and d[i][j] == d[i - 1][j - 1] + (ref[i - 1] != hyp[j - 1]):
            sub += ref[i - 1] != hyp[j - 1]
            i, j = i - 1, j - 1
        elif i > 0 and d[i][j] == d[i - 1][j] + 1:
            dele += 1
            i -= 1
        else:
            ins += 1
            j -= 1
    return ins, dele, sub


def word_error_rate_detail(hypotheses, references, use_cer=False) -> Tuple[float, int, float, float, float]:
    """(WER, reference tokens, insertion rate, deletion rate, substitution rate)."""
    words = ins = dele = sub = 0
    for h, r in zip(hypotheses, references):
        hl, rl = (list(h), list(r)) if use_cer else (h.split(), r.split())
        words += len(rl)
        a, b, c = edit_operations(hl, rl)
        ins, dele, sub = ins + a, dele + b, sub + c
    if not words:
        return float("inf"), 0, float("inf"), float("inf"), float("inf")
    return (ins + dele + sub) / words, words, ins / words, dele / words, sub / words


class WER:
    """Accumulates edit-distance numerator / word-count denominator; ``decoding`` turns model outputs into text."""

    def __init__(self, decoding, use_cer: bool = False, log_prediction: bool = True, fold_consecutive: bool = True,
                 batch_dim_index: int = 0, dist_sync_on_step: bool = False, sync_on_compute: bool = True, **_):
        self.decoding, self.use_cer, self.log_prediction = decoding, use_cer, log_prediction
        self.fold_consecutive, self.batch_dim_index = fold_consecutive, batch_dim_index
        self.sync_on_compute = sync_on_compute
        self.reset()
        self.last_hypotheses: List[str] = []

    def reset(self):
        self.scores = torch.tensor(0, dtype=torch.long)
        self.words = torch.tensor(0, dtype=torch.long)

    def to(self, device):
        return self

    def decode(self, predictions, predictions_lengths):
        from ..decoding.ctc_decoding import AbstractCTCDecoding

        if isinstance(self.decoding, AbstractCTCDecoding):
            return self.decoding.ctc_decoder_predictions_tensor(predictions, predictions_lengths,
                                                                fold_consecutive=self.fold_consecutive)
        if hasattr(self.decoding, "rnnt_decoder_predictions_tensor"):
            return self.decoding.rnnt_decoder_predictions_tensor(predictions, predictions_lengths)
        return self.decoding.decode_predictions_tensor(predictions, predictions_lengths)

    @torch.no_grad()
    def update(self, predictions, predictions_lengths, targets, targets_lengths, predictions_mask=None,
               input_ids=None, **_):
        refs = []
        tg = targets.long().cpu()
        tl = targets_lengths.long().cpu()
        for i in range(tg.shape[0]):
            refs.append(self.decoding.decode_tokens_to_str(tg[i, : tl[i]].tolist()))
        hyps = [h.text for h in self.decode(predictions, predictions_lengths)]
        self.last_hypotheses = hyps
        if self.log_prediction and hyps:
            from .logging import logging

            logging.info(f"reference:{refs[0]}")
            logging.info(f"predicted:{hyps[0]}")
        s = w = 0
        for h, r in zip(hyps, refs):
            hl, rl = (list(h), list(r)) if self.use_cer else (h.split(), r.split())
            w += len(rl)
            s += edit_distance(hl, rl)
        self.scores += s
        self.words += w

    def compute(self):
        scores, words = self.scores.clone().float(), self.words.clone().float()
        if self.sync_on_compute and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
            t = torch.stack([scores, words]).to(dev)
            dist.all_reduce(t)
            scores, words = t[0].cpu(), t[1].cpu()
        return (scores / words if words > 0 else torch.tensor(float("inf"))), scores, words


class GlobalAverageLossMetric:
    def __init__(self, take_avg_loss: bool = True, **_):
        self.take_avg_loss = take_avg_loss
        self.reset()

    def reset(self):
        self.loss_sum, self.num = torch.tensor(0.0, dtype=torch.float64), torch.tensor(0, dtype=torch.long)

    def update(self, loss, num_measurements):
        n = int(num_measurements)
        self.loss_sum += float(loss) * n if self.take_avg_loss else float(loss)
        self.num += n

    def compute(self):
        s, n = self.loss_sum.clone(), self.num.clone().double()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
            t = torch.stack([s, n]).to(dev)
            dist.all_reduce(t)
            s, n = t[0].cpu(), t[1].cpu()
        return (s / n).float() if n > 0 else torch.tensor(float("nan"))


class TopKClassificationAccuracy:
    """``update(logits [N, C], labels [N])`` accumulates, for every k, how often the label is among the k best classes;
    ``compute()`` -> list of accuracies in the order of ``top_k``.  Counts are summed over ranks when a process group exists."""

    def __init__(self, top_k: Sequence[int] = (1,)):
        self.top_k = sorted(set(int(k) for k in top_k))
        self.reset()

    def reset(self):
        self.correct = torch.zeros(len(self.top_k), dtype=torch.float64)
        self.total = 0.0

    @torch.no_grad()
    def update(self, logits: torch.Tensor, labels: torch.Tensor):
        kmax = min(max(self.top_k), logits.shape[-1])
        pred = logits.topk(kmax, dim=-1).indices
        hit = pred == labels.view(-1, 1)
        for i, k in enumerate(self.top_k):
            self.correct[i] += float(hit[:, : min(k, kmax)].any(dim=1).sum())
        self.total += labels.numel()

    def compute(self) -> List[float]:
        c, t = self.correct.clone(), torch.tensor([self.total], dtype=torch.float64)
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            dev = "cuda" if torch.distributed.get_backend() == "nccl" else "cpu"
            c, t = c.to(dev), t.to(dev)
            torch.distributed.all_reduce(c)
            torch.distributed.all_reduce(t)
            c, t = c.cpu(), t.cpu()
        return [float(x / t.clamp(min=1)) for x in c]


class Perplexity:
    """Mean perplexity of a stream of distributions: ``update(probs=...)`` or ``update(logits=...)`` ([..., V]); the entropy of
    every distribution is exponentiated and averaged (``validate_args`` checks that probabilities sum to one)."""

    def __init__(self, validate_args: bool = True):
        self.validate = validate_args
        self.reset()

    def reset(self):
        self.sum, self.n = 0.0, 0

    @torch.no_grad()
    def update(self, probs: Optional[torch.Tensor] = None, logits: Optional[torch.Tensor] = None):
        if (probs is None) == (logits is None):
            raise ValueError("give probs or logits, not both")
        if probs is not None and self.validate and not torch.allclose(probs.sum(-1), torch.ones_like(probs.sum(-1)), atol=1e-4):
            raise ValueError("probabilities do not sum to one")
        logp = torch.log_softmax(logits.float(), -1) if logits is not None else torch.log(probs.float().clamp(min=1e-30))
        ent = -(logp.exp() * logp).sum(-1)
        self.sum += float(ent.exp().sum())
        self.n += ent.numel()

    def compute(self) -> float:
        return self.sum / max(1, self.n)

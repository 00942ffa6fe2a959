"""Lattice ("graph") formulations of the transducer loss: plain RNN-T and the W-Transducer for partially transcribed audio.

The reference builds these lattices as k2 finite-state acceptors and takes the total score in the log semiring
(``parts/k2/graph_transducer.py:38,232`` — ``GraphRnntLoss`` with its grid / composed construction;
``parts/k2/w_transducer.py:26`` — ``GraphWTransducerLoss``; ``parts/k2/rnnt_logprobs.py`` — target / blank log-probabilities
without a full log-softmax tensor).  Here the same lattices are evaluated directly: the grid has a fixed shape, so the total
score is a row-by-row recursion in which each row is a *linear recurrence along the label axis* solved with one cumulative sum
and one cumulative log-sum-exp — ``T`` vectorised steps over ``[B, U+1]`` tensors, differentiable by autograd, no FSA library.

Lattice of the W-Transducer (``w_transducer.py:200-290``): the RNN-T grid plus (a) skip arcs from the start state to
``(t, 0)`` for every later frame — unlabelled audio before the transcript — and (b) skip arcs from ``(t, U)`` to the last
frame — unlabelled audio after it; every skip arc costs ``eps_weight``.  ``last_blank_mode="force_final"`` makes the end skip
land in ``(T-1, U)`` so that the final blank is still scored; ``"allow_ignore"`` lets it bypass that blank.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..core.module import Loss

_NEG = -1.0e30   # "log zero" that keeps gradients finite


def rnnt_logprobs(logits: torch.Tensor, targets: torch.Tensor, blank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Log-probabilities of the only two symbols the lattice uses at every node: the next target and blank.

    logits [B, T, U+1, V], targets [B, U] -> (target_logprobs [B, T, U+1] with the last column = log zero, blank_logprobs
    [B, T, U+1]).  Only the normaliser is reduced over V; the full log-softmax tensor is never materialised."""
    B, T, U1, V = logits.shape
    lse = torch.logsumexp(logits.float(), dim=-1)
    blank_lp = logits[..., blank].float() - lse
    tgt = torch.nn.functional.pad(targets.long(), (0, U1 - targets.shape[1]))[:, None, :, None].expand(B, T, U1, 1)
    tgt_lp = logits.gather(-1, tgt).squeeze(-1).float() - lse
    last = torch.arange(U1, device=logits.device) >= targets.shape[1]
    return tgt_lp.masked_fill(last[None, None, :], _NEG), blank_lp


def _row_scan(entry: torch.Tensor, emit: torch.Tensor) -> torch.Tensor:
    """alpha[u] = logaddexp(entry[u], alpha[u-1] + emit[u-1]) along the last axis (a first-order linear recurrence in the log
    semiring): alpha = E + logcumsumexp(entry - E) with E the exclusive prefix sum of emit."""
    E = torch.cumsum(torch.nn.functional.pad(emit[..., :-1], (1, 0)), dim=-1)   # shifted, not cumsum - emit: log-zero entries cancel badly
    return E + torch.logcumsumexp(entry - E, dim=-1)


class GraphRnntLoss(Loss):
    """RNN-T negative log-likelihood per utterance from joint logits ``[B, T, U+1, V]``."""

    def __init__(self, blank: int, use_grid_implementation: bool = True, connect_composed: bool = False,
                 double_scores: bool = False, cast_to_float32: bool = False, return_graph: bool = False):
        super().__init__()
        self.blank = blank
        self.double_scores = double_scores
        self.cast_to_float32 = cast_to_float32

    # W-Transducer hooks -----------------------------------------------------------------------------------------------
    def _start_skip(self) -> float:
        return _NEG

    def _finish(self, alpha_last: torch.Tensor, blank_last: torch.Tensor, act_lens: torch.Tensor) -> torch.Tensor:
        """alpha_last / blank_last [B, T]: score of node (t, U_b) and of its blank arc; returns the total log-likelihood."""
        idx = (act_lens.long() - 1).clamp(min=0).unsqueeze(1)
        return (alpha_last.gather(1, idx) + blank_last.gather(1, idx)).squeeze(1)

    def forward(self, acts: torch.Tensor, labels: torch.Tensor, act_lens: torch.Tensor, label_lens: torch.Tensor) -> torch.Tensor:
        if self.cast_to_float32:
            acts = acts.float()
        B, T, U1, _ = acts.shape
        labels = labels[:, : U1 - 1]
        tgt_lp, blank_lp = rnnt_logprobs(acts, labels, self.blank)
        dt = torch.float64 if self.double_scores else torch.float32
        tgt_lp, blank_lp = tgt_lp.to(dt), blank_lp.to(dt)
        # emissions beyond each utterance's own length must not carry mass
        u_idx = torch.arange(U1, device=acts.device)[None, :]
        tgt_lp = tgt_lp.masked_fill((u_idx >= label_lens.long()[:, None])[:, None, :], _NEG)
        skip = self._start_skip()
        entry0 = torch.full((B, U1), _NEG, dtype=dt, device=acts.device)
        entry0[:, 0] = 0.0
        alpha = _row_scan(entry0, tgt_lp[:, 0])
        last_idx = label_lens.long().clamp(max=U1 - 1).unsqueeze(1)
        alpha_last = [alpha.gather(1, last_idx)]
        for t in range(1, T):
            entry = alpha + blank_lp[:, t - 1]
            if skip > _NEG / 2:
                first = torch.logaddexp(entry[:, :1], entry.new_full((B, 1), skip))
                entry = torch.cat([first, entry[:, 1:]], dim=1)
            alpha = _row_scan(entry, tgt_lp[:, t])
            alpha_last.append(alpha.gather(1, last_idx))
        alpha_last = torch.cat(alpha_last, dim=1)                                  # [B, T]
        blank_last = blank_lp.gather(2, last_idx[:, None, :].expand(B, T, 1)).squeeze(2)
        return -self._finish(alpha_last, blank_last, act_lens).float()


class GraphWTransducerLoss(GraphRnntLoss):
    """W-Transducer: RNN-T training when text at the beginning and / or the end of the utterance is missing."""

    def __init__(self, blank: int, eps_weight: float = 0.0, last_blank_mode: str = "force_final", use_grid_implementation: bool = True,
                 connect_composed: bool = False, double_scores: bool = False, cast_to_float32: bool = False):
        super().__init__(blank, use_grid_implementation, connect_composed, double_scores, cast_to_float32)
        if last_blank_mode not in ("force_final", "allow_ignore"):
            raise ValueError(f"last_blank_mode must be 'force_final' or 'allow_ignore', got {last_blank_mode!r}")
        self.eps_weight = float(eps_weight)
        self.last_blank_mode = last_blank_mode

    def _start_skip(self) -> float:
        return self.eps_weight

    def _finish(self, alpha_last, blank_last, act_lens):
        B, T = alpha_last.shape
        t_idx = torch.arange(T, device=alpha_last.device)[None, :]
        last = (act_lens.long() - 1).clamp(min=0)[:, None]
        early = torch.where(t_idx < last, alpha_last + self.eps_weight, alpha_last.new_full((), _NEG))
        skipped = torch.logsumexp(early, dim=1)                                    # leave the transcript's last node early
        a_last, b_last = alpha_last.gather(1, last).squeeze(1), blank_last.gather(1, last).squeeze(1)
        if self.last_blank_mode == "force_final":
            return torch.logaddexp(a_last, skipped) + b_last
        return torch.logaddexp(a_last + b_last, skipped)

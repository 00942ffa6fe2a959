"""More losses of the common collection: latent speaker supervision for serialised multi-speaker transcripts, the multi-similarity
metric-learning loss, and the span (start / end) loss.

References: ``common/losses/latent_speaker_supervision_loss.py``, ``multi_similarity_loss.py``, ``spanning_loss.py``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..core.module import Loss

__all__ = ["LatentSpeakerSupervisionLoss", "MultiSimilarityLoss", "SpanningLoss"]


class LatentSpeakerSupervisionLoss(Loss):
    """Labels carry a speaker token only where the speaker changes (``<spk0> hi how are you <spk1> fine``).  For every word position
    the speaker in charge is the last speaker token seen (forward fill); the model's log-probabilities restricted to the speaker
    tokens, renormalised, are trained against that speaker — speaker supervision at every word without emitting extra tokens.
    ``include_ce_loss`` adds the ordinary (label-smoothed) token cross entropy; ``per_speaker_normalization`` averages the
    auxiliary loss per speaker first, so that a speaker with few words weighs as much as a talkative one."""

    def __init__(self, speaker_token_ids: Sequence[int], speaker_loss_weight: float = 1.0, include_ce_loss: bool = False, pad_id: Optional[int] = None,
                 label_smoothing: float = 0.0, speaker_label_smoothing: float = 0.0, eps: float = 1e-6, per_speaker_normalization: bool = True):
        super().__init__()
        self.register_buffer("speaker_token_ids", torch.tensor(list(speaker_token_ids), dtype=torch.long))
        self.w, self.include_ce, self.pad_id = speaker_loss_weight, include_ce_loss, pad_id
        self.ls, self.sls, self.eps, self.per_spk = label_smoothing, speaker_label_smoothing, eps, per_speaker_normalization

    def active_speakers(self, labels: torch.Tensor) -> torch.Tensor:
        """[B, T] index into ``speaker_token_ids`` of the speaker in charge at every position (-1 before the first speaker token)."""
        is_spk = labels.unsqueeze(-1) == self.speaker_token_ids.to(labels.device)          # [B, T, S]
        idx = torch.where(is_spk.any(-1), is_spk.float().argmax(-1), torch.full_like(labels, -1))
        pos = torch.arange(labels.shape[1], device=labels.device).expand_as(labels)
        last = torch.where(idx >= 0, pos, torch.full_like(pos, -1)).cummax(dim=1).values
        return torch.where(last >= 0, idx.gather(1, last.clamp(min=0)), torch.full_like(idx, -1))

    def forward(self, log_probs: torch.Tensor, labels: torch.Tensor, output_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if output_mask is None:
            output_mask = (labels != self.pad_id) if self.pad_id is not None else torch.ones_like(labels, dtype=torch.bool)
        mask = output_mask.bool()
        spk = self.active_speakers(labels)
        is_spk_tok = (labels.unsqueeze(-1) == self.speaker_token_ids.to(labels.device)).any(-1)
        word = mask & (spk >= 0) & ~is_spk_tok                                   # word positions with a known speaker
        sub = log_probs.float().index_select(-1, self.speaker_token_ids.to(log_probs.device))
        sub = sub - torch.logsumexp(sub, dim=-1, keepdim=True)                   # renormalised over the speaker tokens
        S = sub.shape[-1]
        tgt = F.one_hot(spk.clamp(min=0), S).float()
        if self.sls > 0:
            tgt = tgt * (1 - self.sls) + self.sls / S
        nll = -(tgt * sub).sum(-1)                                                # [B, T]
        if self.per_spk:
            per, n_spk = nll.new_zeros(()), 0
            for s in range(S):
                m = word & (spk == s)
                if bool(m.any()):
                    per = per + nll[m].mean()
                    n_spk += 1
            aux = per / max(1, n_spk)
        else:
            aux = (nll * word).sum() / (word.sum() + self.eps)
        loss = self.w * aux
        if self.include_ce:
            V = log_probs.shape[-1]
            t = F.one_hot(labels.clamp(min=0), V).float()
            if self.ls > 0:
                t = t * (1 - self.ls) + self.ls / V
            ce = -(t * log_probs.float()).sum(-1)
            loss = loss + (ce * mask).sum() / (mask.sum() + self.eps)
        return loss


class MultiSimilarityLoss(Loss):
    """Metric learning on L2-normalised embeddings with class labels: for every anchor the hardest informative pairs are mined
    (negatives more similar than the least similar positive minus ``margin``, positives less similar than the most similar negative
    plus ``margin``) and weighted by soft-plus terms around the threshold ``base``."""

    def __init__(self, scale_pos: float = 2.0, scale_neg: float = 40.0, offset: float = 0.5, margin: float = 0.1):
        super().__init__()
        self.sp, self.sn, self.base, self.margin = scale_pos, scale_neg, offset, margin

    def forward(self, logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        e = F.normalize(logits.float(), dim=-1)
        sim = e @ e.t()
        losses = []
        eps = 1e-5
        for i in range(e.shape[0]):
            same = labels == labels[i]
            pos = sim[i][same & (sim[i] < 1 - eps)]
            neg = sim[i][~same]
            if pos.numel() == 0 or neg.numel() == 0:
                continue
            neg = neg[neg + self.margin > pos.min()]
            pos = pos[pos - self.margin < (neg.max() if neg.numel() else pos.new_tensor(-1.0))]
            if pos.numel() == 0 or neg.numel() == 0:
                continue
            lp = torch.log1p(torch.exp(-self.sp * (pos - self.base)).sum()) / self.sp
            ln = torch.log1p(torch.exp(self.sn * (neg - self.base)).sum()) / self.sn
            losses.append(lp + ln)
        if not losses:
            return logits.sum() * 0.0
        return torch.stack(losses).sum() / e.shape[0]


class SpanningLoss(Loss):
    """Extractive spans: ``logits`` [B, T, 2] (start, end scores per position), positions [B]; the loss is the mean of the start
    and end cross entropies, positions outside the sequence are ignored.  Returns ``(loss, start_logits, end_logits)``."""

    def forward(self, logits: torch.Tensor, start_positions: torch.Tensor, end_positions: torch.Tensor):
        start, end = logits[..., 0], logits[..., 1]
        T = start.shape[1]
        sp, ep = start_positions.clamp(0, T), end_positions.clamp(0, T)
        ls = F.cross_entropy(start.float(), sp, ignore_index=T)
        le = F.cross_entropy(end.float(), ep, ignore_index=T)
        return (ls + le) / 2, start, end

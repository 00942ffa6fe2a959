"""Preference optimisation for MagpieTTS: offline DPO / IPO / RPO on (chosen, rejected) generations and online GRPO with
group-normalised rewards.

Reference: ``tts/models/magpietts_preference_optimization.py`` — ``MagpieTTSModelOfflinePODataGen`` (generate N candidates per
text and score them), ``MagpieTTSModelOfflinePO`` (DPO-style losses between the policy and a frozen reference copy on the codec
token log-likelihoods), ``MagpieTTSModelOnlinePO`` (GRPO: sample a group per prompt, rewards from CER / speaker similarity,
advantages normalised inside the group, clipped policy-gradient loss plus a KL term to the reference).
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from .magpietts import MagpieTTSModel


def sequence_logprob(logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """logits [B, T, C, V], targets [B, T, C], mask [B, T] -> summed log-probability of the target codes per sequence."""
    lp = torch.log_softmax(logits.float(), dim=-1).gather(-1, targets.unsqueeze(-1)).squeeze(-1)      # [B, T, C]
    return (lp.sum(-1) * mask).sum(-1)


def preference_loss(pol_chosen, pol_rejected, ref_chosen, ref_rejected, beta: float = 0.1, loss_type: str = "dpo",
                    chosen_reward: Optional[torch.Tensor] = None, rejected_reward: Optional[torch.Tensor] = None):
    """``dpo``: -log sigmoid(beta * margin); ``ipo``: (margin - 1/(2 beta))^2; ``rpo_sq``: squared error between the implicit
    reward gap and the true reward gap.  margin = (pol_c - ref_c) - (pol_r - ref_r).  Returns (loss, chosen_reward, rejected_reward)
    with the implicit rewards detached (for logging the preference accuracy)."""
    margin = (pol_chosen - ref_chosen) - (pol_rejected - ref_rejected)
    if loss_type == "dpo":
        loss = -F.logsigmoid(beta * margin)
    elif loss_type == "ipo":
        loss = (margin - 1.0 / (2.0 * beta)) ** 2
    elif loss_type == "rpo_sq":
        if chosen_reward is None or rejected_reward is None:
            raise ValueError("rpo_sq needs the true rewards of both candidates")
        loss = (beta * margin - (chosen_reward - rejected_reward)) ** 2
    else:
        raise NotImplementedError(f"loss type {loss_type} is not implemented")
    return loss.mean(), (beta * (pol_chosen - ref_chosen)).detach(), (beta * (pol_rejected - ref_rejected)).detach()


def grpo_advantages(rewards: torch.Tensor, eps: float = 1e-4) -> torch.Tensor:
    """rewards [G, N] (N samples for each of G prompts) -> advantages normalised inside every group."""
    mean, std = rewards.mean(dim=1, keepdim=True), rewards.std(dim=1, keepdim=True, unbiased=False)
    return (rewards - mean) / (std + eps)


def grpo_loss(logp_new: torch.Tensor, logp_old: torch.Tensor, advantages: torch.Tensor, ref_logp: Optional[torch.Tensor] = None,
              clip: float = 0.2, kl_beta: float = 0.0, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sequence-level clipped surrogate: ratio = exp((logp_new - logp_old) / len); loss = -min(r A, clip(r) A) + beta * KL(pol || ref)
    with the k3 estimator of the KL divergence."""
    n = lengths.float().clamp(min=1) if lengths is not None else torch.ones_like(logp_new)
    ratio = torch.exp((logp_new - logp_old.detach()) / n)
    surr = torch.minimum(ratio * advantages, ratio.clamp(1 - clip, 1 + clip) * advantages)
    loss = -surr
    if kl_beta > 0 and ref_logp is not None:
        d = (ref_logp.detach() - logp_new) / n
        loss = loss + kl_beta * (torch.exp(d) - d - 1.0)
    return loss.mean()


class MagpieTTSModelOfflinePO(MagpieTTSModel):
    """Trains on batches ``(text, text_len, chosen_audio, chosen_len, rejected_audio, rejected_len[, chosen_reward, rejected_reward])``."""

    def __init__(self, cfg: DictConfig, trainer=None, codec=None, tokenizer=None):
        super().__init__(cfg, trainer=trainer, codec=codec, tokenizer=tokenizer)
        self.beta = float(cfg_get(self._cfg, "dpo_beta", 0.1))
        self.loss_type = str(cfg_get(self._cfg, "dpo_loss_type", "dpo"))
        self.sft_loss_weight = float(cfg_get(self._cfg, "dpo_sft_loss_weight", 0.0))
        self._reference: Optional[MagpieTTSModel] = None

    def freeze_reference(self) -> None:
        """Snapshot the current weights as the frozen reference policy (call once, after loading the starting checkpoint)."""
        codec, self.codec = self.__dict__.get("codec", None), None
        ref = copy.deepcopy(self).eval()
        self.codec = codec
        ref._reference = None
        for p in ref.parameters():
            p.requires_grad_(False)
        object.__setattr__(self, "_reference", ref)        # kept out of the module tree: not trained, not saved twice

    def _seq_logp(self, model, text, text_len, audio, audio_len):
        codes, codes_len = self.audio_to_codes(audio, audio_len)
        codes, codes_len = self.stack_codes(codes, codes_len)
        logits, _, _, xmask = model.forward(text, text_len, codes, codes_len)
        tgt = codes[:, :, 1:].permute(0, 2, 1)
        return sequence_logprob(logits, tgt, xmask.float()), xmask.sum(1)

    def training_step(self, batch, batch_idx):
        if self._reference is None:
            self.freeze_reference()
        text, text_len, ca, cl, ra, rl = batch[:6]
        pc, n_c = self._seq_logp(self, text, text_len, ca, cl)
        pr, _ = self._seq_logp(self, text, text_len, ra, rl)
        with torch.no_grad():
            self._reference.codec = self.codec
            rc, _ = self._seq_logp(self._reference, text, text_len, ca, cl)
            rr, _ = self._seq_logp(self._reference, text, text_len, ra, rl)
        cr, rj = (batch[6], batch[7]) if len(batch) >= 8 else (None, None)
        loss, rew_c, rew_r = preference_loss(pc, pr, rc, rr, self.beta, self.loss_type, cr, rj)
        if self.sft_loss_weight > 0:
            loss = loss + self.sft_loss_weight * (-(pc / n_c.clamp(min=1)).mean())
        self.log_dict({"train_loss": loss.detach(), "preference_accuracy": (rew_c > rew_r).float().mean()})
        return {"loss": loss}


class MagpieTTSModelOnlinePO(MagpieTTSModelOfflinePO):
    """GRPO: ``generate_group`` samples ``num_generations_per_item`` utterances per text, ``reward_fn(audio, audio_len, texts)``
    scores them (e.g. 1 - CER of an ASR model, speaker similarity), and the policy is updated with the clipped surrogate."""

    def __init__(self, cfg: DictConfig, trainer=None, codec=None, tokenizer=None, reward_fn: Optional[Callable] = None):
        super().__init__(cfg, trainer=trainer, codec=codec, tokenizer=tokenizer)
        self.num_generations = int(cfg_get(self._cfg, "num_generations_per_item", 4))
        self.clip = float(cfg_get(self._cfg, "grpo_clip", 0.2))
        self.kl_beta = float(cfg_get(self._cfg, "grpo_beta", 0.0))
        self.reward_fn = reward_fn

    @torch.no_grad()
    def generate_group(self, text, text_len, **infer_kw):
        was = self.training
        self.eval()
        t = text.repeat_interleave(self.num_generations, dim=0)
        tl = text_len.repeat_interleave(self.num_generations, dim=0)
        audio, audio_len = self.infer_batch(t, tl, **infer_kw)[:2]
        self.train(was)
        return t, tl, audio, audio_len

    def training_step(self, batch, batch_idx):
        text, text_len = batch[:2]
        texts = batch[2] if len(batch) > 2 else None
        t, tl, audio, audio_len = self.generate_group(text, text_len, max_decoder_steps=int(cfg_get(self._cfg, "max_decoder_steps", 100)))
        rewards = torch.as_tensor(self.reward_fn(audio, audio_len, texts), dtype=torch.float32, device=text.device).view(text.shape[0], self.num_generations)
        adv = grpo_advantages(rewards).reshape(-1)
        logp_new, n = self._seq_logp(self, t, tl, audio, audio_len)
        ref = None
        if self.kl_beta > 0:
            if self._reference is None:
                self.freeze_reference()
            with torch.no_grad():
                self._reference.codec = self.codec
                ref, _ = self._seq_logp(self._reference, t, tl, audio, audio_len)
        loss = grpo_loss(logp_new, logp_new.detach(), adv, ref, self.clip, self.kl_beta, n)
        self.log_dict({"train_loss": loss.detach(), "mean_reward": rewards.mean(), "reward_std": rewards.std()})
        return {"loss": loss}

"""Sharded data parallelism over the flat parameter arena.

The reference shards models with PyTorch FSDP2 (``speechlm2/models/salm.py:449-543``, ``docs/source/features/parallelisms.rst``).
With all parameters, gradients and optimizer state in ONE flat arena the same memory saving is a slice operation:

* every rank owns the contiguous slice ``[r * S, (r + 1) * S)`` of the arena (``S`` is a multiple of the arena alignment);
* after backward the flat gradient is reduce-scattered, so a rank receives the summed gradient of its slice only;
* AdamW state (two fp32 moments) exists for the slice only and the fused AdamW kernel updates just that slice;
* the updated fp32 master slice is all-gathered and the bf16 working copy refreshed.

Gradient clipping uses the global norm: local sum of squares of the reduced slice, all-reduced.  Checkpoints stay
world-size independent: ``state_dict()`` gathers the moments, ``load_state_dict()`` re-slices them.
``ShardedGradSync`` is the trainer-side strategy object (parameter broadcast, synchronised BatchNorm, no all-reduce).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..core.optim.fused_adamw import ALIGN, FusedAdamW
from ..utils.logging import logging
from .ddp import GradSync


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def reduce_scatter_flat(flat: torch.Tensor, out: torch.Tensor, group=None) -> None:
    """``out <- sum over ranks of flat[r*S:(r+1)*S]`` for this rank ``r`` (NCCL reduce-scatter; all-reduce + slice elsewhere)."""
    ws, r = _world(group), _rank(group)
    if ws == 1:
        out.copy_(flat[: out.numel()])
        return
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, flat, group=group)
    else:
        tmp = flat.clone()
        dist.all_reduce(tmp, group=group)
        out.copy_(tmp[r * out.numel():(r + 1) * out.numel()])


def all_gather_flat(full: torch.Tensor, shard: torch.Tensor, group=None) -> None:
    ws = _world(group)
    if ws == 1:
        full[: shard.numel()].copy_(shard)
        return
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(full, shard, group=group)
    else:
        dist.all_gather(list(full.chunk(ws)), shard.contiguous(), group=group)


class ShardedFusedAdamW(FusedAdamW):
    def __init__(self, params, group=None, **kw):
        self.group = group
        self.ws, self.rk = _world(group), _rank(group)
        kw["arena_pad_multiple"] = ALIGN * self.ws
        super().__init__(params, **kw)

    def _alloc_state(self) -> None:
        a = self.arena
        self.shard_size = a.numel // self.ws
        self.lo, self.hi = self.rk * self.shard_size, (self.rk + 1) * self.shard_size
        self.exp_avg = torch.zeros(self.shard_size, dtype=torch.float32, device=a.device)
        self.exp_avg_sq = torch.zeros(self.shard_size, dtype=torch.float32, device=a.device)
        self._grad_shard = torch.zeros(self.shard_size, dtype=torch.float32, device=a.device)
        self.grads_already_reduced = False      # set when a gradient all-reduce ran before step()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        from .. import ops

        a = self.arena
        self._step += 1
        if self.grads_already_reduced or self.ws == 1:
            self._grad_shard.copy_(a.grad[self.lo:self.hi])
        else:
            a.grad.div_(self.ws)
            reduce_scatter_flat(a.grad, self._grad_shard, self.group)
        if self.max_grad_norm > 0:
            sq = self._grad_shard.double().pow(2).sum().float().view(1)
            if self.ws > 1:
                dist.all_reduce(sq, group=self.group)
            norm = sq.sqrt() * self.grad_scale
            self._scalars[0] = norm[0]
            self._scalars[1] = self.grad_scale * torch.clamp(self.max_grad_norm / (norm[0] + 1e-6), max=1.0)
            self._scalars[2] = torch.where(torch.isfinite(norm[0]), self._scalars[2], torch.ones_like(self._scalars[2]))
        else:
            self._scalars[1] = self.grad_scale
        for gi, (start, end) in zip(self._nonempty, a.group_ranges):
            s, e = max(start, self.lo), min(end, self.hi)
            if s >= e:
                continue
            g = self.param_groups[gi]
            b1, b2 = g["betas"]
            ls, le = s - self.lo, e - self.lo
            ops.adamw_flat(a.master[s:e], self._grad_shard[ls:le], self.exp_avg[ls:le], self.exp_avg_sq[ls:le], None,
                           lr=float(g["lr"]), beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"], step=self._step,
                           scalars=self._scalars)
        if self.ws > 1:
            all_gather_flat(a.master, a.master[self.lo:self.hi].clone(), self.group)
        a.refresh_lowp()
        return loss

    # ------------------------------------------------------------------ world-size independent checkpoints
    def _gather_state(self, shard: torch.Tensor) -> torch.Tensor:
        full = torch.zeros(self.arena.numel, dtype=shard.dtype, device=shard.device)
        all_gather_flat(full, shard, self.group)
        return full

    def state_dict(self) -> Dict[str, Any]:
        full_m, full_v = self._gather_state(self.exp_avg), self._gather_state(self.exp_avg_sq)
        keep = (self.exp_avg, self.exp_avg_sq)
        self.exp_avg, self.exp_avg_sq = full_m, full_v
        try:
            return super().state_dict()
        finally:
            self.exp_avg, self.exp_avg_sq = keep

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        keep = (self.exp_avg, self.exp_avg_sq)
        self.exp_avg = torch.zeros(self.arena.numel, dtype=torch.float32, device=self.arena.device)
        self.exp_avg_sq = torch.zeros_like(self.exp_avg)
        try:
            super().load_state_dict(state_dict)
            keep[0].copy_(self.exp_avg[self.lo:self.hi])
            keep[1].copy_(self.exp_avg_sq[self.lo:self.hi])
        finally:
            self.exp_avg, self.exp_avg_sq = keep


class ShardedGradSync(GradSync):
    """Trainer strategy for ``ShardedFusedAdamW``: broadcasts the initial parameters and wires synchronised BatchNorm, but
    launches no gradient all-reduce — the optimizer reduce-scatters the flat gradient itself."""

    def __init__(self, model, optimizers, world_size, device, sync_batchnorm: bool = False, **kw):
        super().__init__(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm, **kw)
        self.sharded = [o for o in optimizers if isinstance(o, ShardedFusedAdamW)]
        if not self.sharded:
            logging.warning("strategy 'fsdp' without a sharded optimizer (optim.name: sharded_adamw): gradients are all-reduced "
                            "as in plain data parallelism")

    def mark_ready(self, param):
        if not self.sharded:
            super().mark_ready(param)

    def finish_step(self):
        if not self.sharded:
            return super().finish_step()
        # parameters outside the arena (if any) still need a plain all-reduce
        rest = [p for p in self.params if self.arena is None or id(p) not in self.arena.offsets]
        for p in rest:
            if p.grad is not None:
                p.grad.div_(self.world_size)
                dist.all_reduce(p.grad)

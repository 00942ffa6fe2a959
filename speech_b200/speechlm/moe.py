"""Sparse mixture-of-experts feed-forward block (Qwen3-MoE / Mixtral layout) with expert parallelism.

Every token is routed to ``top_k`` of ``num_experts`` SwiGLU experts; the block's output is the router-weighted sum of the
chosen experts' outputs.  Expert weights are kept stacked (``gate_up [E, 2I, H]``, ``down [E, H, I]``) so that the tokens of
one expert form one contiguous GEMM after a sort by expert ("grouped GEMM" order).

Expert parallelism (``apply_expert_parallel``): rank ``r`` of the group keeps experts ``[r E/W, (r+1) E/W)``.  Forward is
dispatch -> local experts -> combine: token copies are sorted by destination rank, exchanged with one all-to-all of the
per-expert counts and one of the rows, processed, and returned by the mirrored all-to-all; both exchanges are autograd
functions whose backward is the opposite exchange.  The reference obtains the same from Automodel's MoE layers (grouped GEMM
+ token dispatcher) when ``SALMAutomodel`` runs an MoE LLM with an ``ep`` mesh dimension
(``speechlm2/models/salm_automodel.py:721-800``: ``setup_moe_options``, load-balance metrics, aux-loss scaling).

The expert-parallel group is the data-parallel group (every data-parallel rank owns a different slice of the experts).
Gradients of expert-parallel parameters are complete on their owner (every rank's tokens reach it) and must not be averaged
over the data-parallel group; they carry ``_expert_parallel = True`` and a gradient hook divides them by the group size so
that they match the scale of the averaged dense gradients.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn


class _AllToAllRows(torch.autograd.Function):
    """Exchange rows of a ``[N, H]`` tensor: ``send_counts[r]`` consecutive rows go to rank ``r``."""

    @staticmethod
    def forward(ctx, x, send_counts: List[int], recv_counts: List[int], group):
        ctx.group, ctx.send, ctx.recv = group, send_counts, recv_counts
        out = x.new_empty((sum(recv_counts),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


def _all_to_all_rows_by_lists(x, send_counts, recv_counts, group):
    """``all_to_all_single`` where the backend has it, lists of tensors otherwise (both give the same result)."""
    return _AllToAllRows.apply(x, send_counts, recv_counts, group)


class SparseMoEBlock(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int, norm_topk_prob: bool = True,
                 aux_loss_coef: float = 0.0):
        super().__init__()
        self.hidden, self.inner, self.E, self.k = hidden_size, intermediate_size, num_experts, top_k
        self.norm_topk_prob, self.aux_loss_coef = norm_topk_prob, aux_loss_coef
        self.gate = nn.Linear(hidden_size, num_experts, bias=False)
        self.gate_up = nn.Parameter(torch.empty(num_experts, 2 * intermediate_size, hidden_size))
        self.down = nn.Parameter(torch.empty(num_experts, hidden_size, intermediate_size))
        nn.init.normal_(self.gate_up, std=0.02)
        nn.init.normal_(self.down, std=0.02)
        self.ep_group = None
        self.ep_rank, self.ep_size = 0, 1
        self.tp_size = 1                                           # set by the tensor-parallel plan (router gradients are summed over it)
        self.local_first, self.local_n = 0, num_experts
        self.aux_loss: Optional[torch.Tensor] = None            # set by forward in training; the model adds it to its loss
        self.track_load = False
        self.register_buffer("expert_load", torch.zeros(num_experts), persistent=False)

    # ------------------------------------------------------------------ pieces
    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [N, H] -> (weights [N, k], experts [N, k], router probabilities [N, E])."""
        probs = torch.softmax(self.gate(x).float(), dim=-1)
        w, idx = probs.topk(self.k, dim=-1)
        if self.norm_topk_prob:
            w = w / w.sum(dim=-1, keepdim=True)
        return w, idx, probs

    def experts_forward(self, xs: torch.Tensor, counts: List[int], first: int = 0) -> torch.Tensor:
        """``xs``: rows sorted by expert; ``counts[e]`` rows belong to stored expert ``first + e``."""
        out = xs.new_empty(xs.shape)
        o = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            h = F.linear(xs[o:o + n], self.gate_up[first + e].to(xs.dtype))
            g, u = h.chunk(2, dim=-1)
            out[o:o + n] = F.linear(F.silu(g) * u, self.down[first + e].to(xs.dtype))
            o += n
        return out

    def load_balancing_loss(self, probs: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Switch-Transformer auxiliary loss: ``E * sum_e (fraction of routed copies to e) * (mean router probability of e)``;
        1.0 for a uniform router.  Under expert / data parallelism both factors are averaged over the group's tokens."""
        f = torch.zeros(self.E, device=probs.device, dtype=torch.float32).index_add_(
            0, idx.reshape(-1), torch.ones(idx.numel(), device=probs.device))
        n = torch.tensor(float(idx.shape[0]), device=probs.device)
        p = probs.sum(dim=0)
        if self.ep_group is not None:
            stats = torch.cat([f, n.view(1)])
            dist.all_reduce(stats, group=self.ep_group)
            f, n = stats[:-1], stats[-1]
            # the router probabilities carry gradient: the value is the group's sum, the gradient flows through this rank's
            # share, scaled by the group size because data-parallel averaging will divide it again
            p_all = p.detach().clone()
            dist.all_reduce(p_all, group=self.ep_group)
            p = p * self.ep_size + (p_all - p.detach() * self.ep_size)
        return self.E * ((f / (n * self.k)) * (p / n)).sum()

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        N = x2.shape[0]
        w, idx, probs = self.route(x2)
        if self.training and self.aux_loss_coef > 0:
            self.aux_loss = self.aux_loss_coef / self.tp_size * self.load_balancing_loss(probs, idx)
        flat_e = idx.reshape(-1)                                   # [N k] expert of every token copy
        order = flat_e.argsort(stable=True)
        tok = order // self.k
        xs = x2.index_select(0, tok)                               # copies sorted by expert
        counts = torch.bincount(flat_e, minlength=self.E)
        if self.track_load:
            self.expert_load += counts.detach().to(self.expert_load.dtype)
        if self.ep_group is None:
            ys = self.experts_forward(xs, counts.tolist())
        else:
            ys = self._expert_parallel_forward(xs, counts)
        ys = ys * w.reshape(-1)[order].unsqueeze(-1).to(ys.dtype)
        out = torch.zeros_like(x2).index_add_(0, tok, ys)
        return out.view(shape)

    def _expert_parallel_forward(self, xs: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        W, L = self.ep_size, self.local_n
        # counts[e] copies go to the owner of expert e; tell every owner how many rows of each of its experts to expect
        recv_counts = torch.empty_like(counts)                     # [W * L]: from rank r, for my local expert l
        dist.all_to_all_single(recv_counts, counts, group=self.ep_group)
        send = counts.view(W, L).sum(dim=1).tolist()
        recv_mat = recv_counts.view(W, L)
        recv = recv_mat.sum(dim=1).tolist()
        got = _all_to_all_rows_by_lists(xs, send, recv, self.ep_group)      # grouped by source rank, then by local expert
        # regroup by local expert so that each expert runs one GEMM over the rows of all sources
        src_rank = torch.repeat_interleave(torch.arange(W, device=xs.device), torch.tensor(recv, device=xs.device))
        loc = torch.repeat_interleave(torch.arange(L, device=xs.device).repeat(W), recv_mat.reshape(-1))
        perm = (loc * W + src_rank).argsort(stable=True)
        ys = self.experts_forward(got.index_select(0, perm), recv_mat.sum(dim=0).tolist(), first=0)
        back = torch.empty_like(ys).index_copy_(0, perm, ys) if ys.shape[0] else ys
        return _all_to_all_rows_by_lists(back, recv, send, self.ep_group)

    # ------------------------------------------------------------------ checkpoints in the per-expert layout
    def load_per_expert(self, sd: Dict[str, torch.Tensor], prefix: str = "") -> None:
        """``{prefix}experts.{e}.gate_proj.weight`` / ``up_proj`` / ``down_proj`` and ``{prefix}gate.weight`` (the published
        Qwen3-MoE / Mixtral-style layout) into the stacked parameters; under expert parallelism only the local experts are read."""
        with torch.no_grad():
            self.gate.weight.copy_(sd[f"{prefix}gate.weight"])
            for l in range(self.local_n):
                e = self.local_first + l
                self.gate_up[l, : self.inner].copy_(sd[f"{prefix}experts.{e}.gate_proj.weight"])
                self.gate_up[l, self.inner:].copy_(sd[f"{prefix}experts.{e}.up_proj.weight"])
                self.down[l].copy_(sd[f"{prefix}experts.{e}.down_proj.weight"])

    def per_expert_state(self, prefix: str = "") -> Dict[str, torch.Tensor]:
        out = {f"{prefix}gate.weight": self.gate.weight.detach().clone()}
        for l in range(self.local_n):
            e = self.local_first + l
            out[f"{prefix}experts.{e}.gate_proj.weight"] = self.gate_up[l, : self.inner].detach().clone()
            out[f"{prefix}experts.{e}.up_proj.weight"] = self.gate_up[l, self.inner:].detach().clone()
            out[f"{prefix}experts.{e}.down_proj.weight"] = self.down[l].detach().clone()
        return out


def apply_expert_parallel(module: nn.Module, group) -> int:
    """Shard the experts of every :class:`SparseMoEBlock` under ``module`` over ``group`` in place; returns the number of
    blocks changed.  Router weights stay replicated (their gradients are averaged like every dense parameter)."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    n = 0
    for blk in module.modules():
        if not isinstance(blk, SparseMoEBlock) or blk.ep_group is not None:
            continue
        if blk.E % W:
            raise ValueError(f"{blk.E} experts cannot be split over {W} ranks")
        L = blk.E // W
        for name in ("gate_up", "down"):
            full = getattr(blk, name)
            p = nn.Parameter(full.data[r * L:(r + 1) * L].clone(), requires_grad=full.requires_grad)
            p._expert_parallel = True
            p._no_dp_sync = True
            from ..parallel.tp import mark_model_parallel

            mark_model_parallel(p, group, 0, r, W)
            p.register_hook(lambda g, W=W: g / W)
            setattr(blk, name, p)
        blk.ep_group, blk.ep_rank, blk.ep_size, blk.local_first, blk.local_n = group, r, W, r * L, L
        n += 1
    return n


def moe_aux_loss(module: nn.Module) -> Optional[torch.Tensor]:
    """Sum of the auxiliary losses recorded by the MoE blocks in the last forward (``None`` when there is none)."""
    terms = [b.aux_loss for b in module.modules() if isinstance(b, SparseMoEBlock) and b.aux_loss is not None]
    for b in module.modules():
        if isinstance(b, SparseMoEBlock):
            b.aux_loss = None
    return torch.stack(terms).sum() if terms else None


def enable_load_tracking(module: nn.Module, on: bool = True) -> None:
    for b in module.modules():
        if isinstance(b, SparseMoEBlock):
            b.track_load = on
            b.expert_load.zero_()


def collect_expert_loads(module: nn.Module, dp_group=None, reset: bool = True) -> Dict[str, torch.Tensor]:
    """``{block name: tokens routed to each expert since the last call}`` summed over ``dp_group``."""
    out = {}
    for name, b in module.named_modules():
        if isinstance(b, SparseMoEBlock):
            load = b.expert_load.clone()
            if dp_group is not None:
                dist.all_reduce(load, group=dp_group)
            out[name] = load
            if reset:
                b.expert_load.zero_()
    return out


def load_balance_summary(loads: Dict[str, torch.Tensor], top_k: int = 5) -> Dict[str, float]:
    """Brief metrics per model: worst max/mean load ratio over the blocks, mean coefficient of variation, share of idle experts."""
    if not loads:
        return {}
    ratios, cvs, idle = [], [], []
    for v in loads.values():
        m = v.mean().clamp(min=1e-9)
        ratios.append(float(v.max() / m))
        cvs.append(float(v.std(unbiased=False) / m))
        idle.append(float((v == 0).float().mean()))
    return {"moe/max_over_mean_load": max(ratios), "moe/load_cv": sum(cvs) / len(cvs), "moe/idle_expert_fraction": sum(idle) / len(idle)}

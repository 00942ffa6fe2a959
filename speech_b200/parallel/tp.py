"""Tensor and sequence parallelism for transformer blocks.

Column-parallel projections (q / k / v / gate / up) keep a slice of the output features, row-parallel projections (o / down)
a slice of the input features; one reduction per attention / MLP block restores the full activation.  With sequence
parallelism the residual stream is sharded over the sequence between blocks: the block input is all-gathered and the block
output reduce-scattered instead of all-reduced (the plan of the reference's ``salm.py:491-504``: ``SequenceParallel`` norms,
``ColwiseParallel`` q/k/v/gate/up, ``RowwiseParallel`` o/down).

The collectives are differentiable autograd functions over ``torch.distributed`` groups (NCCL on GPUs, gloo in CPU tests).
``PipelinedRowParallel`` overlaps a row-parallel GEMM with its reduction by splitting the rows into chunks: chunk ``i`` is
reduced on the communication stream (by the peer-memory kernel when a symmetric buffer is available) while chunk ``i+1`` is
still in the GEMM.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x


class CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone(), ctx.group), None


class ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel region)."""

    @staticmethod
    def forward(ctx, x, group):
        return _all_reduce(x.clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


def _all_gather_dim(x: torch.Tensor, group, dim: int) -> torch.Tensor:
    ws = dist.get_world_size(group)
    x = x.contiguous()
    if dim == 0 and dist.get_backend(group) == "nccl":
        out = torch.empty((ws * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    parts = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x: torch.Tensor, group, dim: int) -> torch.Tensor:
    """Sum over the group, keep this rank's chunk along ``dim``: a true reduce-scatter on NCCL (each rank receives 1/W of the
    data); gloo has none, so CPU tests reduce everything and slice."""
    ws, r = dist.get_world_size(group), dist.get_rank(group)
    if dist.get_backend(group) == "nccl":
        xs = x.movedim(dim, 0).contiguous()
        out = torch.empty((xs.shape[0] // ws,) + tuple(xs.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, xs, group=group)
        return out.movedim(0, dim).contiguous()
    return _all_reduce(x.clone(), group).chunk(ws, dim=dim)[r].contiguous()


class GatherFromSP(torch.autograd.Function):
    """All-gather along the sequence dim forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _all_gather_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim(g, ctx.group, ctx.dim), None, None


class ReduceScatterToSP(torch.autograd.Function):
    """Reduce-scatter along the sequence dim forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _reduce_scatter_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.group, ctx.dim), None, None


class ScatterToSP(torch.autograd.Function):
    """Keep this rank's chunk of a replicated tensor along ``dim`` (entry of the sequence-parallel region); all-gather backward."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        ws, r = dist.get_world_size(group), dist.get_rank(group)
        return x.chunk(ws, dim=dim)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.group, ctx.dim), None, None


class GatherFromSPReplicated(torch.autograd.Function):
    """All-gather forward; the gathered tensor is consumed identically on every rank (replicated loss), so the backward keeps
    this rank's chunk of the (identical) gradient."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _all_gather_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        ws, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        return g.chunk(ws, dim=ctx.dim)[r].contiguous(), None, None


class FusedColumnParallelFn(torch.autograd.Function):
    """``y = all_gather_rows(x_local) @ w_local^T`` as ONE kernel over peer memory (``parallel.fused.AllGatherGemm``: remote row
    shards are copied once by the GEMM's own idle warps while the tensor pipe works on the local rows), and its backward
    ``dx_local = reduce_scatter_rows(dy @ w_local)`` as ONE kernel too (``GemmReduceScatter``: the epilogue adds every tile into
    the owner rank's accumulator over NVLink).  The weight gradient needs the gathered input once more (NCCL all-gather)."""

    @staticmethod
    def forward(ctx, x_local, weight, bias, ops_pair):
        ag, rs = ops_pair
        from ..ops import lowp

        wl = lowp(weight, torch.bfloat16)
        y = ag(x_local.contiguous(), wl.contiguous(), bias=bias)
        ctx.save_for_backward(x_local)
        ctx.weight, ctx.bias, ctx.pair = weight, bias, ops_pair
        return y

    @staticmethod
    def backward(ctx, dy):
        (x_local,) = ctx.saved_tensors
        ag, rs = ctx.pair
        weight, bias = ctx.weight, ctx.bias
        from ..ops import lowp, native

        wl = lowp(weight, torch.bfloat16).contiguous()        # [N_local, K]
        dy = dy.contiguous()
        # dx [rows, K] = dy [rows, N_local] @ w [N_local, K]: the "weight" of that GEMM is w^T, i.e. w read MN-major
        dx_local = rs(dy, wl.t().contiguous(), out_dtype=torch.bfloat16)
        x_full = _all_gather_dim(x_local, ag.group, 0)
        N, K = wl.shape
        dw = torch.zeros((N, K), dtype=torch.float32, device=dy.device)
        native.gemm(dy, x_full, dw, M=N, N=K, K=dy.shape[0], a_mn=True, lda=dy.stride(0), b_mn=True, ldb=x_full.stride(0), beta=1.0)
        db = dy.float().sum(0) if bias is not None else None
        return dx_local, dw.to(weight.dtype), db, None


class FusedRowParallelFn(torch.autograd.Function):
    """``y_local = reduce_scatter_rows(x @ w_local^T)`` (one GEMM + reduce-scatter kernel) with backward
    ``dx = all_gather_rows(dy_local) @ w_local`` (one all-gather + GEMM kernel)."""

    @staticmethod
    def forward(ctx, x, weight, ops_pair):
        ag, rs = ops_pair
        from ..ops import lowp

        wl = lowp(weight, torch.bfloat16).contiguous()        # [N, K_local]
        y_local = rs(x.contiguous(), wl, out_dtype=torch.bfloat16)
        ctx.save_for_backward(x)
        ctx.weight, ctx.pair = weight, ops_pair
        return y_local

    @staticmethod
    def backward(ctx, dy_local):
        (x,) = ctx.saved_tensors
        ag, rs = ctx.pair
        weight = ctx.weight
        from ..ops import lowp, native

        wl = lowp(weight, torch.bfloat16).contiguous()        # [N, K_local]
        dy_local = dy_local.contiguous()
        # dx [rows, K_local] = gather(dy) [rows, N] @ w [N, K_local]: the GEMM's weight argument is w^T [K_local, N]
        dx = ag(dy_local, wl.t().contiguous())
        dy_full = _all_gather_dim(dy_local, ag.group, 0)
        N, K = wl.shape
        dw = torch.zeros((N, K), dtype=torch.float32, device=x.device)
        native.gemm(dy_full, x, dw, M=N, N=K, K=x.shape[0], a_mn=True, lda=dy_full.stride(0), b_mn=True, ldb=x.stride(0), beta=1.0)
        return dx, dw.to(weight.dtype), None


def mark_model_parallel(p: torch.Tensor, group, dim: int, rank: int, ws: int, gather=None, take=None) -> None:
    """Record how a parameter that holds one slice of a larger tensor relates to the whole: ``p._mp_gather(local) -> full``
    (a collective over ``group``) and ``p._mp_slice(full) -> local``.  Checkpoint code uses the pair to write full tensors and
    to cut this rank's slice out of them again, so files do not depend on the parallel layout."""
    def _gather(local: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(local) for _ in range(ws)]
        dist.all_gather(parts, local.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    def _take(full: torch.Tensor) -> torch.Tensor:
        return full.chunk(ws, dim=dim)[rank].clone()

    p._mp_gather = gather or _gather
    p._mp_slice = take or _take


def mp_full(p: torch.Tensor, local: torch.Tensor) -> torch.Tensor:
    g = getattr(p, "_mp_gather", None)
    return g(local) if g is not None else local


def mp_local(p: torch.Tensor, full: torch.Tensor, local_shape) -> torch.Tensor:
    if tuple(full.shape) == tuple(local_shape):
        return full
    t = getattr(p, "_mp_slice", None)
    if t is None:
        raise ValueError(f"checkpoint tensor of shape {tuple(full.shape)} does not fit a parameter of shape {tuple(local_shape)}")
    out = t(full)
    if tuple(out.shape) != tuple(local_shape):
        raise ValueError(f"slice of shape {tuple(out.shape)} does not fit a parameter of shape {tuple(local_shape)}")
    return out


def _shard_linear(lin: nn.Linear, dim: int, rank: int, ws: int, group=None) -> None:
    """Keep this rank's slice of the weight (dim 0 = output features / column-parallel, 1 = input features / row-parallel)."""
    w = lin.weight.data
    if w.shape[dim] % ws:
        raise ValueError(f"cannot split dimension of size {w.shape[dim]} over {ws} ranks")
    lin.weight = nn.Parameter(w.chunk(ws, dim=dim)[rank].clone(), requires_grad=lin.weight.requires_grad)
    lin.weight._tensor_parallel = True          # one slice of a larger weight: norms and checkpoints treat it as such
    if group is not None:
        mark_model_parallel(lin.weight, group, dim, rank, ws)
    if dim == 0:
        lin.out_features = lin.weight.shape[0]
        if lin.bias is not None:
            lin.bias = nn.Parameter(lin.bias.data.chunk(ws, dim=0)[rank].clone(), requires_grad=lin.bias.requires_grad)
            lin.bias._tensor_parallel = True
            if group is not None:
                mark_model_parallel(lin.bias, group, 0, rank, ws)
    else:
        lin.in_features = lin.weight.shape[1]
        if lin.bias is not None and rank != 0:
            lin.bias.data.zero_()            # the bias is added once, by rank 0's partial sum


def apply_tensor_parallel_llm(llm, group, sequence_parallel: bool = False) -> None:
    """Shard every decoder layer of ``speechlm.llm.CausalLM`` over ``group`` in place.

    ``sequence_parallel``: the residual stream between blocks is sharded along the sequence (dim 1): the embeddings are
    scattered on entry, every norm works on its shard, the normalised shard is all-gathered in front of the column-parallel
    projections, the row-parallel projections end in a reduce-scatter, and the final hidden states are gathered in front of the
    output head (the reference's plan: ``salm.py:459-532``, ``SequenceParallel`` norms, ``Colwise`` / ``Rowwise`` linears)."""
    ws, r = dist.get_world_size(group), dist.get_rank(group)
    if ws == 1:
        return
    cfg = llm.config
    if cfg.num_attention_heads % ws or cfg.num_key_value_heads % ws:
        raise ValueError(f"heads ({cfg.num_attention_heads} / {cfg.num_key_value_heads}) are not divisible by tp={ws}")
    for layer in llm.model.layers:
        att, mlp = layer.self_attn, layer.mlp
        dense = hasattr(mlp, "gate_proj")
        for lin in (att.q_proj, att.k_proj, att.v_proj) + ((mlp.gate_proj, mlp.up_proj) if dense else ()):
            _shard_linear(getattr(lin, "base", lin), 0, r, ws, group)
        for lin in (att.o_proj,) + ((mlp.down_proj,) if dense else ()):
            _shard_linear(getattr(lin, "base", lin), 1, r, ws, group)
        if not dense:
            _shard_experts_inner(mlp, r, ws, group)
        att.n_q, att.n_kv = cfg.num_attention_heads // ws, cfg.num_key_value_heads // ws
        if sequence_parallel:
            layer.tp_reduce = (lambda x, g=group: ReduceScatterToSP.apply(x, g, 1))
            for norm in (layer.input_layernorm, layer.post_attention_layernorm):
                fwd = norm.forward
                norm.forward = (lambda x, f=fwd, g=group: GatherFromSP.apply(f(x), g, 1))
                for p in norm.parameters():
                    _sum_grad_over_group(p, group)    # gradients of shard-wise norms are partial: summed over the group
        else:
            layer.tp_reduce = (lambda x, g=group: ReduceFromTP.apply(x, g))
            _wrap_inputs(layer, group)
        # per-head norms of queries / keys are replicated weights that see only this rank's heads
        for name in ("q_norm", "k_norm"):
            nm = getattr(att, name, None)
            if isinstance(nm, nn.Module):
                for p in nm.parameters():
                    _sum_grad_over_group(p, group)
    if sequence_parallel:
        llm.model.sp_scatter = (lambda x, g=group: ScatterToSP.apply(x, g, 1))
        llm.model.sp_gather = (lambda x, g=group: GatherFromSPReplicated.apply(x, g, 1))
        for p in llm.model.norm.parameters():
            _sum_grad_over_group(p, group)


def apply_context_parallel_llm(llm, group) -> None:
    """Context parallelism for ``speechlm.llm.CausalLM``: every rank of ``group`` carries a contiguous ``T / W`` slice of the
    sequence through the blocks; each attention module all-gathers keys and values along time (backward: reduce-scatter of their
    gradients) and attends with its local queries under the causal / packed-sequence mask of the full sequence.  Parameter
    gradients cover the local tokens only, so the group is part of the gradient-averaging group, like data parallelism."""
    if dist.get_world_size(group) == 1:
        return
    for layer in llm.model.layers:
        layer.self_attn.cp_gather = (lambda t, g=group: GatherFromSP.apply(t.contiguous(), g, 2))
    llm.model.cp_group = group


def _shard_experts_inner(blk, rank: int, ws: int, group) -> None:
    """Mixture-of-experts block under tensor parallelism: every expert's inner dimension is split (gate and up halves alike),
    so each rank produces a partial sum of every expert's output and the usual reduction after the block completes it.  The
    router is replicated and routes identically on all ranks; its gradient arrives through the partial outputs and is summed."""
    E, I, H = blk.E, blk.inner, blk.hidden
    if I % ws:
        raise ValueError(f"expert inner size {I} is not divisible by tp={ws}")
    gu = blk.gate_up.data.view(E, 2, I, H).chunk(ws, dim=2)[rank].reshape(E, 2 * (I // ws), H).clone()
    dn = blk.down.data.chunk(ws, dim=2)[rank].clone()
    blk.gate_up = nn.Parameter(gu, requires_grad=blk.gate_up.requires_grad)
    blk.down = nn.Parameter(dn, requires_grad=blk.down.requires_grad)
    blk.gate_up._tensor_parallel = blk.down._tensor_parallel = True

    def gather_gu(local):            # [E, 2 I/W, H] slices -> [E, 2 I, H] with the gate and up halves kept apart
        parts = [torch.empty_like(local) for _ in range(ws)]
        dist.all_gather(parts, local.contiguous(), group=group)
        return torch.cat([q.view(E, 2, I // ws, H) for q in parts], dim=2).reshape(E, 2 * I, H)

    mark_model_parallel(blk.gate_up, group, 1, rank, ws, gather=gather_gu,
                        take=lambda full: full.view(E, 2, I, H).chunk(ws, dim=2)[rank].reshape(E, 2 * (I // ws), H).clone())
    mark_model_parallel(blk.down, group, 2, rank, ws)
    blk.inner = I // ws
    blk.tp_size = ws              # the auxiliary loss is the same on every rank: scaled so that the summed router gradient counts it once
    _sum_grad_over_group(blk.gate.weight, group)


def clip_grad_norm_mesh(params, max_norm: float, tp_group=None, dp_shard_group=None, sharded=lambda p: False) -> torch.Tensor:
    """Global-norm clipping on a mesh.  A parameter tagged ``_tensor_parallel`` is one slice of a weight split over
    ``tp_group``: its squared norm is summed over that group.  A parameter for which ``sharded(p)`` holds is a slice over
    ``dp_shard_group`` and is summed there.  All other parameters are replicas and count once, so that every rank arrives at
    the same norm (the reference groups DTensor gradients by mesh and placement to the same end, ``salm_automodel.py:551-567``)."""
    params = [p for p in params if p.grad is not None]
    if not params:
        return torch.zeros(())
    dev = params[0].grad.device
    sq = {"rep": torch.zeros((), device=dev, dtype=torch.float32), "tp": torch.zeros((), device=dev, dtype=torch.float32),
          "dp": torch.zeros((), device=dev, dtype=torch.float32), "tpdp": torch.zeros((), device=dev, dtype=torch.float32)}
    for p in params:
        key = ("tp" if getattr(p, "_tensor_parallel", False) else "") + ("dp" if sharded(p) else "") or "rep"
        sq[key] += p.grad.detach().float().pow(2).sum()
    if tp_group is not None:
        buf = torch.stack([sq["tp"], sq["tpdp"]])
        dist.all_reduce(buf, group=tp_group)
        sq["tp"], sq["tpdp"] = buf[0], buf[1]
    if dp_shard_group is not None:
        buf = torch.stack([sq["dp"], sq["tpdp"]])
        dist.all_reduce(buf, group=dp_shard_group)
        sq["dp"], sq["tpdp"] = buf[0], buf[1]
    norm = (sq["rep"] + sq["tp"] + sq["dp"] + sq["tpdp"]).sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad.dtype))
    return norm


def _sum_grad_over_group(p: nn.Parameter, group) -> None:
    """A replicated parameter whose gradient on each rank covers only part of the work (a sequence shard, this rank's heads):
    the incoming gradient of every backward pass is summed over ``group`` before it is accumulated, so gradient accumulation
    and sharded optimizers that consume gradients inside backward both see the full gradient."""
    if getattr(p, "_partial_grad_group", None) is not None:
        return
    p._partial_grad_group = group
    p._sequence_parallel = True

    def hook(g, group=group):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=group)
        return g
    p.register_hook(hook)


def allreduce_sequence_parallel_grads(module: nn.Module, group) -> None:
    """Sum partial gradients of replicated parameters over the tensor-parallel group after backward.  Parameters prepared by
    :func:`apply_tensor_parallel_llm` do this themselves in a gradient hook and are skipped; the call remains for modules
    whose parameters were tagged ``_sequence_parallel`` by hand."""
    for p in module.parameters():
        if getattr(p, "_sequence_parallel", False) and getattr(p, "_partial_grad_group", None) is None and p.grad is not None:
            dist.all_reduce(p.grad, group=group)


def _wrap_inputs(layer, group) -> None:
    """Mark the (replicated) normalised activations entering the column-parallel projections so that their gradients are
    summed over the group."""
    for norm in (layer.input_layernorm, layer.post_attention_layernorm):
        fwd = norm.forward
        norm.forward = (lambda x, f=fwd, g=group: CopyToTP.apply(f(x), g))


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, group, bias: bool = True, gather_output: bool = False):
        super().__init__()
        ws = dist.get_world_size(group)
        self.group, self.gather_output = group, gather_output
        self.linear = nn.Linear(in_features, out_features // ws, bias=bias)

    def forward(self, x):
        y = self.linear(CopyToTP.apply(x, self.group))
        return GatherFromSP.apply(y, self.group, -1) if self.gather_output else y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, group, bias: bool = True):
        super().__init__()
        ws = dist.get_world_size(group)
        self.group = group
        self.linear = nn.Linear(in_features // ws, out_features, bias=False)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x):
        y = ReduceFromTP.apply(self.linear(x), self.group)
        return y + self.bias if self.bias is not None else y


def vocab_parallel_cross_entropy(local_logits: torch.Tensor, targets: torch.Tensor, group, ignore_index: int = -100) -> torch.Tensor:
    """Cross entropy when the vocabulary dimension of the logits is sharded over ``group`` (the reference runs its loss under
    ``loss_parallel()``, ``salm.py:221-230``).  Per-token losses; ignored positions give 0."""
    ws, r = dist.get_world_size(group), dist.get_rank(group)
    Vl = local_logits.shape[-1]
    lo = r * Vl
    x = local_logits.float()
    m = x.max(dim=-1).values.detach()
    m_all = m.clone()
    dist.all_reduce(m_all, op=dist.ReduceOp.MAX, group=group)
    se = torch.exp(x - m_all.unsqueeze(-1)).sum(-1)
    se = ReduceFromTP.apply(se, group)
    inside = (targets >= lo) & (targets < lo + Vl)
    idx = (targets - lo).clamp(min=0, max=Vl - 1)
    tgt = torch.where(inside, x.gather(-1, idx.unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
    tgt = ReduceFromTP.apply(tgt, group)
    loss = torch.log(se) + m_all - tgt
    return torch.where(targets == ignore_index, torch.zeros_like(loss), loss)


class PipelinedRowParallel:
    """``y = reduce(x @ W_local^T)`` with the reduction of row-chunk ``i`` overlapping the GEMM of chunk ``i+1``.

    ``reducer(flat_fp32)`` is an in-place all-reduce on the current stream (for instance ``parallel.symm.PeerAllReduce``);
    without one, NCCL's asynchronous all-reduce is used.  Forward only (inference / frozen layers)."""

    def __init__(self, group, chunks: int = 4, reducer: Optional[Callable[[torch.Tensor], None]] = None):
        self.group, self.chunks, self.reducer = group, chunks, reducer
        self.comm = torch.cuda.Stream() if torch.cuda.is_available() else None

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        from .. import ops

        rows = x.reshape(-1, x.shape[-1])
        outs, works = [], []
        for part in rows.chunk(self.chunks, dim=0):
            y = ops.linear(part, weight, None).float()
            if self.comm is not None and x.is_cuda:
                self.comm.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm):
                    if self.reducer is not None:
                        self.reducer(y.view(-1))
                    else:
                        works.append(dist.all_reduce(y, group=self.group, async_op=True))
                y.record_stream(self.comm)
            else:
                dist.all_reduce(y, group=self.group)
            outs.append(y)
        for w in works:
            w.wait()
        if self.comm is not None and x.is_cuda:
            torch.cuda.current_stream().wait_stream(self.comm)
        return torch.cat(outs, dim=0).reshape(*x.shape[:-1], weight.shape[0]).to(x.dtype)

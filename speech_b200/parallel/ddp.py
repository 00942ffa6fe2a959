"""Data-parallel gradient exchange owned by the framework.

The reference wraps models in Lightning's ``DDPStrategy`` (bucketed NCCL all-reduce inside PyTorch's c10d
reducer, 25 MB buckets, overlapped with backward; ``docs/source/features/parallelisms.rst:10-40``) and turns
BatchNorm into ``SyncBatchNorm`` (``examples/asr/conf/fastconformer/fast-conformer_transducer_bpe.yaml:263``).
Here the exchange is a strategy object the trainer calls:

* ``GradSync`` — bucketed all-reduce of gradients through ``torch.distributed`` (gloo on CPU, NCCL on GPUs).
  With the flat optimizer arena the buckets are slices of one buffer, so there is no flatten / unflatten copy.
  Buckets are launched as soon as every gradient in them is final (signalled by the ops' backward or by
  post-accumulate hooks) on a side stream, overlapping the rest of backward.  This is the *baseline* path.
* ``PeerGradSync`` — the same bucket protocol where each bucket is reduced by a hand-written kernel over
  NVLink peer memory (cast to bf16 + scale into a symmetric buffer, reduce-scatter by peer loads, all-gather
  by peer stores), see ``speech_b200.parallel.symm``.
* synchronised BatchNorm statistics and other tiny reductions ride ``small_allreduce``.

Initial parameter values are broadcast from rank 0 so that all ranks start identical.
"""
from __future__ import annotations

import contextlib
import os
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.logging import logging

DEFAULT_BUCKET_MB = 25


def small_allreduce(t: torch.Tensor, op=None) -> torch.Tensor:
    """All-reduce a tiny tensor (statistics, flags, lengths); differentiable for SUM via a custom function."""
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return t
    return _AllReduceSum.apply(t) if (op is None and t.requires_grad) else _plain_allreduce(t, op)


def _plain_allreduce(t, op=None):
    buf = t.detach().clone()
    if dist.get_backend() != "nccl" and buf.is_cuda:
        cpu = buf.cpu()
        dist.all_reduce(cpu, op=op or dist.ReduceOp.SUM)
        return cpu.to(buf.device)
    dist.all_reduce(buf, op=op or dist.ReduceOp.SUM)
    return buf


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _plain_allreduce(x)

    @staticmethod
    def backward(ctx, g):
        return _plain_allreduce(g)


class GradSync:
    def __init__(self, model: torch.nn.Module, optimizers, world_size: int, device: torch.device,
                 bucket_mb: float = DEFAULT_BUCKET_MB, sync_batchnorm: bool = False, grad_dtype: Optional[torch.dtype] = None,
                 group=None):
        """``group``: the process group gradients are averaged over (default: all ranks).  On a device mesh it is the
        data-parallel group; ``world_size`` is then that group's size."""
        self.model, self.world_size, self.device = model, world_size, device
        self.group = group
        self._src = dist.get_global_rank(group, 0) if group is not None else 0
        self.arena = next((o.arena for o in optimizers if hasattr(o, "arena")), None)
        # parameters tagged ``_no_dp_sync`` (expert-parallel experts: every rank owns different ones) stay out of the exchange
        self.params = [p for p in model.parameters() if p.requires_grad and not getattr(p, "_no_dp_sync", False)]
        if self.arena is not None and any(getattr(p, "_no_dp_sync", False) and id(p) in self.arena.offsets for p in model.parameters()):
            raise ValueError("expert-parallel parameters cannot live in the flat optimizer arena, which is exchanged as a whole: "
                             "set `fused_optimizer: false` (or another optim.name) for models with expert parallelism")
        self.bucket_bytes = int(bucket_mb * 1024 * 1024)
        self._sync_enabled = True
        self._works: List[Any] = []
        self.comm_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._broadcast_parameters()
        if sync_batchnorm:
            self.enable_sync_batchnorm()
        self._build_buckets()

    # ------------------------------------------------------------------ setup
    def _broadcast_parameters(self):
        with torch.no_grad():
            if self.arena is not None:
                dist.broadcast(self.arena.master, self._src, group=self.group)
                self.arena.refresh_lowp()
                rest = [p for p in self.model.parameters() if id(p) not in self.arena.offsets]
            else:
                rest = list(self.model.parameters())
            rest = [p for p in rest if not getattr(p, "_no_dp_sync", False)]
            for t in rest + list(self.model.buffers()):
                if t.is_floating_point() or t.dtype in (torch.long, torch.int):
                    dist.broadcast(t.data, self._src, group=self.group)

    def enable_sync_batchnorm(self):
        """Conformer conv modules reduce their BatchNorm sums over all ranks (one small all-reduce per layer)."""
        n = 0
        for m in self.model.modules():
            if hasattr(m, "bn_stats_reduce"):
                m.bn_stats_reduce = small_allreduce
                n += 1
        for name, m in self.model.named_modules():
            if isinstance(m, torch.nn.modules.batchnorm._BatchNorm) and self.device.type == "cuda":
                pass  # plain torch BatchNorm layers outside the fused conv module keep local statistics
        logging.info(f"synchronised BatchNorm statistics enabled on {n} conv modules")

    def _build_buckets(self):
        """Buckets in reverse parameter order (the order gradients become ready in backward)."""
        self.buckets: List[Dict[str, Any]] = []
        if self.arena is not None:
            a = self.arena
            elems = max(1, self.bucket_bytes // 4)
            end = a.numel
            # walk parameters backwards, cutting whenever the slice reaches the bucket size
            plist = sorted(a.params, key=lambda p: a.offsets[id(p)][0], reverse=True)
            cur_end, cur_params = end, []
            for p in plist:
                o, n = a.offsets[id(p)]
                cur_params.append(p)
                if cur_end - o >= elems:
                    self.buckets.append({"start": o, "end": cur_end, "params": cur_params})
                    cur_end, cur_params = o, []
            if cur_params:
                self.buckets.append({"start": 0, "end": cur_end, "params": cur_params})
            for b in self.buckets:
                b["view"] = a.grad[b["start"]:b["end"]]
            rest = [p for p in self.params if id(p) not in a.offsets]
        else:
            rest = self.params
        cur, size = [], 0
        for p in reversed(rest):
            cur.append(p)
            size += p.numel() * 4
            if size >= self.bucket_bytes:
                self.buckets.append({"params": cur, "view": None})
                cur, size = [], 0
        if cur:
            self.buckets.append({"params": cur, "view": None})
        self._bucket_of = {}
        for bi, b in enumerate(self.buckets):
            for p in b["params"]:
                self._bucket_of[id(p)] = bi
        self._hooks = []
        if self.arena is not None:
            # kernels that write a gradient straight into the arena report it here (autograd hooks do not fire for them)
            self.arena.grad_ready = self.mark_ready
        for p in self.params:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(p)))

    def _make_hook(self, p):
        def hook(param):
            self.mark_ready(param)

        return hook

    # ------------------------------------------------------------------ step protocol
    def begin_step(self):
        self._pending = [{id(p) for p in b["params"]} for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._complete = [False] * len(self.buckets)
        self._next = 0          # buckets are launched strictly in index order, the same order on every rank
        self._works = []
        self.launched_in_backward = 0

    @contextlib.contextmanager
    def no_sync(self):
        prev = self._sync_enabled
        self._sync_enabled = False
        try:
            yield
        finally:
            self._sync_enabled = prev

    def mark_ready(self, param):
        """Called when ``param``'s gradient for this step is final."""
        if not self._sync_enabled or not hasattr(self, "_pending"):
            return
        bi = self._bucket_of.get(id(param))
        if bi is None or self._launched[bi]:
            return
        self._pending[bi].discard(id(param))
        if not self._pending[bi]:
            self._complete[bi] = True
            # Launch only the consecutive prefix of complete buckets.  The order in which gradients become final may differ
            # between ranks (a parameter unused on one rank, conditional heads); the collective of launch k must nevertheless
            # pair the same bucket on every rank, as c10d's reducer guarantees with its fixed bucket order.
            while self._next < len(self.buckets) and self._complete[self._next]:
                self._launch(self._next)
                self._next += 1
                self.launched_in_backward += 1

    def _launch(self, bi: int):
        self._launched[bi] = True
        b = self.buckets[bi]
        if b["view"] is not None:
            self._reduce_flat(b["view"])
        else:
            grads = [p.grad for p in b["params"] if p.grad is not None]
            if grads:
                flat = torch.cat([g.reshape(-1) for g in grads])
                self._reduce_flat(flat)
                b["_unflatten"] = (flat, grads)

    def _reduce_flat(self, flat: torch.Tensor):
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.comm_stream):
                flat.div_(self.world_size)
                w = dist.all_reduce(flat, async_op=True, group=self.group)
        else:
            flat.div_(self.world_size)
            w = dist.all_reduce(flat, async_op=True, group=self.group)
        self._works.append(w)

    def finish_step(self):
        """Launch whatever has not been launched (unused parameters), wait for all buckets."""
        for bi in range(self._next, len(self.buckets)):
            if not self._launched[bi]:
                self._launch(bi)
        self._next = len(self.buckets)
        for w in self._works:
            w.wait()
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        for b in self.buckets:
            uf = b.pop("_unflatten", None)
            if uf is not None:
                flat, grads = uf
                off = 0
                for g in grads:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
        self._works = []


def build_grad_sync(model, optimizers, strategy_spec, world_size: int, device: torch.device, sync_batchnorm: bool = False):
    if world_size <= 1 or not dist.is_initialized():
        return None
    kind = strategy_spec if isinstance(strategy_spec, str) else getattr(strategy_spec, "kind", "auto")
    if any(type(o).__name__ == "FullyShardedAdamW" for o in optimizers):
        # a fully-sharded optimizer brings its own gradient path (reduce-scatter per unit), whatever the strategy string says
        from .fsdp2 import FSDP2GradSync

        return FSDP2GradSync(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm)
    if kind in ("auto", "ddp", "ddp_find_unused_parameters_true", "nccl"):
        use_peer = device.type == "cuda" and os.environ.get("SPEECH_B200_PEER_ALLREDUCE", "1") == "1"
        if use_peer and kind != "nccl":
            from .symm import PeerGradSync

            if os.environ.get("SPEECH_B200_PEER_ALLREDUCE_STRICT", "0") == "1":
                return PeerGradSync(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm)
            try:
                return PeerGradSync(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm)
            except Exception as e:  # noqa: BLE001
                logging.warning(f"peer-memory gradient exchange unavailable ({e}); using NCCL all-reduce")
        return GradSync(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm)
    if kind in ("fsdp", "fsdp2", "zero", "sharded"):
        from .fsdp import ShardedGradSync

        return ShardedGradSync(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm)
    if hasattr(strategy_spec, "build_grad_sync"):
        return strategy_spec.build_grad_sync(model, optimizers, world_size, device)
    raise ValueError(f"unknown strategy {strategy_spec}")

"""Fully-sharded data parallelism (ZeRO-3): parameters, gradients and optimizer state exist as 1/W slices per rank.

The reference applies PyTorch FSDP2 ``fully_shard`` per transformer layer and once on the root
(``nemo/collections/speechlm2/models/salm.py:534-543``, ``docs/source/features/parallelisms.rst``).  The same unit structure is used
here on flat buffers:

* a **unit** is a module whose parameters are gathered and freed together (every Conformer / Transformer layer), plus one
  *root* unit for everything else (front end, embeddings, heads), which stays gathered for the whole step;
* every unit's parameters are laid out contiguously and padded so that they split into ``W`` equal slices.  Rank ``r`` owns
  slice ``r`` of every unit: fp32 master weights, both AdamW moments, the reduced fp32 gradient (only with global clipping) and a
  bf16 working copy of the slice.  On GPUs the bf16 slices live in a symmetric buffer every rank can address;
* before a unit's forward, and again before its backward, the full bf16 parameters are gathered into one of two pooled buffers
  (``csrc/peer_fsdp.cu``: plain peer loads, up-cast to an fp32 image for ``parameter.data`` in the same pass); the next unit in
  execution order is prefetched on the communication stream while the current one computes.  After the unit's forward /
  backward the pool slot is simply reused: nothing is kept;
* a unit's fp32 gradients are produced into one of two pooled gradient buffers.  When all of them are final (the same
  per-parameter readiness protocol as the data-parallel engine, ``parallel/ddp.py``) one kernel pair reduces them: each rank
  packs its unit gradient to bf16 in its symmetric gradient buffer, then sums ITS slice over all ranks by peer loads and
  either applies AdamW to its master / moment slices on the spot (no global clipping: the update is finished when backward
  is) or stores the reduced slice and its sum of squares for a clipped update in ``step()``.

Without a CUDA device (tests, gloo) the same protocol runs on ``torch.distributed`` collectives in fp32.
Peak memory per rank: ``(4 + 8 + 2 [+ 4]) * P / W`` bytes persistent plus two parameter and two gradient pool slots of the
largest unit; ``memory_report()`` prints the figures next to the replicated ``16 * P + 2 * P``.
"""
from __future__ import annotations

import ctypes
import math
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.optim.optimizer import Optimizer

from ..utils.logging import logging

ALIGN = 128


class SbFsdpArgs(ctypes.Structure):
    _fields_ = [("grad_bufs", ctypes.c_void_p), ("buf_off", ctypes.c_longlong), ("flags_off", ctypes.c_longlong),
                ("slice", ctypes.c_longlong), ("rank", ctypes.c_int), ("world", ctypes.c_int), ("ctas", ctypes.c_int),
                ("epoch", ctypes.c_uint), ("status", ctypes.c_void_p), ("grad_shard", ctypes.c_void_p), ("sumsq", ctypes.c_void_p),
                ("master", ctypes.c_void_p), ("exp_avg", ctypes.c_void_p), ("exp_avg_sq", ctypes.c_void_p),
                ("lowp_shard", ctypes.c_void_p), ("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("wd", ctypes.c_float), ("bc1", ctypes.c_float), ("rsqrt_bc2", ctypes.c_float),
                ("mode", ctypes.c_int)]


def default_units(model: torch.nn.Module) -> List[torch.nn.Module]:
    """Every element of a ``ModuleList`` named ``layers`` (Conformer, Transformer and LLM stacks) is a unit."""
    units = []
    for name, m in model.named_modules():
        if isinstance(m, torch.nn.ModuleList) and name.split(".")[-1] in ("layers", "blocks", "h"):
            units.extend(list(m))
    return units


class _Unit:
    def __init__(self, index: int, module: Optional[torch.nn.Module], params: List[torch.nn.Parameter], world: int):
        self.index, self.module, self.params = index, module, params
        self.offsets: Dict[int, Tuple[int, int]] = {}
        off = 0
        for p in params:
            n = p.numel()
            self.offsets[id(p)] = (off, n)
            off += (n + ALIGN - 1) // ALIGN * ALIGN
        step = ALIGN * world
        self.numel = max(step, (off + step - 1) // step * step)
        self.slice = self.numel // world
        self.gathered = False
        self.slot = None                 # pool slot currently holding the gathered parameters
        self.gslot = None                # gradient pool slot of the running backward
        self.shard_base = 0              # offset of this unit's slice inside the rank's flat shard buffers


class FullyShardedAdamW(Optimizer):
    """AdamW over 1/W slices; owns the sharded storage and drives gather / reduce-scatter for ``FSDP2GradSync``."""

    def __init__(self, model: torch.nn.Module, units: Optional[Sequence[torch.nn.Module]] = None, lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 1e-2, max_grad_norm: float = 0.0, group=None, device=None, ctas: int = 12,
                 gather_blocks: int = 32, replicate_group=None):
        """``group``: the ranks a unit is sharded over (default: all).  ``replicate_group``: hybrid sharding (HSDP) — ranks that
        hold the SAME slice in different shard groups; their reduced gradient slices are averaged before the update, which
        then runs in ``step()`` on every replica identically."""
        params = [p for p in model.parameters() if p.requires_grad]
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else params[0].device
        self.cuda = self.device.type == "cuda"
        self.max_grad_norm = float(max_grad_norm or 0.0)
        self.replicate_group = replicate_group
        self.replicas = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.ctas, self.gather_blocks = int(ctas), int(gather_blocks)
        self._step = 0
        self._shapes = {id(p): tuple(p.shape) for p in params}
        # ---- units
        unit_modules = list(units) if units is not None else default_units(model)
        claimed: Dict[int, int] = {}
        self.units: List[_Unit] = []
        for m in unit_modules:
            ps = [p for p in m.parameters() if p.requires_grad and id(p) not in claimed]
            if not ps:
                continue
            u = _Unit(len(self.units), m, ps, self.world)
            for p in ps:
                claimed[id(p)] = u.index
            self.units.append(u)
        rest = [p for p in params if id(p) not in claimed]
        self.root = _Unit(len(self.units), None, rest, self.world) if rest else None
        all_units = self.units + ([self.root] if self.root is not None else [])
        self.all_units = all_units
        self.unit_of = {id(p): u for u in all_units for p in u.params}
        base = 0
        for u in all_units:
            u.shard_base = base
            base += u.slice
        self.shard_numel = base
        self.total_numel = sum(p.numel() for p in params)
        dev = self.device
        # ---- persistent slices
        self.master = torch.zeros(base, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(base, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(base, dtype=torch.float32, device=dev)
        self.deferred_update = self.max_grad_norm > 0 or self.replicas > 1       # the update waits for step()
        self.grad_shard = torch.zeros(base, dtype=torch.float32, device=dev) if (self.deferred_update or not self.cuda or self.world == 1) else None
        self._scalars = torch.zeros(4, dtype=torch.float32, device=dev)
        self._setup_comm(base)
        # ---- pools: two parameter slots and two gradient slots of the largest unit, dedicated buffers for the root
        big = max((u.numel for u in self.units), default=ALIGN)
        self.lowp_dtype = torch.bfloat16 if self.cuda else None
        self.pool_f32 = [torch.zeros(big, dtype=torch.float32, device=dev) for _ in range(2)]
        self.pool_lowp = [torch.zeros(big, dtype=torch.bfloat16, device=dev) for _ in range(2)] if self.cuda else [None, None]
        self.pool_grad = [torch.zeros(big, dtype=torch.float32, device=dev) for _ in range(2)]
        self.pool_owner: List[Optional[_Unit]] = [None, None]
        if self.root is not None:
            self.root_f32 = torch.zeros(self.root.numel, dtype=torch.float32, device=dev)
            self.root_lowp = torch.zeros(self.root.numel, dtype=torch.bfloat16, device=dev) if self.cuda else None
            self.root_grad = torch.zeros(self.root.numel, dtype=torch.float32, device=dev)
        self.comm_stream = torch.cuda.Stream(device=dev) if self.cuda else None
        self._pool_free_event: List[Optional[Any]] = [None, None]
        self._gpool_free_event: List[Optional[Any]] = [None, None]
        # ---- take the parameters: slices of the initial values become the master shards; parameter.data is re-pointed on gather
        with torch.no_grad():
            for u in all_units:
                flat = torch.zeros(u.numel, dtype=torch.float32, device=dev)
                for p in u.params:
                    o, n = u.offsets[id(p)]
                    flat[o:o + n].copy_(p.data.reshape(-1).to(dev))
                if self.world > 1:
                    dist.broadcast(flat, dist.get_global_rank(group, 0) if group is not None else 0, group=group)   # start from the group's first rank
                self.master[u.shard_base:u.shard_base + u.slice].copy_(flat[self.rank * u.slice:(self.rank + 1) * u.slice])
                for p in u.params:
                    p.data = torch.empty(0, dtype=torch.float32, device=dev)   # nothing is replicated while a unit is not gathered
        self._refresh_lowp_shards()
        self._install_hooks()
        if self.root is not None:
            self._gather(self.root)

    # ------------------------------------------------------------------ communication back ends
    def _setup_comm(self, shard_numel: int) -> None:
        self.param_buf = self.grad_buf = None
        if self.cuda and self.world > 1:
            from ..ops import native
            from .symm import SymmetricBuffer

            self.native = native
            lib = native.lib()
            lib.sb_fsdp_flags_bytes.restype = ctypes.c_longlong
            self.flags_bytes = int(lib.sb_fsdp_flags_bytes())
            self.param_buf = SymmetricBuffer(shard_numel * 2, self.device, self.group)
            self.lowp_shard = self.param_buf.tensor[: shard_numel * 2].view(torch.bfloat16)
            big = max(u.numel for u in (self.units + ([self.root] if self.root is not None else [])))
            self.grad_half = -(-big * 2 // 256) * 256
            self.grad_buf = SymmetricBuffer(self.flags_bytes + 2 * self.grad_half, self.device, self.group)
            self.epoch = 0
        elif self.cuda:
            from ..ops import native

            self.native = native
            self.lowp_shard = torch.zeros(shard_numel, dtype=torch.bfloat16, device=self.device)
        else:
            self.lowp_shard = None

    def _refresh_lowp_shards(self) -> None:
        if self.lowp_shard is not None:
            self.lowp_shard.copy_(self.master)
        if self.cuda and self.world > 1:
            torch.cuda.synchronize(self.device)
            self.param_buf.barrier()          # every rank's slices are in place before anybody gathers them

    # ------------------------------------------------------------------ gather / free
    def _views(self, u: _Unit, f32: torch.Tensor, lowp: Optional[torch.Tensor], grad: Optional[torch.Tensor], attach: bool = True) -> None:
        """Point the unit's parameters at their gathered images.  ``grad``: the unit's gradient slot; with ``attach`` it also
        becomes ``parameter.grad`` (autograd accumulates into it), otherwise only the kernels' ``_grad_view`` is set (its address
        is fixed per unit, and the whole-layer executor records it when it first meets the layer, in forward)."""
        # A unit always lands in the same pool slot and the same gradient slot, so the views are built once per (unit, buffers);
        # later calls only re-attach ``.grad`` (begin_step clears it).  Building ~6 tensor views for each of a block's ~40
        # parameters on every visit costs about a millisecond of host time per unit, more than a Conformer block computes.
        key = (f32.data_ptr(), 0 if lowp is None else lowp.data_ptr(), 0 if grad is None else grad.data_ptr())
        if getattr(u, "_view_key", None) == key:
            if attach and grad is not None:
                for p in u.params:
                    p.grad = p._grad_view
            return
        for p in u.params:
            o, n = u.offsets[id(p)]
            shape = self._shape_of(p)
            p.data = f32[o:o + n].view(shape)
            if lowp is not None:
                p._lowp = lowp[o:o + n].view(shape)
            if grad is not None:
                p._grad_view = grad[o:o + n].view(shape)
                if attach:
                    p.grad = p._grad_view
            p._arena = self
        u._view_key = key if grad is not None else None

    def _shape_of(self, p) -> Tuple[int, ...]:
        return self._shapes[id(p)]

    def _gather(self, u: _Unit, slot: Optional[int] = None) -> None:
        """Full parameters of ``u`` into its pool slot (or the root buffers), on the communication stream when there is one."""
        if u is self.root:
            f32, lowp = self.root_f32, self.root_lowp
        else:
            slot = u.index % 2 if slot is None else slot
            f32, lowp = self.pool_f32[slot], self.pool_lowp[slot]
            self.pool_owner[slot] = u
            u.slot = slot
        n = u.numel
        if self.cuda and self.world > 1:
            lib = self.native.lib()
            cur = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(cur)          # the slot's previous user has been enqueued before this point
            with torch.cuda.stream(self.comm_stream):
                rc = lib.sb_fsdp_gather(ctypes.c_void_p(self.param_buf.ptrs_dev), ctypes.c_longlong(u.shard_base * 2), ctypes.c_longlong(u.slice),
                                        ctypes.c_int(self.world), ctypes.c_void_p(lowp.data_ptr()), ctypes.c_void_p(f32.data_ptr()),
                                        ctypes.c_int(self.gather_blocks), self.native._stream())
                if rc != 0:
                    raise RuntimeError(f"sb_fsdp_gather failed with code {rc}")
                self.native.launch_count += 1
                u.ready_event = torch.cuda.Event()
                u.ready_event.record()
        elif self.world > 1:
            parts = list(f32[:n].chunk(self.world))
            dist.all_gather(parts, self.master[u.shard_base:u.shard_base + u.slice].contiguous(), group=self.group)
            u.ready_event = None
        else:
            f32[:n].copy_(self.master[u.shard_base:u.shard_base + u.slice])
            if lowp is not None:
                lowp[:n].copy_(f32[:n])
            u.ready_event = None
        u.gathered = True
        self._views(u, f32, lowp, self.root_grad if u is self.root else self.pool_grad[u.index % 2], attach=False)

    def _wait_gathered(self, u: _Unit) -> None:
        ev = getattr(u, "ready_event", None)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            u.ready_event = None

    def _ensure(self, u: _Unit, prefetch: Optional[_Unit]) -> None:
        if not u.gathered or (u is not self.root and self.pool_owner[u.index % 2] is not u):
            self._gather(u)
        self._wait_gathered(u)
        if prefetch is not None and prefetch is not self.root and (not prefetch.gathered or self.pool_owner[prefetch.index % 2] is not prefetch):
            self._gather(prefetch)

    def _free(self, u: _Unit) -> None:
        if u is not self.root:
            u.gathered = False      # the slot is reused by the unit two positions further on

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        for i, u in enumerate(self.units):
            nxt = self.units[i + 1] if i + 1 < len(self.units) else None
            prv = self.units[i - 1] if i > 0 else None
            u.module.register_forward_pre_hook(lambda m, a, u=u, nxt=nxt: self._ensure(u, nxt))
            u.module.register_forward_hook(lambda m, a, o, u=u: self._free(u))
            u.module.register_full_backward_pre_hook(lambda m, g, u=u, prv=prv: self._pre_backward(u, prv))

    def _pre_backward(self, u: _Unit, prefetch: Optional[_Unit]) -> None:
        self._ensure(u, prefetch)
        self._attach_grads(u)

    def _attach_grads(self, u: _Unit) -> None:
        if u.gslot is not None:
            return
        if u is self.root:
            g = self.root_grad
        else:
            gs = u.index % 2
            ev = self._gpool_free_event[gs]
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)     # the slot's previous reduction has read it
                self._gpool_free_event[gs] = None
            g = self.pool_grad[gs]
        g[:u.numel].zero_()
        u.gslot = 0
        slot = u.index % 2 if u.slot is None else u.slot
        f32 = self.root_f32 if u is self.root else self.pool_f32[slot]
        lowp = self.root_lowp if u is self.root else self.pool_lowp[slot]
        self._views(u, f32, lowp, g)

    # ------------------------------------------------------------------ step protocol (called by FSDP2GradSync)
    def begin_step(self) -> None:
        for u in self.all_units:
            u.gslot = None
            for p in u.params:
                p.grad = None
        if self.root is not None:
            self._wait_gathered(self.root)
            self._attach_grads(self.root)
        if self.deferred_update:
            self._scalars[3] = 0.0

    def grad_ready(self, param) -> None:       # the arena protocol of the native kernels (parallel/ddp.py wires the real one)
        pass

    def reduce_unit(self, u: _Unit) -> None:
        """All gradients of ``u`` are final: reduce-scatter them (and update at once when there is no global clipping)."""
        if u.gslot is None:
            self._attach_grads(u)                # unit without any gradient this step: contributes zeros
        g = self.root_grad if u is self.root else self.pool_grad[u.index % 2]
        sl = slice(u.shard_base, u.shard_base + u.slice)
        grp = self.param_groups[0]
        fused_update = not self.deferred_update
        if self.cuda and self.world > 1:
            cur = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(cur)
            with torch.cuda.stream(self.comm_stream):
                self.epoch += 1
                h = self.epoch & 1
                a = SbFsdpArgs()
                a.grad_bufs = self.grad_buf.ptrs_dev
                a.buf_off = self.flags_bytes + h * self.grad_half
                a.flags_off = 0
                a.slice, a.rank, a.world, a.ctas, a.epoch = u.slice, self.rank, self.world, self.ctas, self.epoch
                if fused_update:
                    a.mode = 0
                    a.master = self.master[sl].data_ptr()
                    a.exp_avg, a.exp_avg_sq = self.exp_avg[sl].data_ptr(), self.exp_avg_sq[sl].data_ptr()
                    a.lowp_shard = self.lowp_shard[sl].data_ptr()
                    b1, b2 = grp["betas"]
                    a.lr, a.beta1, a.beta2, a.eps, a.wd = float(grp["lr"]), b1, b2, grp["eps"], grp["weight_decay"]
                else:
                    a.mode = 1
                    a.grad_shard = self.grad_shard[sl].data_ptr()
                    a.sumsq = self._scalars[3:].data_ptr()
                rc = self.native.lib().sb_fsdp_reduce_scatter(ctypes.byref(a), ctypes.c_void_p(g.data_ptr()),
                                                              ctypes.c_void_p(self.grad_buf.tensor.data_ptr()), ctypes.c_float(1.0 / self.world),
                                                              ctypes.c_int(self._step + 1), self.native._stream())
                if rc != 0:
                    raise RuntimeError(f"sb_fsdp_reduce_scatter failed with code {rc}")
                self.native.launch_count += 2
                if u is not self.root:
                    ev = torch.cuda.Event()
                    ev.record()
                    self._gpool_free_event[u.index % 2] = ev
        else:
            gu = g[:u.numel]
            if self.world > 1:
                gu = gu / self.world
                dist.all_reduce(gu, group=self.group)
            mine = gu[self.rank * u.slice:(self.rank + 1) * u.slice]
            if self.grad_shard is not None:
                self.grad_shard[sl].copy_(mine)
            if fused_update:
                self._adamw_range(u.shard_base, u.shard_base + u.slice, self._step + 1)
        u.gslot = None

    def _adamw_range(self, lo: int, hi: int, step: int, coef: Optional[torch.Tensor] = None) -> None:
        grp = self.param_groups[0]
        b1, b2 = grp["betas"]
        g = self.grad_shard[lo:hi]
        if coef is not None:
            g = g * coef
        if self.cuda:
            from .. import ops

            if not hasattr(self, "_unit_scalars"):
                self._unit_scalars = torch.tensor([0.0, 1.0, 0.0, 0.0], dtype=torch.float32, device=self.device)
            ops.adamw_flat(self.master[lo:hi], g.contiguous(), self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], self.lowp_shard[lo:hi],
                           lr=float(grp["lr"]), beta1=b1, beta2=b2, eps=grp["eps"], weight_decay=grp["weight_decay"], step=step,
                           scalars=self._unit_scalars)
            return
        m, v, p = self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], self.master[lo:hi]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        p.mul_(1 - grp["lr"] * grp["weight_decay"]).addcdiv_(m, v.sqrt() / math.sqrt(bc2) + grp["eps"], value=-grp["lr"] / bc1)

    @torch.no_grad()
    def step(self, closure=None):
        """With global clipping: the clipped update of all slices.  Without: only the bookkeeping (updates already ran, unit by
        unit, inside backward).  Ends with the barrier after which peers may gather the new slices."""
        self._step += 1
        if self.cuda and self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        if self.replicas > 1:
            self.grad_shard.div_(self.replicas)
            dist.all_reduce(self.grad_shard, group=self.replicate_group)
        if self.max_grad_norm > 0:
            if getattr(self, "_tp_mask", None) is not None:
                # tensor-parallel model: slices of tensor-parallel parameters differ over the tp group and are summed there;
                # everything else is replicated over it and counted once
                g2 = self.grad_shard.double().pow(2)
                sq_tp = (g2 * self._tp_mask).sum().float().view(1)
                sq_rep = g2.sum().float().view(1) - sq_tp
                dist.all_reduce(sq_tp, group=self._tp_group)
                sq = sq_tp + sq_rep
            elif self.cuda and self.world > 1 and self.replicas == 1:
                sq = self._scalars[3:4].clone()
            else:
                sq = self.grad_shard.double().pow(2).sum().float().view(1)
            if self.world > 1:
                dist.all_reduce(sq, group=self.group)
            norm = sq.sqrt()
            self._scalars[0] = norm[0]
            coef = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
            self._adamw_range(0, self.shard_numel, self._step, coef)
        elif self.replicas > 1:
            self._adamw_range(0, self.shard_numel, self._step)
        if self.cuda and self.world > 1:
            self.param_buf.barrier()           # device-side barrier on the current stream: every rank's new slices are in place
        for u in self.units:
            u.gathered = False
        if self.root is not None:
            self._gather(self.root)
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        pass           # gradient slots are zeroed when a unit's backward starts

    def set_tensor_parallel(self, tp_group, is_tp_param) -> None:
        """Make the clipping norm exact on a (data-parallel x tensor-parallel) mesh.  ``is_tp_param(p)`` says whether ``p``
        holds one tensor-parallel slice of a larger weight (its squared gradient norm is then summed over ``tp_group``);
        other parameters are replicas over that group and enter the norm once."""
        mask = torch.zeros(self.shard_numel, dtype=torch.bool, device=self.device)
        for u in self.all_units:
            lo, hi = self.rank * u.slice, (self.rank + 1) * u.slice
            for q in u.params:
                if not is_tp_param(q):
                    continue
                o, n = u.offsets[id(q)]
                a, b = max(o, lo), min(o + n, hi)
                if a < b:
                    mask[u.shard_base + a - lo:u.shard_base + b - lo] = True
        self._tp_mask, self._tp_group = mask, tp_group

    @property
    def last_grad_norm(self) -> torch.Tensor:
        return self._scalars[0]

    # ------------------------------------------------------------------ full views for checkpoints / evaluation
    def gather_full_state(self) -> Dict[int, torch.Tensor]:
        """``id(param) -> full fp32 tensor`` (a collective: every rank must call it)."""
        out = {}
        for u in self.all_units:
            full = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
            if self.world > 1:
                dist.all_gather(list(full.chunk(self.world)), self.master[u.shard_base:u.shard_base + u.slice].contiguous(), group=self.group)
            else:
                full.copy_(self.master[u.shard_base:u.shard_base + u.slice])
            for p in u.params:
                o, n = u.offsets[id(p)]
                out[id(p)] = full[o:o + n].view(self._shape_of(p)).clone()
        return out

    # ------------------------------------------------------------------ checkpoints (independent of the number of ranks)
    def _gather_flat(self, u: _Unit, shard: torch.Tensor) -> torch.Tensor:
        full = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
        mine = shard[u.shard_base:u.shard_base + u.slice].contiguous()
        if self.world > 1:
            dist.all_gather(list(full.chunk(self.world)), mine, group=self.group)
        else:
            full.copy_(mine)
        return full

    def _names(self) -> Dict[int, str]:
        return {id(p): n for n, p in self.model.named_parameters()}

    def full_model_state_dict(self) -> Dict[str, torch.Tensor]:
        """``model.state_dict()`` with every sharded parameter replaced by its full fp32 value (CPU tensors).  Parameters of
        units that are not gathered hold no data, so the plain ``state_dict`` must not be saved.  A collective."""
        names = self._names()
        full = self.gather_full_state()
        sd = {}
        for k, v in self.model.state_dict().items():
            sd[k] = v.detach().cpu() if torch.is_tensor(v) else v
        from .tp import mp_full

        by_id = {id(q): q for q in self.model.parameters()}
        prefix_free = {n: mp_full(by_id[i], full[i]).cpu() for i, n in names.items() if i in full}     # tensor-parallel slices -> whole
        for k in list(sd):
            if k in prefix_free:
                sd[k] = prefix_free[k]
        return sd

    def load_full_params(self, state_dict: Dict[str, torch.Tensor]) -> None:
        """Take this rank's slices of the full parameter values in ``state_dict`` (names as in ``model.named_parameters()``);
        entries that are missing keep their current value.  Every rank calls it with the same dictionary."""
        names = self._names()
        with torch.no_grad():
            for u in self.all_units:
                flat = self._gather_flat(u, self.master) if any(names[id(q)] not in state_dict for q in u.params) else \
                    torch.zeros(u.numel, dtype=torch.float32, device=self.device)
                for q in u.params:
                    t = state_dict.get(names[id(q)])
                    if t is not None:
                        from .tp import mp_local

                        o, n = u.offsets[id(q)]
                        t = mp_local(q, t, self._shape_of(q))            # this rank's tensor-parallel slice of a full tensor
                        flat[o:o + n].copy_(t.reshape(-1).to(self.device, torch.float32))
                self.master[u.shard_base:u.shard_base + u.slice].copy_(flat[self.rank * u.slice:(self.rank + 1) * u.slice])
                u.gathered = False
        self._refresh_lowp_shards()
        if self.root is not None:
            self._gather(self.root)

    def state_dict(self) -> Dict[str, Any]:
        """Moments as full tensors in the parameters' own shapes, keyed by parameter name: no padding and no slice boundaries
        enter the file, so the checkpoint loads at any number of ranks (and into a replicated AdamW of the same model).  The
        reference needs a patch of its sharded optimizer for the same property (``core/optim/flash_optim.py:22``: uneven
        FSDP2 shards in the saved optimizer state).  A collective."""
        names = self._names()
        state = {}
        for u in self.all_units:
            m, v = self._gather_flat(u, self.exp_avg), self._gather_flat(u, self.exp_avg_sq)
            for q in u.params:
                o, n = u.offsets[id(q)]
                shape = self._shape_of(q)
                from .tp import mp_full

                state[names[id(q)]] = {"exp_avg": mp_full(q, m[o:o + n].view(shape)).cpu().clone(),
                                       "exp_avg_sq": mp_full(q, v[o:o + n].view(shape)).cpu().clone()}
        groups = [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]
        return {"format": "fully_sharded_adamw/full-by-name", "step": self._step, "state": state, "param_groups": groups}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd.get("format") != "fully_sharded_adamw/full-by-name":
            raise ValueError("not a FullyShardedAdamW state dict (expected the full-by-name format)")
        names = self._names()
        self._step = int(sd.get("step", 0))
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update({k: v for k, v in saved.items() if k != "params"})
        with torch.no_grad():
            for u in self.all_units:
                m = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
                v = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
                for q in u.params:
                    st = sd["state"].get(names[id(q)])
                    if st is None:
                        continue
                    from .tp import mp_local

                    o, n = u.offsets[id(q)]
                    shape = self._shape_of(q)
                    m[o:o + n].copy_(mp_local(q, st["exp_avg"], shape).reshape(-1).to(self.device, torch.float32))
                    v[o:o + n].copy_(mp_local(q, st["exp_avg_sq"], shape).reshape(-1).to(self.device, torch.float32))
                lo, hi = self.rank * u.slice, (self.rank + 1) * u.slice
                self.exp_avg[u.shard_base:u.shard_base + u.slice].copy_(m[lo:hi])
                self.exp_avg_sq[u.shard_base:u.shard_base + u.slice].copy_(v[lo:hi])

    def memory_report(self) -> Dict[str, float]:
        per = 4 + 8 + (2 if self.cuda else 0) + (4 if self.grad_shard is not None else 0)
        persistent = self.shard_numel * per
        big = max((u.numel for u in self.units), default=0)
        pools = 2 * big * (4 + (2 if self.cuda else 0)) + 2 * big * 4
        root = (self.root.numel * (4 + 4 + (2 if self.cuda else 0))) if self.root is not None else 0
        replicated = self.total_numel * (16 + 2)
        rep = {"params": self.total_numel, "world": self.world, "persistent_bytes_per_rank": persistent, "pool_bytes": pools,
               "root_bytes": root, "replicated_bytes": replicated, "persistent_fraction_of_replicated": persistent / max(1, replicated)}
        logging.info(f"fully-sharded state: {rep}")
        return rep


class FSDP2GradSync:
    """Trainer strategy object for ``FullyShardedAdamW``: a unit is reduced as soon as every gradient in it is final."""

    def __init__(self, model, optimizers, world_size: int, device: torch.device, sync_batchnorm: bool = False, **_):
        self.opt = next(o for o in optimizers if isinstance(o, FullyShardedAdamW))
        self.model, self.world_size, self.device = model, world_size, device
        self.comm_stream = self.opt.comm_stream
        self.order = list(reversed(self.opt.units)) + ([self.opt.root] if self.opt.root is not None else [])
        self.buckets = [{"params": u.params, "unit": u} for u in self.order]
        self._bucket_of = {id(p): bi for bi, b in enumerate(self.buckets) for p in b["params"]}
        self._sync_enabled = True
        self.opt.grad_ready = self.mark_ready
        for p in (q for b in self.buckets for q in b["params"]):
            p.register_post_accumulate_grad_hook(lambda param: self.mark_ready(param))
        self.launched_in_backward = 0
        if sync_batchnorm:
            from .ddp import small_allreduce

            for m in model.modules():
                if hasattr(m, "bn_stats_reduce"):
                    m.bn_stats_reduce = small_allreduce

    def begin_step(self):
        self.opt.begin_step()
        self._pending = [{id(p) for p in b["params"]} for b in self.buckets]
        self._done = [False] * len(self.buckets)
        self._complete = [False] * len(self.buckets)
        self._next = 0
        self.launched_in_backward = 0

    def no_sync(self):
        import contextlib

        return contextlib.nullcontext()

    def mark_ready(self, param):
        if not hasattr(self, "_pending"):
            return
        bi = self._bucket_of.get(id(param))
        if bi is None or self._done[bi]:
            return
        self._pending[bi].discard(id(param))
        if not self._pending[bi]:
            self._complete[bi] = True
            # strictly in bucket order (the same on every rank); the root closes the step and is reduced in finish_step
            while self._next < len(self.buckets) - (1 if self.opt.root is not None else 0) and self._complete[self._next]:
                self._reduce(self._next)
                self._next += 1
                self.launched_in_backward += 1

    def _reduce(self, bi: int):
        self._done[bi] = True
        self.opt.reduce_unit(self.buckets[bi]["unit"])

    def finish_step(self):
        for bi in range(self._next, len(self.buckets)):
            if not self._done[bi]:
                self._reduce(bi)
        self._next = len(self.buckets)
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

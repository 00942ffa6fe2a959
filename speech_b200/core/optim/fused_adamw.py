"""Flat-arena AdamW.

All trainable parameters of a model are re-homed into one contiguous fp32 *master* buffer,
with matching flat buffers for gradients, both Adam moments and a bf16 *working copy* that
the GEMM kernels read.  One optimizer step is then a single kernel launch per parameter group
that reads gradient + moments + master weights once and writes moments, master weights and
the bf16 copy once — instead of the several passes of a per-tensor or ``foreach`` AdamW
(what the reference uses: ``torch.optim.AdamW`` via ``nemo/core/optim/optimizers.py:36``).

Gradient clipping is folded into the same pass: the global gradient norm is computed by one
reduction over the flat gradient buffer and the clip coefficient is read by the update kernel
from device memory, so no host synchronisation is needed.

The flat layout is also what the data-parallel gradient exchange operates on
(``speech_b200.parallel.ddp``): buckets are plain slices of the flat gradient buffer.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
from torch.optim.optimizer import Optimizer

ALIGN = 128  # elements; keeps every bf16 view 256-byte aligned (TMA needs 16)


class ParamArena:
    """Owns the flat buffers and points ``param.data`` / ``param.grad`` / ``param._lowp`` into them."""

    def __init__(self, groups: List[List[torch.nn.Parameter]], lowp_dtype: Optional[torch.dtype] = torch.bfloat16,
                 fusion_groups: Optional[List[List[torch.nn.Parameter]]] = None, pad_multiple: int = 1):
        groups = [self._reorder(g, fusion_groups or []) for g in groups]
        params = [p for g in groups for p in g]
        if not params:
            raise ValueError("ParamArena needs at least one parameter")
        dev = params[0].device
        self.device = dev
        self.params = params
        self.group_ranges: List[Tuple[int, int]] = []
        self.offsets: Dict[int, Tuple[int, int]] = {}
        off = 0
        for g in groups:
            start = off
            for p in g:
                if p.device != dev:
                    raise ValueError("All parameters of an arena must live on one device")
                if p.dtype != torch.float32:
                    raise ValueError("Arena parameters must be fp32 master weights")
                n = p.numel()
                self.offsets[id(p)] = (off, n)
                off += (n + ALIGN - 1) // ALIGN * ALIGN
            self.group_ranges.append((start, off))
        self.used_numel = off
        off = (off + pad_multiple - 1) // pad_multiple * pad_multiple   # sharded optimizers want equal slices per rank
        self.numel = off
        self.master = torch.zeros(off, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(off, dtype=torch.float32, device=dev)
        self.lowp = torch.zeros(off, dtype=lowp_dtype, device=dev) if lowp_dtype is not None else None
        with torch.no_grad():
            for p in params:
                o, n = self.offsets[id(p)]
                view = self.master[o:o + n].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.grad[o:o + n].view(p.shape)
                if self.lowp is not None:
                    p._lowp = self.lowp[o:o + n].view(p.shape)
                    p._lowp.copy_(view)
                p._grad_view = p.grad
                p._arena = self
        self.lowp_version = 0

    @staticmethod
    def _reorder(group, fusion_groups):
        """Move the members of each fusion group next to its first member (order inside the group kept)."""
        in_group = {id(p) for p in group}
        follow = {}
        skip = set()
        for fg in fusion_groups:
            if len(fg) < 2 or not all(id(p) in in_group for p in fg):
                continue
            if any(p.numel() % ALIGN for p in fg[:-1]) or any(id(p) in skip or id(p) in follow for p in fg):
                continue
            follow[id(fg[0])] = fg[1:]
            skip.update(id(p) for p in fg[1:])
        out = []
        for p in group:
            if id(p) in skip:
                continue
            out.append(p)
            out.extend(follow.get(id(p), []))
        return out

    def fuse(self, params):
        """Zero-copy stacked view over parameters that are adjacent in the arena, or ``None``.

        The result is a view of the master buffer with ``_lowp`` (working copy) and ``_grad_view`` (flat gradient)
        attributes, which is all the native GEMM wrappers need from a weight."""
        offs = [self.offsets.get(id(p)) for p in params]
        if any(o is None for o in offs):
            return None
        for (o, n), (o2, _) in zip(offs[:-1], offs[1:]):
            if o + n != o2:
                return None
        start = offs[0][0]
        total = sum(n for _, n in offs)
        tail = tuple(params[0].shape[1:])
        if any(tuple(p.shape[1:]) != tail for p in params):
            return None
        shape = (sum(p.shape[0] for p in params),) + tail
        view = self.master[start:start + total].view(shape)
        # autograd must see the stacked weight as a trainable leaf, or custom Functions skip its gradient (needs_input_grad);
        # the gradient itself is written by the kernels into ``_grad_view``, never into ``view.grad``
        view.requires_grad_(any(p.requires_grad for p in params))
        view._grad_view = self.grad[start:start + total].view(shape)
        if self.lowp is not None:
            view._lowp = self.lowp[start:start + total].view(shape)
        view._arena = self
        view._members = list(params)
        return view

    def refresh_lowp(self) -> None:
        if self.lowp is not None:
            self.lowp.copy_(self.master)

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p in self.params:
            o, n = self.offsets[id(p)]
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * o:
                p.grad = self.grad[o:o + n].view(p.shape)


class FusedAdamW(Optimizer):
    """AdamW (decoupled weight decay) over a :class:`ParamArena`.

    Args mirror ``torch.optim.AdamW``; ``max_grad_norm`` (> 0) enables fused global-norm clipping,
    ``lowp_dtype`` selects the dtype of the working copy (``None`` disables it).
    """

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 max_grad_norm: float = 0.0, lowp_dtype: Optional[torch.dtype] = torch.bfloat16, amsgrad: bool = False,
                 fusion_groups=None, arena_pad_multiple: int = 1, **_unused):
        if amsgrad:
            raise ValueError("FusedAdamW does not implement amsgrad")
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.max_grad_norm = float(max_grad_norm or 0.0)
        groups = [[p for p in g["params"] if p.requires_grad] for g in self.param_groups]
        self._nonempty = [i for i, g in enumerate(groups) if g]
        self.arena = ParamArena([groups[i] for i in self._nonempty], lowp_dtype=lowp_dtype, fusion_groups=fusion_groups,
                                pad_multiple=arena_pad_multiple)
        a = self.arena
        self._alloc_state()
        self._step = 0
        # device scalars: [0] = sum of squares / grad norm, [1] = clip coefficient, [2] = found-inf flag
        self._scalars = torch.zeros(4, dtype=torch.float32, device=a.device)
        self._scalars[1] = 1.0
        self.grad_scale: float = 1.0  # extra multiplier applied to gradients (e.g. 1/accumulation)

    def _alloc_state(self) -> None:
        self.exp_avg = torch.zeros_like(self.arena.master)
        self.exp_avg_sq = torch.zeros_like(self.arena.master)

    # ------------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = False) -> None:
        self.arena.zero_grad()

    @property
    def last_grad_norm(self) -> torch.Tensor:
        return self._scalars[0]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        from ... import ops

        a = self.arena
        self._step += 1
        if self.max_grad_norm > 0:
            ops.grad_norm_clip_coef(a.grad, self._scalars, self.max_grad_norm, self.grad_scale)
        else:
            self._scalars[1] = self.grad_scale
        for gi, (start, end) in zip(self._nonempty, a.group_ranges):
            g = self.param_groups[gi]
            b1, b2 = g["betas"]
            ops.adamw_flat(
                a.master[start:end], a.grad[start:end], self.exp_avg[start:end], self.exp_avg_sq[start:end],
                a.lowp[start:end] if a.lowp is not None else None,
                lr=float(g["lr"]), beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"], step=self._step,
                scalars=self._scalars,
            )
        return loss

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> Dict[str, Any]:
        a = self.arena
        state = {}
        idx = 0
        packed_groups = []
        for g in self.param_groups:
            ids = []
            for p in g["params"]:
                if id(p) in a.offsets:
                    o, n = a.offsets[id(p)]
                    state[idx] = {
                        "step": torch.tensor(float(self._step)),
                        "exp_avg": self.exp_avg[o:o + n].view(p.shape).clone(),
                        "exp_avg_sq": self.exp_avg_sq[o:o + n].view(p.shape).clone(),
                    }
                ids.append(idx)
                idx += 1
            packed_groups.append({**{k: v for k, v in g.items() if k != "params"}, "params": ids})
        return {"state": state, "param_groups": packed_groups, "fused_step": self._step}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        a = self.arena
        idx = 0
        for g, sg in zip(self.param_groups, state_dict["param_groups"]):
            for k, v in sg.items():
                if k != "params":
                    g[k] = v
            for p in g["params"]:
                st = state_dict["state"].get(idx, state_dict["state"].get(str(idx)))
                if st is not None and id(p) in a.offsets:
                    o, n = a.offsets[id(p)]
                    self.exp_avg[o:o + n].copy_(st["exp_avg"].reshape(-1))
                    self.exp_avg_sq[o:o + n].copy_(st["exp_avg_sq"].reshape(-1))
                    self._step = int(float(st.get("step", self._step)))
                idx += 1
        self._step = int(state_dict.get("fused_step", self._step))
        a.refresh_lowp()

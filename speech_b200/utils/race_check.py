"""Race checks that need no sanitizer: run a step twice and compare bit for bit, and surround output buffers with guard bands.

A data race between CTAs, a read of a buffer before its producer finished, or a write past the end of a tile shows up as (a) two
runs of the same deterministic computation that differ in some bits, or (b) a sentinel next to an output that no longer holds
its pattern.  Both checks run on any device; on CUDA they synchronise.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

__all__ = ["GuardedTensor", "RunTwiceReport", "flatten_tensors", "guarded_empty", "run_twice"]

_SENTINEL_BYTE = 0xA5


def flatten_tensors(obj: Any, prefix: str = "out") -> List[Tuple[str, torch.Tensor]]:
    """Every tensor inside nested tuples / lists / dicts, with a path name."""
    if torch.is_tensor(obj):
        return [(prefix, obj)]
    if isinstance(obj, dict):
        return [t for k, v in obj.items() for t in flatten_tensors(v, f"{prefix}.{k}")]
    if isinstance(obj, (list, tuple)):
        return [t for i, v in enumerate(obj) for t in flatten_tensors(v, f"{prefix}[{i}]")]
    return []


@dataclass
class RunTwiceReport:
    identical: bool
    mismatches: List[Dict[str, Any]] = field(default_factory=list)

    def raise_if_different(self):
        if not self.identical:
            lines = [f"{m['name']}: {m['count']} of {m['numel']} elements differ, max |a-b| = {m['max_abs']:.3e}, first at {m['first']}" for m in self.mismatches]
            raise AssertionError("two runs of the same step differ:\n  " + "\n  ".join(lines))


def _bits(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    if t.dtype == torch.float64:
        return t.view(torch.int64)
    return t


def run_twice(step: Callable[[], Any], *, parameters: Sequence[torch.nn.Parameter] = (), seed: int = 0,
              reset: Optional[Callable[[], None]] = None) -> RunTwiceReport:
    """Calls ``step()`` twice from the same random state and compares all tensors it returns, plus the ``.grad`` of ``parameters``,
    bit for bit (NaNs with the same payload count as equal).  ``reset`` runs before each call (e.g. to restore buffers the step
    updates in place); gradients of ``parameters`` are cleared before each call."""
    runs: List[List[Tuple[str, torch.Tensor]]] = []
    for _ in range(2):
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)
        if reset is not None:
            reset()
        for p in parameters:
            p.grad = None
        out = step()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        named = [(n, t.detach().clone()) for n, t in flatten_tensors(out)]
        named += [(f"grad[{i}]", p.grad.detach().clone()) for i, p in enumerate(parameters) if p.grad is not None]
        runs.append(named)
    a, b = runs
    rep = RunTwiceReport(identical=True)
    if [n for n, _ in a] != [n for n, _ in b]:
        rep.identical = False
        rep.mismatches.append({"name": "<structure>", "count": 0, "numel": 0, "max_abs": float("nan"), "first": "tensor sets differ"})
        return rep
    for (n, x), (_, y) in zip(a, b):
        if x.shape != y.shape or x.dtype != y.dtype:
            rep.identical = False
            rep.mismatches.append({"name": n, "count": -1, "numel": x.numel(), "max_abs": float("nan"), "first": f"{tuple(x.shape)} vs {tuple(y.shape)}"})
            continue
        ne = _bits(x) != _bits(y)
        if bool(ne.any()):
            idx = ne.flatten().nonzero()[0].item()
            diff = (x.double() - y.double()).abs() if x.is_floating_point() else (x != y).double()
            rep.identical = False
            rep.mismatches.append({"name": n, "count": int(ne.sum()), "numel": x.numel(), "max_abs": float(torch.nan_to_num(diff).max()),
                                   "first": tuple(int(v) for v in torch.unravel_index(torch.tensor(idx), x.shape)) if x.dim() else ()})
    return rep


class GuardedTensor:
    """A tensor carved out of a larger allocation with ``guard_bytes`` of sentinel bytes before and after it.  Hand ``.tensor`` to
    a kernel as its output, then call ``check()``: it raises when any guard byte changed and names the side and the offset."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device="cpu", guard_bytes: int = 4096, fill: Optional[float] = None):
        esz = torch.empty((), dtype=dtype).element_size()
        guard_bytes = (guard_bytes + 255) // 256 * 256                          # keeps the payload 256-byte aligned
        numel = 1
        for s in shape:
            numel *= int(s)
        self._payload = numel * esz
        self._guard = guard_bytes
        total = 2 * guard_bytes + (self._payload + 255) // 256 * 256
        self._raw = torch.full((total,), _SENTINEL_BYTE, dtype=torch.uint8, device=device)
        self.tensor = self._raw[guard_bytes: guard_bytes + self._payload].view(dtype).view(*shape)
        if fill is not None:
            self.tensor.fill_(fill)

    def violations(self) -> List[Tuple[str, int]]:
        """``(side, byte offset from the payload edge)`` of the first changed byte on each side."""
        out = []
        front = self._raw[: self._guard] != _SENTINEL_BYTE
        if bool(front.any()):
            out.append(("before", self._guard - int(front.nonzero()[-1])))       # distance back from the payload start
        back = self._raw[self._guard + self._payload:] != _SENTINEL_BYTE
        if bool(back.any()):
            out.append(("after", int(back.nonzero()[0])))
        return out

    def check(self, what: str = "buffer"):
        v = self.violations()
        if v:
            raise AssertionError(f"{what}: guard band overwritten " + ", ".join(f"{side} the payload at byte offset {off}" for side, off in v))


def guarded_empty(shape, dtype, device="cpu", guard_bytes: int = 4096, fill: Optional[float] = None) -> GuardedTensor:
    return GuardedTensor(shape, dtype, device, guard_bytes, fill)

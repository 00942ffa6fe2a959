"""Autograd wrappers of the LLM-block kernels (``csrc/llm_ops.cu``): RMSNorm, SwiGLU and rotary position embedding on bf16
activations.  Each function has a plain PyTorch fp32 restatement in the same file (``*_reference``) that serves CPU tensors,
other dtypes and the numerics tests."""
from __future__ import annotations

import ctypes

import torch

from .native import _check, _ptr, _stream, lib


# ------------------------------------------------------------------------------------------------ fp32 restatements
def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * xf).to(x.dtype)


def swiglu_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(gate) * up


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[B, T, H, D]``, cos / sin ``[B, T, D]`` (rotate-half convention)."""
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return (x.float() * cos.unsqueeze(2) + rot.float() * sin.unsqueeze(2)).to(x.dtype)


# ------------------------------------------------------------------------------------------------ kernels
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().sb_rmsnorm_fwd(_ptr(x2), _ptr(weight), _ptr(y), _ptr(rstd), ctypes.c_longlong(rows), ctypes.c_int(D),
                                    ctypes.c_float(eps), _stream()), "sb_rmsnorm_fwd")
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        dg = torch.zeros(D, dtype=torch.float32, device=dy.device) if ctx.needs_input_grad[1] else None
        _check(lib().sb_rmsnorm_bwd(_ptr(dy2), _ptr(x2), _ptr(weight), _ptr(rstd), _ptr(dx), _ptr(dg), ctypes.c_longlong(rows),
                                    ctypes.c_int(D), _stream()), "sb_rmsnorm_bwd")
        return dx.view(ctx.shape), dg, None


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        g, u = gate.contiguous(), up.contiguous()
        y = torch.empty_like(g)
        _check(lib().sb_swiglu_fwd(_ptr(g), _ptr(u), _ptr(y), ctypes.c_longlong(g.numel()), _stream()), "sb_swiglu_fwd")
        ctx.save_for_backward(g, u)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dy = dy.contiguous()
        dg, du = torch.empty_like(g), torch.empty_like(u)
        _check(lib().sb_swiglu_bwd(_ptr(dy), _ptr(g), _ptr(u), _ptr(dg), _ptr(du), ctypes.c_longlong(g.numel()), _stream()), "sb_swiglu_bwd")
        return dg, du


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        B, T, H, D = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _check(lib().sb_rope(_ptr(xc), _ptr(cos), _ptr(sin), _ptr(y), ctypes.c_longlong(B * T * H), ctypes.c_int(H), ctypes.c_int(D),
                             ctypes.c_int(0), _stream()), "sb_rope")
        ctx.save_for_backward(cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, T, H, D = dy.shape
        dyc = dy.contiguous()
        dx = torch.empty_like(dyc)
        _check(lib().sb_rope(_ptr(dyc), _ptr(cos), _ptr(sin), _ptr(dx), ctypes.c_longlong(B * T * H), ctypes.c_int(H), ctypes.c_int(D),
                             ctypes.c_int(1), _stream()), "sb_rope")
        return dx, None, None


def _native_ok(*ts: torch.Tensor) -> bool:
    from . import _use_native

    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and _use_native(ts[0])


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if _native_ok(x) and weight.dtype == torch.float32 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 12288 and x.numel() > 0:
        return _RMSNormFn.apply(x, weight, eps)
    return rmsnorm_reference(x, weight, eps)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if _native_ok(gate, up) and gate.numel() % 8 == 0 and gate.numel() > 0 and gate.shape == up.shape:
        return _SwiGLUFn.apply(gate, up)
    return swiglu_reference(gate, up)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[B, T, H, D]``; cos / sin fp32 ``[B, T, D]`` contiguous."""
    if _native_ok(x) and x.shape[-1] % 16 == 0 and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() \
            and cos.shape == (x.shape[0], x.shape[1], x.shape[3]) and x.numel() > 0:
        return _RopeFn.apply(x, cos, sin)
    return rope_reference(x, cos, sin)

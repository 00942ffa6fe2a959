"""Autograd wrappers of the channels-last sub-sampling kernels (``csrc/subsampling.cu``).

The FastConformer front end (reference ``nemo/collections/asr/parts/submodules/subsampling.py:184-257``: Conv2d(1->C, 3, s2) +
ReLU, then [depthwise Conv2d(C, 3, s2) + pointwise Conv2d(C, 1) + ReLU] per further halving, masking between layers) runs as

    conv1 + ReLU (kernel)  ->  depthwise (kernel)  ->  pointwise + ReLU (tcgen05 GEMM)  ->  ...  ->  masked flatten (kernel)

with activations in ``[B, T, F, C]`` bf16.  Parameter gradients are accumulated straight into the optimizer arena when the
parameters live in one (``param._grad_view``), as the GEMM wrappers do; otherwise autograd receives fresh tensors.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import native
from .native import _check, _ptr, _stream, lib


def _i(v):
    return ctypes.c_int(int(v))


def _ll(v):
    return ctypes.c_longlong(int(v))


def _grad_target(param: torch.Tensor):
    """(fp32 buffer to accumulate into, True if it is the arena's own view)."""
    gv = getattr(param, "_grad_view", None)
    if gv is not None and gv.is_cuda:
        return gv.view(-1), True
    return torch.zeros(param.numel(), dtype=torch.float32, device=param.device), False


def _grad_done(param: torch.Tensor, buf: torch.Tensor, in_arena: bool):
    if in_arena:
        arena = getattr(param, "_arena", None)
        cb = getattr(arena, "grad_ready", None) if arena is not None else None
        if cb is not None:
            cb(param)
        return None
    return buf.view(param.shape)


def out_extent(n: int, pad_total: int) -> int:
    return (n + pad_total - 3) // 2 + 1


class _Conv1DwFn(torch.autograd.Function):
    """features -> conv1 + ReLU -> depthwise conv; the first layer's backward is fused into the depthwise backward."""

    @staticmethod
    def forward(ctx, x, L0, L1, L2, w0, b0, wdw, bdw, pad, pad_total):
        B, T, F = x.shape
        C = w0.shape[0]
        xf = x if x.dtype == torch.float32 else x.float()
        T1, F1 = out_extent(T, pad_total), out_extent(F, pad_total)
        T2, F2 = out_extent(T1, pad_total), out_extent(F1, pad_total)
        y1 = torch.empty((B, T1, F1, C), dtype=torch.bfloat16, device=x.device)
        z2 = torch.empty((B, T2, F2, C), dtype=torch.bfloat16, device=x.device)
        w0f, wdwf = w0.detach().reshape(-1).float(), wdw.detach().reshape(-1).float()
        b0f = b0.detach().float() if b0 is not None else None
        bdwf = bdw.detach().float() if bdw is not None else None
        _check(lib().sb_subs_conv1_fwd(_ptr(xf), _ll(xf.stride(0)), _ll(xf.stride(1)), _ll(xf.stride(2)), _ptr(L0), _ptr(L1), _ptr(w0f),
                                       _ptr(b0f), _ptr(y1), _i(B), _i(T), _i(F), _i(T1), _i(F1), _i(C), _i(pad), _stream()),
               "sb_subs_conv1_fwd")
        _check(lib().sb_subs_dw_fwd(_ptr(y1), _ptr(L1), _ptr(L2), _ptr(wdwf), _ptr(bdwf), _ptr(z2), _i(B), _i(T1), _i(F1), _i(T2), _i(F2),
                                    _i(C), _i(pad), _stream()), "sb_subs_dw_fwd")
        native.launch_count += 2
        ctx.save_for_backward(xf, L0, L1, L2, y1, wdwf)
        ctx.params = (w0, b0, wdw, bdw)
        ctx.pad = pad
        return z2

    @staticmethod
    def backward(ctx, dz2):
        xf, L0, L1, L2, y1, wdwf = ctx.saved_tensors
        w0, b0, wdw, bdw = ctx.params
        B, T, F = xf.shape
        _, T1, F1, C = y1.shape
        _, T2, F2, _ = dz2.shape
        dz2 = dz2.contiguous()
        gw, gw_a = _grad_target(wdw)
        gb, gb_a = _grad_target(bdw) if bdw is not None else (torch.zeros(C, device=xf.device), False)
        gw0, gw0_a = _grad_target(w0)
        gb0, gb0_a = _grad_target(b0) if b0 is not None else (torch.zeros(C, device=xf.device), False)
        _check(lib().sb_subs_dw_bwd(_ptr(dz2), _ptr(y1), _ptr(L1), _ptr(L2), _ptr(wdwf), None, _ptr(gw), _ptr(gb), _i(B), _i(T1), _i(F1),
                                    _i(T2), _i(F2), _i(C), _i(ctx.pad), _ptr(xf), _ll(xf.stride(0)), _ll(xf.stride(1)),
                                    _ll(xf.stride(2)), _ptr(L0), _i(T), _i(F), _i(ctx.pad), _ptr(gw0), _ptr(gb0), _stream()),
               "sb_subs_dw_bwd")
        native.launch_count += 1
        return (None, None, None, None, _grad_done(w0, gw0, gw0_a), _grad_done(b0, gb0, gb0_a) if b0 is not None else None,
                _grad_done(wdw, gw, gw_a), _grad_done(bdw, gb, gb_a) if bdw is not None else None, None, None)


class _DwFn(torch.autograd.Function):
    """Depthwise 3x3 / stride-2 convolution over ``[B, T, F, C]`` with length masks on both sides."""

    @staticmethod
    def forward(ctx, yin, Lin, Lout, wdw, bdw, pad, pad_total):
        B, Ti, Fi, C = yin.shape
        To, Fo = out_extent(Ti, pad_total), out_extent(Fi, pad_total)
        yin = yin.contiguous()
        z = torch.empty((B, To, Fo, C), dtype=torch.bfloat16, device=yin.device)
        wf = wdw.detach().reshape(-1).float()
        bf = bdw.detach().float() if bdw is not None else None
        _check(lib().sb_subs_dw_fwd(_ptr(yin), _ptr(Lin), _ptr(Lout), _ptr(wf), _ptr(bf), _ptr(z), _i(B), _i(Ti), _i(Fi), _i(To), _i(Fo),
                                    _i(C), _i(pad), _stream()), "sb_subs_dw_fwd")
        native.launch_count += 1
        ctx.save_for_backward(yin, Lin, Lout, wf)
        ctx.params = (wdw, bdw)
        ctx.pad = pad
        return z

    @staticmethod
    def backward(ctx, dz):
        yin, Lin, Lout, wf = ctx.saved_tensors
        wdw, bdw = ctx.params
        B, Ti, Fi, C = yin.shape
        _, To, Fo, _ = dz.shape
        dz = dz.contiguous()
        dyin = torch.empty_like(yin)
        gw, gw_a = _grad_target(wdw)
        gb, gb_a = _grad_target(bdw) if bdw is not None else (torch.zeros(C, device=yin.device), False)
        _check(lib().sb_subs_dw_bwd(_ptr(dz), _ptr(yin), _ptr(Lin), _ptr(Lout), _ptr(wf), _ptr(dyin), _ptr(gw), _ptr(gb), _i(B), _i(Ti),
                                    _i(Fi), _i(To), _i(Fo), _i(C), _i(ctx.pad), None, _ll(0), _ll(0), _ll(0), None, _i(0), _i(0), _i(0),
                                    None, None, _stream()), "sb_subs_dw_bwd")
        native.launch_count += 1
        return (dyin, None, None, _grad_done(wdw, gw, gw_a), _grad_done(bdw, gb, gb_a) if bdw is not None else None, None, None)


class _MaskFlattenFn(torch.autograd.Function):
    """``[B, T, F, C] -> [B, T, C * F]`` in the reference's channel-major order, rows beyond each length zeroed."""

    @staticmethod
    def forward(ctx, y, L):
        B, T, F, C = y.shape
        y = y.contiguous()
        out = torch.empty((B, T, C * F), dtype=y.dtype, device=y.device)
        _check(lib().sb_subs_mask_transpose(_ptr(y), _ptr(L), _ptr(out), _i(B), _i(T), _i(F), _i(C), _stream()), "sb_subs_mask_transpose")
        native.launch_count += 1
        ctx.save_for_backward(L)
        ctx.shape = (B, T, F, C)
        return out

    @staticmethod
    def backward(ctx, dout):
        (L,) = ctx.saved_tensors
        B, T, F, C = ctx.shape
        dout = dout.contiguous()
        dy = torch.empty((B, T, F, C), dtype=dout.dtype, device=dout.device)
        _check(lib().sb_subs_mask_transpose(_ptr(dout), _ptr(L), _ptr(dy), _i(B), _i(T), _i(C), _i(F), _stream()), "sb_subs_mask_transpose")
        native.launch_count += 1
        return dy, None


def supported(channels: int, sampling_num: int, feat_in: int) -> bool:
    return channels % 8 == 0 and 8 <= channels <= 512 and 256 % (channels // 8) == 0 and sampling_num >= 2 and feat_in >= 8


def dw_striding_forward(x: torch.Tensor, lengths: torch.Tensor, conv_layers: List[torch.nn.Module], out_weight, out_bias, causal: bool):
    """Whole front end.  ``conv_layers`` = [conv1, dw, pw, dw, pw, ...] (activation modules left out).  Returns
    ``([B, T', d_model] bf16, lengths')``."""
    from . import linear

    pad, pad_total = (2, 3) if causal else (1, 2)
    L = [lengths.to(torch.int64).contiguous()]
    n_stages = 1 + (len(conv_layers) - 1) // 2
    for _ in range(n_stages):
        L.append(torch.div(L[-1] + pad_total - 3, 2, rounding_mode="floor") + 1)
    conv1, dw, pw = conv_layers[0], conv_layers[1], conv_layers[2]
    z = _Conv1DwFn.apply(x, L[0], L[1], L[2], conv1.weight, conv1.bias, dw.weight, dw.bias, pad, pad_total)
    B, T2, F2, C = z.shape
    y = linear(z.view(B * T2 * F2, C), pw.weight, pw.bias, act="relu").view(B, T2, F2, -1)
    for s in range(2, n_stages):
        dw, pw = conv_layers[2 * s - 1], conv_layers[2 * s]
        z = _DwFn.apply(y, L[s], L[s + 1], dw.weight, dw.bias, pad, pad_total)
        Bz, Tz, Fz, Cz = z.shape
        y = linear(z.view(Bz * Tz * Fz, Cz), pw.weight, pw.bias, act="relu").view(Bz, Tz, Fz, -1)
    flat = _MaskFlattenFn.apply(y, L[n_stages])
    return linear(flat, out_weight, out_bias), L[n_stages]

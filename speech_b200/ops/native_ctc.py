"""CTC loss on the kernels of csrc/ctc.cu (per-utterance negative log-likelihood, gradient w.r.t. the log-probs)."""
from __future__ import annotations

import ctypes

import torch

from . import native as N


def _i(x):
    return ctypes.c_int(int(x))


def _ll(x):
    return ctypes.c_longlong(int(x))


class _CTCFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, log_probs, targets, in_len, tgt_len, blank, zero_infinity):
        B, T, V = log_probs.shape
        dev = log_probs.device
        lp = log_probs.float().contiguous()
        targets = targets.long().contiguous()
        in_len = in_len.long().clamp(max=T).contiguous()
        tgt_len = tgt_len.long().clamp(max=targets.shape[1]).contiguous()
        Smax = 2 * targets.shape[1] + 1
        alpha = torch.empty((B, T, Smax), dtype=torch.float32, device=dev)
        beta = torch.empty((B, T, Smax), dtype=torch.float32, device=dev)
        nll = torch.empty(B, dtype=torch.float32, device=dev)
        N._check(N.lib().sb_ctc_forward(N._ptr(lp), _ll(V), _ll(T * V), N._ptr(targets), _i(targets.shape[1]), N._ptr(in_len),
                                        N._ptr(tgt_len), N._ptr(alpha), N._ptr(beta), N._ptr(nll), _i(B), _i(T), _i(Smax), _i(blank),
                                        _i(1 if zero_infinity else 0), N._stream()), "sb_ctc_forward")
        ctx.save_for_backward(lp, targets, in_len, tgt_len, alpha, beta, nll)
        ctx.cfg = (B, T, V, Smax, blank, log_probs.dtype)
        return nll.clone()

    @staticmethod
    def backward(ctx, dloss):
        lp, targets, in_len, tgt_len, alpha, beta, nll = ctx.saved_tensors
        B, T, V, Smax, blank, dtype = ctx.cfg
        grad = torch.zeros((B, T, V), dtype=torch.float32, device=lp.device)
        up = dloss.float().contiguous()
        N._check(N.lib().sb_ctc_backward(N._ptr(lp), _ll(V), _ll(T * V), N._ptr(targets), _i(targets.shape[1]), N._ptr(in_len),
                                         N._ptr(tgt_len), N._ptr(alpha), N._ptr(beta), N._ptr(nll), N._ptr(up), N._ptr(grad), _ll(V),
                                         _ll(T * V), _i(B), _i(T), _i(Smax), _i(blank), N._stream()), "sb_ctc_backward")
        return grad.to(dtype), None, None, None, None, None


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank, zero_infinity=True):
    if 2 * targets.shape[1] + 1 > 1024:
        from . import reference

        return reference.ctc_loss(log_probs, targets, input_lengths, target_lengths, blank, zero_infinity)
    return _CTCFn.apply(log_probs, targets, input_lengths, target_lengths, int(blank), bool(zero_infinity))

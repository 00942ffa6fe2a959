"""Fused joint + RNNT/TDT loss on the sm_100a kernels (see csrc/transducer.cu).

The joint's output layer is evaluated a few utterances at a time (chunks sized to stay L2-resident) with the tcgen05
GEMM; only per-node scalars (log-sum-exps and the blank / label / duration log-probs) survive a chunk, so the
``B x T x U x V`` logits tensor never exists.  Backward recomputes each chunk's logits, forms d(logits) in bf16 and
feeds it straight into the two gradient GEMMs (``dH = dZ W`` with the ReLU mask in its epilogue, ``dW += dZ^T H``).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import native as N

CHUNK_ROWS = 16384


def _i(x):
    return ctypes.c_int(int(x))


def _dur_array(durations: Sequence[int]):
    arr = (ctypes.c_int * 8)(*([int(d) for d in durations] + [0] * (8 - len(durations))))
    return arr


FREE_LABEL = 256     # flag on the duration count: multi-blank arc model (see csrc/transducer.cu, struct Durations)


def _lattice_forward(lpb, lpl, lpd, f_len, y_len, B, T, U1, durations, need_beta: bool, flag: int = 0):
    dev = lpb.device
    alpha = torch.empty((B, T, U1), dtype=torch.float32, device=dev)
    beta = torch.empty((B, T, U1), dtype=torch.float32, device=dev) if need_beta else None
    ll = torch.empty(B, dtype=torch.float32, device=dev)
    N._check(N.lib().sb_transducer_alpha_beta(N._ptr(lpb), N._ptr(lpl), N._ptr(lpd), N._ptr(f_len), N._ptr(y_len), N._ptr(alpha),
                                              N._ptr(beta), N._ptr(ll), _i(B), _i(T), _i(U1), _dur_array(durations),
                                              _i(len(durations) + flag), N._stream()), "sb_transducer_alpha_beta")
    return alpha, beta, ll


def _node_grads(lpb, lpl, lpd, alpha, beta, ll, upstream, f_len, y_len, B, T, U1, durations, fastemit, flag: int = 0):
    dev = lpb.device
    D = len(durations)
    gb = torch.empty((B, T, U1), dtype=torch.float32, device=dev)
    gl = torch.empty((B, T, U1), dtype=torch.float32, device=dev)
    gd = torch.empty((B, T, U1, max(D, 1)), dtype=torch.float32, device=dev)
    N._check(N.lib().sb_transducer_node_grads(N._ptr(lpb), N._ptr(lpl), N._ptr(lpd), N._ptr(alpha), N._ptr(beta), N._ptr(ll),
                                              N._ptr(upstream), N._ptr(f_len), N._ptr(y_len), N._ptr(gb), N._ptr(gl), N._ptr(gd),
                                              _i(B), _i(T), _i(U1), _dur_array(durations), _i(D + flag), ctypes.c_float(fastemit),
                                              N._stream()), "sb_transducer_node_grads")
    return gb, gl, gd


class _JointLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f, g, weight, bias, targets, f_len, y_len, blank, durations, sigma, fastemit, drop_p=0.0):
        B, T, Hj = f.shape
        U1 = g.shape[1]
        dev = f.device
        D = len(durations)
        wl = N._lowp_weight(weight)            # [V, Hj]
        V = wl.shape[0]
        V1 = V - D
        f = f.contiguous()
        g = g.contiguous()
        targets = targets.long().contiguous()
        f_len = f_len.long().contiguous()
        y_len = y_len.long().contiguous()
        nodes = B * T * U1
        lse_tok = torch.empty(nodes, dtype=torch.float32, device=dev)
        lse_dur = torch.empty(nodes, dtype=torch.float32, device=dev) if D else None
        lpb = torch.empty(nodes, dtype=torch.float32, device=dev)
        lpl = torch.empty(nodes, dtype=torch.float32, device=dev)
        lpd = torch.empty((nodes, D), dtype=torch.float32, device=dev) if D else None
        nb_chunk = max(1, CHUNK_ROWS // (T * U1))
        ldz = (V + 3) // 4 * 4
        rows_max = min(B, nb_chunk) * T * U1
        h = torch.empty((rows_max, Hj), dtype=torch.bfloat16, device=dev)
        z = torch.empty((rows_max, ldz), dtype=torch.float32, device=dev)
        drop_p = float(drop_p)
        seed = N._next_dropout_seed() if drop_p > 0.0 else 0
        for b0 in range(0, B, nb_chunk):
            nb = min(nb_chunk, B - b0)
            rows = nb * T * U1
            N._check(N.lib().sb_joint_build_h(N._ptr(f), N._ptr(g), N._ptr(h), _i(b0), _i(nb), _i(T), _i(U1), _i(Hj),
                                              ctypes.c_longlong(T * Hj), ctypes.c_longlong(U1 * Hj), ctypes.c_float(drop_p),
                                              ctypes.c_ulonglong(seed), N._stream()), "sb_joint_build_h")
            N.gemm(h, wl, z, M=rows, N=V, K=Hj, ldd=ldz, bias=bias)
            N._check(N.lib().sb_joint_lse_gather(N._ptr(z), _i(ldz), N._ptr(targets), _i(targets.shape[1]), N._ptr(lse_tok),
                                                 N._ptr(lse_dur), N._ptr(lpb), N._ptr(lpl), N._ptr(lpd), _i(b0), _i(nb), _i(T),
                                                 _i(U1), _i(V1), _i(D), _i(blank), ctypes.c_float(sigma), N._stream()),
                     "sb_joint_lse_gather")
        need_grad = any(ctx.needs_input_grad[:4])
        alpha, beta, ll = _lattice_forward(lpb, lpl, lpd, f_len, y_len, B, T, U1, durations, need_grad)
        ctx.save_for_backward(f, g, targets, f_len, y_len, lse_tok, lse_dur, lpb, lpl, lpd, alpha, beta, ll)
        ctx.weight, ctx.bias = weight, bias
        ctx.cfg = (B, T, U1, Hj, V, V1, D, blank, list(durations), fastemit, nb_chunk, ldz)
        ctx.drop = (drop_p, seed)
        loss = -ll
        return loss * (1.0 + fastemit) if fastemit else loss

    @staticmethod
    def backward(ctx, dloss):
        f, g, targets, f_len, y_len, lse_tok, lse_dur, lpb, lpl, lpd, alpha, beta, ll = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        B, T, U1, Hj, V, V1, D, blank, durations, fastemit, nb_chunk, ldz = ctx.cfg
        drop_p, seed = ctx.drop
        drop_scale = 1.0
        if drop_p > 0.0:
            t8 = min(255, int(drop_p * 256.0 + 0.5))          # the kernels' 8-bit threshold (common.cuh, sb_dropout_threshold)
            drop_scale = 256.0 / (256.0 - t8) if t8 else 1.0
        dev = f.device
        wl = N._lowp_weight(weight)
        up = dloss.float().contiguous()
        gb, gl, gd = _node_grads(lpb, lpl, lpd, alpha, beta, ll, up, f_len, y_len, B, T, U1, durations, fastemit)
        lddz = (V + 7) // 8 * 8
        rows_max = min(B, nb_chunk) * T * U1
        h = torch.empty((rows_max, Hj), dtype=torch.bfloat16, device=dev)
        z = torch.empty((rows_max, ldz), dtype=torch.float32, device=dev)
        dz = torch.empty((rows_max, lddz), dtype=torch.bfloat16, device=dev)
        dh = torch.empty((rows_max, Hj), dtype=torch.bfloat16, device=dev)
        df = torch.empty((B, T, Hj), dtype=torch.float32, device=dev)
        dg = torch.empty((B, U1, Hj), dtype=torch.float32, device=dev)
        gw = getattr(weight, "_grad_view", None)
        direct_w = gw is not None and gw.is_cuda
        dW = gw.view(V, Hj) if direct_w else torch.zeros((V, Hj), dtype=torch.float32, device=dev)
        gbv = getattr(bias, "_grad_view", None) if bias is not None else None
        direct_b = gbv is not None and gbv.is_cuda
        dB = (gbv if direct_b else torch.zeros(V, dtype=torch.float32, device=dev)) if bias is not None else None
        for b0 in range(0, B, nb_chunk):
            nb = min(nb_chunk, B - b0)
            rows = nb * T * U1
            N._check(N.lib().sb_joint_build_h(N._ptr(f), N._ptr(g), N._ptr(h), _i(b0), _i(nb), _i(T), _i(U1), _i(Hj),
                                              ctypes.c_longlong(T * Hj), ctypes.c_longlong(U1 * Hj), ctypes.c_float(drop_p),
                                              ctypes.c_ulonglong(seed), N._stream()), "sb_joint_build_h")
            N.gemm(h, wl, z, M=rows, N=V, K=Hj, ldd=ldz, bias=bias)
            N._check(N.lib().sb_joint_dlogits(N._ptr(z), _i(ldz), N._ptr(targets), _i(targets.shape[1]), N._ptr(lse_tok),
                                              N._ptr(lse_dur), N._ptr(gb), N._ptr(gl), N._ptr(gd), N._ptr(dz), _i(lddz), _i(b0),
                                              _i(nb), _i(T), _i(U1), _i(V1), _i(D), _i(blank), ctypes.c_float(-1.0), N._stream()),
                     "sb_joint_dlogits")
            # dH = scale * dZ W, masked by relu'(h): dropped units are zero in h, so the same mask removes them
            N.gemm(dz, wl, dh, M=rows, N=Hj, K=V, lda=lddz, b_mn=True, ldb=Hj, aux=h, dact="relu", ldx=Hj, alpha=drop_scale)
            # dW += dZ^T H
            N.gemm(dz, h, dW, M=V, N=Hj, K=rows, a_mn=True, lda=lddz, b_mn=True, ldb=Hj, beta=1.0)
            if dB is not None:
                N.colsum(dz[:rows, :V], dB, accumulate=True)
            N._check(N.lib().sb_joint_reduce_dh(N._ptr(dh), N._ptr(df), N._ptr(dg), _i(b0), _i(nb), _i(T), _i(U1), _i(Hj),
                                                N._stream()), "sb_joint_reduce_dh")
        arena = getattr(weight, "_arena", None)
        cb = getattr(arena, "grad_ready", None) if arena is not None else None
        if cb is not None:
            if direct_w:
                cb(weight)
            if direct_b:
                cb(bias)
        return (df.to(torch.bfloat16), dg.to(torch.bfloat16), None if direct_w else dW.view(weight.shape),
                None if (bias is None or direct_b) else dB, None, None, None, None, None, None, None, None)


def transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank, durations, sigma, fastemit_lambda=0.0, dropout_p=0.0):
    """Per-utterance negative log-likelihood; f: [B,T,H], g: [B,U+1,H] (bf16), w: [V+1+D, H], b: [V+1+D].  ``dropout_p`` is the
    joint network's dropout (applied to the hidden lattice after the activation)."""
    Hj = f.shape[-1]
    if Hj % 8 != 0 or g.shape[1] > 1024 or len(durations) > 8:
        from . import reference

        return reference.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank, durations, sigma, "relu",
                                               fastemit_lambda, 4)
    T_max = f.shape[1]
    return _JointLossFn.apply(f, g, w, b, targets, f_len.clamp(max=T_max), y_len, int(blank), tuple(durations), float(sigma),
                              float(fastemit_lambda), float(dropout_p))


class _LatticeLossFn(torch.autograd.Function):
    """Loss from materialised joint logits [B,T,U1,V] (non-fused joint): same lattice kernels, one chunk = everything."""

    @staticmethod
    def forward(ctx, logits, targets, f_len, y_len, blank, durations, sigma):
        B, T, U1, V = logits.shape
        D = len(durations)
        V1 = V - D
        dev = logits.device
        z = logits.float().contiguous().view(B * T * U1, V)
        targets = targets.long().contiguous()
        f_len, y_len = f_len.long().contiguous(), y_len.long().contiguous()
        nodes = B * T * U1
        lse_tok = torch.empty(nodes, dtype=torch.float32, device=dev)
        lse_dur = torch.empty(nodes, dtype=torch.float32, device=dev) if D else None
        lpb = torch.empty(nodes, dtype=torch.float32, device=dev)
        lpl = torch.empty(nodes, dtype=torch.float32, device=dev)
        lpd = torch.empty((nodes, D), dtype=torch.float32, device=dev) if D else None
        N._check(N.lib().sb_joint_lse_gather(N._ptr(z), _i(V), N._ptr(targets), _i(targets.shape[1]), N._ptr(lse_tok), N._ptr(lse_dur),
                                             N._ptr(lpb), N._ptr(lpl), N._ptr(lpd), _i(0), _i(B), _i(T), _i(U1), _i(V1), _i(D),
                                             _i(blank), ctypes.c_float(sigma), N._stream()), "sb_joint_lse_gather")
        alpha, beta, ll = _lattice_forward(lpb, lpl, lpd, f_len, y_len, B, T, U1, durations, ctx.needs_input_grad[0])
        ctx.save_for_backward(z, targets, f_len, y_len, lse_tok, lse_dur, lpb, lpl, lpd, alpha, beta, ll)
        ctx.cfg = (B, T, U1, V, V1, D, blank, list(durations), logits.dtype)
        return -ll

    @staticmethod
    def backward(ctx, dloss):
        z, targets, f_len, y_len, lse_tok, lse_dur, lpb, lpl, lpd, alpha, beta, ll = ctx.saved_tensors
        B, T, U1, V, V1, D, blank, durations, dtype = ctx.cfg
        gb, gl, gd = _node_grads(lpb, lpl, lpd, alpha, beta, ll, dloss.float().contiguous(), f_len, y_len, B, T, U1, durations, 0.0)
        lddz = (V + 7) // 8 * 8
        dz = torch.empty((B * T * U1, lddz), dtype=torch.bfloat16, device=z.device)
        N._check(N.lib().sb_joint_dlogits(N._ptr(z), _i(V), N._ptr(targets), _i(targets.shape[1]), N._ptr(lse_tok), N._ptr(lse_dur),
                                          N._ptr(gb), N._ptr(gl), N._ptr(gd), N._ptr(dz), _i(lddz), _i(0), _i(B), _i(T), _i(U1),
                                          _i(V1), _i(D), _i(blank), ctypes.c_float(-1.0), N._stream()), "sb_joint_dlogits")
        return dz[:, :V].reshape(B, T, U1, V).to(dtype), None, None, None, None, None, None


def transducer_loss_from_logits(logits, targets, f_len, y_len, blank, durations, sigma=0.0):
    if logits.shape[2] > 1024 or len(durations) > 8:
        from . import reference

        return reference.tdt_loss_from_logits(logits, targets, f_len, y_len, blank, durations, sigma)
    return _LatticeLossFn.apply(logits, targets, f_len, y_len, int(blank), tuple(durations), float(sigma))


class _MultiBlankLatticeFn(torch.autograd.Function):
    """Multi-blank RNNT lattice on the native wavefront kernels: ``arcs`` [B, T, U1, n] are the log-probs of the blank symbols
    (the standard blank first), ``label`` [B, T, U1] those of the next target token; returns the negative log-likelihood per
    utterance and, in backward, the occupancy-weighted gradients of both."""

    @staticmethod
    def forward(ctx, arcs, label, f_len, y_len, durations):
        B, T, U1, D = arcs.shape
        arcs, label = arcs.float().contiguous(), label.float().contiguous()
        f_len, y_len = f_len.long().contiguous(), y_len.long().contiguous()
        zero = torch.zeros_like(label)
        alpha, beta, ll = _lattice_forward(zero, label, arcs, f_len, y_len, B, T, U1, durations, True, FREE_LABEL)
        ctx.save_for_backward(zero, label, arcs, alpha, beta, ll, f_len, y_len)
        ctx.durations = list(durations)
        return -ll

    @staticmethod
    def backward(ctx, dloss):
        zero, label, arcs, alpha, beta, ll, f_len, y_len = ctx.saved_tensors
        B, T, U1, D = arcs.shape
        _, gl, gd = _node_grads(zero, label, arcs, alpha, beta, ll, dloss.float().contiguous(), f_len, y_len, B, T, U1, ctx.durations,
                                0.0, FREE_LABEL)
        return gd, gl, None, None, None


def multiblank_loss_from_logits(logits, targets, f_len, y_len, blank: int, big_blank_durations: Sequence[int], sigma: float = 0.0):
    """Multi-blank RNNT loss (reference ``losses/rnnt.py`` ``multiblank_rnnt`` on the Numba kernels ``gpu_rnnt_kernel.py:411,570,720``):
    the big-blank symbols sit right before the standard blank in the vocabulary; one log-softmax over all symbols, minus sigma."""
    B, T, U1, _ = logits.shape
    nb = len(big_blank_durations)
    if U1 > 1024 or nb + 1 > 8:
        from . import reference

        return reference.multiblank_loss_from_logits(logits, targets, f_len, y_len, blank, big_blank_durations, sigma)
    tok = torch.log_softmax(logits.float(), dim=-1) - sigma
    arcs = torch.stack([tok[..., blank]] + [tok[..., blank - nb + i] for i in range(nb)], dim=-1)
    tgt = torch.cat([targets, targets.new_zeros(B, 1)], dim=1).clamp(min=0).long()
    label = torch.gather(tok, 3, tgt[:, None, :, None].expand(B, T, U1, 1)).squeeze(-1)
    return _MultiBlankLatticeFn.apply(arcs, label, f_len, y_len, (1,) + tuple(int(d) for d in big_blank_durations))

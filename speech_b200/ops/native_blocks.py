"""Autograd wrappers for the attention and convolution-module kernel pipelines.

Attention (Transformer-XL relative-position, and the plain variant) is a sequence of batched tcgen05 GEMMs with the
softmax / rel-shift / mask / dropout kernel in between; the backward pass is built from the same GEMM kernel in its
MN-major operand modes, so no tensor is ever transposed in memory.  Per (batch, head) problems are addressed through
the GEMM's two batch indices with the strides of the [B, T, H, dk] layout (or of a fused [B, T, 3, H, dk] QKV buffer).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import native as N


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


def _bhd(t: torch.Tensor) -> Tuple[int, int, int]:
    """(row stride, head stride, batch stride) in elements of a [B, T, H, dk] view with contiguous dk."""
    assert t.stride(3) == 1
    return t.stride(1), t.stride(2), t.stride(0)


def _gemm_ok(t: torch.Tensor) -> bool:
    return t.stride(3) == 1 and t.stride(1) % 8 == 0 and t.stride(2) % 8 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def _prep_mask(mask, B, Tq, Tk):
    if mask is None:
        return None, 0
    m = mask
    if m.dim() == 4:
        m = m[:, 0]
    m = m.to(torch.uint8).contiguous()
    assert m.shape[-2:] == (Tq, Tk), f"mask shape {tuple(m.shape)} vs ({Tq},{Tk})"
    return m, (Tq if m.shape[0] > 1 else 0)


class _AttentionFn(torch.autograd.Function):
    """ctx = softmax(((q+u) k^T + shift((q+v) p^T)) / sqrt(dk)) v ; with p=None it is plain attention."""

    @staticmethod
    def forward(ctx, q, k, v, p, bias_u, bias_v, mask, scale, drop_p, seed):
        ctx.fused = k is None  # q is then a fused [B, T, 3, H, dk] buffer: one input, one gradient
        if ctx.fused:
            qkv = q if _gemm_ok(q[:, :, 0]) else q.contiguous()
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        B, Tq, H, dk = q.shape
        Tk = k.shape[1]
        dev = q.device
        rel = p is not None
        q = q if _gemm_ok(q) else q.contiguous()
        k = k if _gemm_ok(k) else k.contiguous()
        v = v if _gemm_ok(v) else v.contiguous()
        HD = H * dk
        if rel:
            P = p.shape[1]
            p = p if _gemm_ok(p) else p.contiguous()
            qu = torch.empty((B, Tq, H, dk), dtype=torch.bfloat16, device=dev)
            qv = torch.empty((B, Tq, H, dk), dtype=torch.bfloat16, device=dev)
            if q.stride(2) != dk:
                q = q.contiguous()
            N._check(N.lib().sb_add_pos_bias(N._ptr(q), ctypes.c_longlong(q.stride(1)), N._ptr(bias_u), N._ptr(bias_v),
                                             N._ptr(qu), N._ptr(qv), ctypes.c_longlong(B * Tq), ctypes.c_int(HD), N._stream())
                     if q.stride(0) == Tq * q.stride(1) else -77, "sb_add_pos_bias")
        else:
            qu, qv, P = q, None, 0
        ldac = _round8(Tk)
        AC = torch.empty((B, H, Tq, ldac), dtype=torch.float32, device=dev)
        qs, ks = _bhd(qu), _bhd(k)
        N.gemm(qu, k, AC, M=Tq, N=Tk, K=dk, lda=qs[0], ldb=ks[0], ldd=ldac, batch=(H, B), a_bs=(qs[1], qs[2]),
               b_bs=(ks[1], ks[2]), d_bs=(Tq * ldac, H * Tq * ldac))
        BD, ldbd = None, 0
        if rel:
            ldbd = _round8(P)
            BD = torch.empty((B, H, Tq, ldbd), dtype=torch.float32, device=dev)
            ps = _bhd(p)
            vs_ = _bhd(qv)
            N.gemm(qv, p, BD, M=Tq, N=P, K=dk, lda=vs_[0], ldb=ps[0], ldd=ldbd, batch=(H, B), a_bs=(vs_[1], vs_[2]),
                   b_bs=(ps[1], ps[2] if p.shape[0] > 1 else 0), d_bs=(Tq * ldbd, H * Tq * ldbd))
        ldp = _round8(Tk)
        Pm = torch.empty((B, H, Tq, ldp), dtype=torch.bfloat16, device=dev)
        Pd = torch.empty_like(Pm) if drop_p > 0 else None
        m8, mbs = _prep_mask(mask, B, Tq, Tk)
        N._check(N.lib().sb_relpos_softmax_fwd(N._ptr(AC), N._ptr(BD), N._ptr(m8), ctypes.c_int(mbs), N._ptr(Pm), N._ptr(Pd),
                                               ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(Tq), ctypes.c_int(Tk),
                                               ctypes.c_int(ldac), ctypes.c_int(ldbd), ctypes.c_int(ldp), ctypes.c_float(scale),
                                               ctypes.c_float(drop_p), ctypes.c_ulonglong(seed), N._stream()),
                 "sb_relpos_softmax_fwd")
        out = torch.empty((B, Tq, H, dk), dtype=torch.bfloat16, device=dev)
        Pu = Pd if Pd is not None else Pm
        vs = _bhd(v)
        N.gemm(Pu, v, out, M=Tq, N=dk, K=Tk, lda=ldp, b_mn=True, ldb=vs[0], ldd=HD, batch=(H, B), a_bs=(Tq * ldp, H * Tq * ldp),
               b_bs=(vs[1], vs[2]), d_bs=(dk, Tq * HD))
        ctx.save_for_backward(qu, qv, k, v, p, Pm, Pd)
        ctx.bias_u, ctx.bias_v = bias_u, bias_v
        ctx.dims = (B, Tq, Tk, H, dk, P, ldp, ldbd)
        ctx.scale, ctx.drop_p, ctx.seed = scale, drop_p, seed
        del AC, BD
        return out.view(B, Tq, HD)

    @staticmethod
    def backward(ctx, dout):
        qu, qv, k, v, p, Pm, Pd = ctx.saved_tensors
        B, Tq, Tk, H, dk, P, ldp, ldbd = ctx.dims
        HD = H * dk
        dev = dout.device
        rel = p is not None
        do = dout.reshape(B, Tq, H, dk)
        if not _gemm_ok(do):
            do = do.contiguous()
        dos, vs, ks = _bhd(do), _bhd(v), _bhd(k)
        Pu = Pd if Pd is not None else Pm
        if ctx.fused:
            dqkv = torch.empty((B, Tq, 3, H, dk), dtype=torch.bfloat16, device=dev)
            dQ, dK, dV = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        else:
            dqkv = None
            dQ = torch.empty((B, Tq, H, dk), dtype=torch.bfloat16, device=dev)
            dK = torch.empty((B, Tk, H, dk), dtype=torch.bfloat16, device=dev)
            dV = torch.empty((B, Tk, H, dk), dtype=torch.bfloat16, device=dev)
        sQ, sK, sV = _bhd(dQ), _bhd(dK), _bhd(dV)
        # dV = Pu^T dO
        N.gemm(Pu, do, dV, M=Tk, N=dk, K=Tq, a_mn=True, lda=ldp, b_mn=True, ldb=dos[0], ldd=sV[0], batch=(H, B),
               a_bs=(Tq * ldp, H * Tq * ldp), b_bs=(dos[1], dos[2]), d_bs=(sV[1], sV[2]))
        # dPd = dO V^T
        lddp = _round8(Tk)
        dPd = torch.empty((B, H, Tq, lddp), dtype=torch.float32, device=dev)
        N.gemm(do, v, dPd, M=Tq, N=Tk, K=dk, lda=dos[0], ldb=vs[0], ldd=lddp, batch=(H, B), a_bs=(dos[1], dos[2]),
               b_bs=(vs[1], vs[2]), d_bs=(Tq * lddp, H * Tq * lddp))
        dAC = torch.empty((B, H, Tq, ldp), dtype=torch.bfloat16, device=dev)
        dBD = torch.empty((B, H, Tq, ldbd), dtype=torch.bfloat16, device=dev) if rel else None
        N._check(N.lib().sb_relpos_softmax_bwd(N._ptr(Pm), N._ptr(dPd), N._ptr(dAC), N._ptr(dBD), ctypes.c_int(B), ctypes.c_int(H),
                                               ctypes.c_int(Tq), ctypes.c_int(Tk), ctypes.c_int(ldp), ctypes.c_int(lddp),
                                               ctypes.c_int(ldbd), ctypes.c_float(ctx.scale), ctypes.c_float(ctx.drop_p),
                                               ctypes.c_ulonglong(ctx.seed), N._stream()), "sb_relpos_softmax_bwd")
        del dPd
        # dK = dAC^T (q+u)
        qs = _bhd(qu)
        N.gemm(dAC, qu, dK, M=Tk, N=dk, K=Tq, a_mn=True, lda=ldp, b_mn=True, ldb=qs[0], ldd=sK[0], batch=(H, B),
               a_bs=(Tq * ldp, H * Tq * ldp), b_bs=(qs[1], qs[2]), d_bs=(sK[1], sK[2]))
        dp = du = dv_bias = None
        if not rel:
            # dQ = dAC K
            N.gemm(dAC, k, dQ, M=Tq, N=dk, K=Tk, lda=ldp, b_mn=True, ldb=ks[0], ldd=sQ[0], batch=(H, B),
                   a_bs=(Tq * ldp, H * Tq * ldp), b_bs=(ks[1], ks[2]), d_bs=(sQ[1], sQ[2]))
        else:
            # dQu = dAC K ;  dQ = dBD p + dQu  (the sum is the second GEMM's residual epilogue)
            dQu = torch.empty((B, Tq, H, dk), dtype=torch.bfloat16, device=dev)
            N.gemm(dAC, k, dQu, M=Tq, N=dk, K=Tk, lda=ldp, b_mn=True, ldb=ks[0], ldd=HD, batch=(H, B),
                   a_bs=(Tq * ldp, H * Tq * ldp), b_bs=(ks[1], ks[2]), d_bs=(dk, Tq * HD))
            ps = _bhd(p)
            N.gemm(dBD, p, dQ, M=Tq, N=dk, K=P, lda=ldbd, b_mn=True, ldb=ps[0], ldd=sQ[0], batch=(H, B),
                   a_bs=(Tq * ldbd, H * Tq * ldbd), b_bs=(ps[1], ps[2] if p.shape[0] > 1 else 0), d_bs=(sQ[1], sQ[2]),
                   residual=dQu, ldr=HD, r_bs=(dk, Tq * HD))
            if ctx.needs_input_grad[3]:
                vs_ = _bhd(qv)
                if p.shape[0] == 1:
                    dp = torch.empty((1, P, H, dk), dtype=torch.bfloat16, device=dev)
                    N.gemm(dBD, qv, dp, M=P, N=dk, K=Tq, a_mn=True, lda=ldbd, b_mn=True, ldb=vs_[0], ldd=HD, batch=(H, B),
                           a_bs=(Tq * ldbd, H * Tq * ldbd), b_bs=(vs_[1], vs_[2]), d_bs=(dk, 0), fold_batch1=True)
                else:
                    dp = torch.empty((B, P, H, dk), dtype=torch.bfloat16, device=dev)
                    N.gemm(dBD, qv, dp, M=P, N=dk, K=Tq, a_mn=True, lda=ldbd, b_mn=True, ldb=vs_[0], ldd=HD, batch=(H, B),
                           a_bs=(Tq * ldbd, H * Tq * ldbd), b_bs=(vs_[1], vs_[2]), d_bs=(dk, P * HD))
            if ctx.needs_input_grad[4] or ctx.needs_input_grad[5]:
                # d(u) = colsum(dQu);  d(v) = colsum(dQ - dQu)
                su = torch.zeros(HD, dtype=torch.float32, device=dev)
                sq = torch.zeros(HD, dtype=torch.float32, device=dev)
                N.colsum(dQu.view(B * Tq, HD), su, accumulate=True)
                dq2 = dQ.reshape(B * Tq, HD) if not ctx.fused else torch.as_strided(dQ, (B * Tq, HD), (sQ[0], 1))
                N.colsum(dq2, sq, accumulate=True)
                du = N._write_param_grad(ctx.bias_u, lambda out, beta: out.view(-1).add_(su) if beta else out.view(-1).copy_(su), (H, dk))
                dv_bias = N._write_param_grad(ctx.bias_v, lambda out, beta: out.view(-1).add_(sq - su) if beta else out.view(-1).copy_(sq - su), (H, dk))
        if ctx.fused:
            return dqkv, None, None, dp, du, dv_bias, None, None, None, None
        return dQ, dK, dV, dp, du, dv_bias, None, None, None, None


_seed_counter = [0x1234567]


def _next_seed() -> int:
    _seed_counter[0] = (_seed_counter[0] * 6364136223846793005 + 1442695040888963407) & ((1 << 63) - 1)
    return _seed_counter[0]


def relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask=None, dropout_p: float = 0.0, training: bool = False, qkv=None):
    """``qkv``: optional fused [B, T, 3, H, dk] buffer that q, k and v are slices of (self-attention without a cache); it is
    then the single differentiable input, which keeps autograd from assembling three padded gradient tensors."""
    dk = q.shape[-1]
    if dk % 8 != 0:
        from . import reference

        return reference.relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask, dropout_p, training)
    drop = float(dropout_p) if training else 0.0
    if qkv is not None:
        return _AttentionFn.apply(qkv, None, None, p.to(torch.bfloat16), pos_bias_u, pos_bias_v, mask, 1.0 / math.sqrt(dk),
                                  drop, _next_seed() if drop > 0 else 0)
    return _AttentionFn.apply(q, k, v, p.to(torch.bfloat16), pos_bias_u, pos_bias_v, mask, 1.0 / math.sqrt(dk), drop,
                              _next_seed() if drop > 0 else 0)


def mha_attention(q, k, v, mask=None, scale=None, dropout_p: float = 0.0, training: bool = False):
    dk = q.shape[-1]
    if dk % 8 != 0:
        from . import reference

        return reference.mha_attention(q, k, v, mask, dropout_p, training, scale)
    drop = float(dropout_p) if training else 0.0
    return _AttentionFn.apply(q, k, v, None, None, None, mask, scale if scale is not None else 1.0 / math.sqrt(dk), drop,
                              _next_seed() if drop > 0 else 0)


# ------------------------------------------------------------------------------------------------ conv module core
class _ConvCoreFn(torch.autograd.Function):
    """s = silu(BatchNorm(dwconv(mask(glu(g))))) on channels-last activations (see csrc/convmod.cu)."""

    @staticmethod
    def forward(ctx, g, dw_weight, dw_bias, gamma, beta, running_mean, running_var, pad_mask, training, momentum, eps,
                left_pad, stats_reduce):
        B, T, C2 = g.shape
        C = C2 // 2
        K = dw_weight.shape[-1]
        dev = g.device
        g = g.contiguous()
        w2 = dw_weight.reshape(C, K).contiguous()
        pad8 = pad_mask.to(torch.uint8).contiguous() if pad_mask is not None else None
        y = torch.empty((B, T, C), dtype=torch.bfloat16, device=dev)
        stats = torch.zeros(2 * C + 1, dtype=torch.float32, device=dev) if training else None
        N._check(N.lib().sb_glu_dwconv_fwd(N._ptr(g), N._ptr(pad8), N._ptr(w2), N._ptr(dw_bias), N._ptr(y), N._ptr(stats),
                                           ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(K),
                                           ctypes.c_int(left_pad), N._stream()), "sb_glu_dwconv_fwd")
        count = float(B * T)
        count_t = None
        if training and stats_reduce is not None:
            # the global element count travels with the sums, and the kernels read it from device memory (no host sync)
            stats[2 * C] = count
            stats = stats_reduce(stats)
            count_t = stats[2 * C:]
        mean_rstd = torch.empty(2 * C, dtype=torch.float32, device=dev)
        N._check(N.lib().sb_bn_finalize(N._ptr(stats), ctypes.c_float(count), N._ptr(count_t), N._ptr(mean_rstd), N._ptr(running_mean),
                                        N._ptr(running_var), ctypes.c_int(C), ctypes.c_float(eps), ctypes.c_float(momentum),
                                        ctypes.c_int(1 if training else 0), N._stream()), "sb_bn_finalize")
        s = torch.empty((B, T, C), dtype=torch.bfloat16, device=dev)
        N._check(N.lib().sb_bn_silu_fwd(N._ptr(y), N._ptr(mean_rstd), N._ptr(gamma), N._ptr(beta), N._ptr(s),
                                        ctypes.c_longlong(B * T), ctypes.c_int(C), N._stream()), "sb_bn_silu_fwd")
        ctx.save_for_backward(g, y, mean_rstd, pad8, w2)
        ctx.params = (dw_weight, dw_bias, gamma, beta)
        ctx.cfg = (B, T, C, K, left_pad, training, count, stats_reduce)
        ctx.count_t = count_t
        return s

    @staticmethod
    def backward(ctx, ds):
        g, y, mean_rstd, pad8, w2 = ctx.saved_tensors
        dw_weight, dw_bias, gamma, beta = ctx.params
        B, T, C, K, left, training, count, stats_reduce = ctx.cfg
        dev = ds.device
        ds = ds.contiguous()
        sums = torch.zeros(2 * C, dtype=torch.float32, device=dev)
        N._check(N.lib().sb_bn_silu_bwd_stats(N._ptr(ds), N._ptr(y), N._ptr(mean_rstd), N._ptr(gamma), N._ptr(beta), N._ptr(sums),
                                              ctypes.c_longlong(B * T), ctypes.c_int(C), N._stream()), "sb_bn_silu_bwd_stats")
        local_sums = sums
        if training and stats_reduce is not None:
            sums = stats_reduce(sums.clone())
        dg = torch.empty((B, T, 2 * C), dtype=torch.bfloat16, device=dev)
        gw = getattr(dw_weight, "_grad_view", None)
        gb = getattr(dw_bias, "_grad_view", None) if dw_bias is not None else None
        direct = gw is not None and gw.is_cuda and (dw_bias is None or gb is not None)
        dwt = gw.view(C, K) if direct else torch.zeros((C, K), dtype=torch.float32, device=dev)
        dbt = (gb if direct else torch.zeros(C, dtype=torch.float32, device=dev)) if dw_bias is not None else None
        N._check(N.lib().sb_dwconv_glu_bwd(N._ptr(ds), N._ptr(y), N._ptr(g), N._ptr(pad8), N._ptr(w2), N._ptr(mean_rstd),
                                           N._ptr(gamma), N._ptr(beta), N._ptr(sums), ctypes.c_float(count), N._ptr(ctx.count_t),
                                           ctypes.c_int(1 if training else 0), N._ptr(dg), N._ptr(dwt), N._ptr(dbt),
                                           ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(K), ctypes.c_int(left),
                                           N._stream()), "sb_dwconv_glu_bwd")
        # BatchNorm affine gradients are the (local) sums computed above
        dgamma = N._write_param_grad(gamma, lambda out, b_: out.add_(local_sums[C:]) if b_ else out.copy_(local_sums[C:]), (C,))
        dbeta = N._write_param_grad(beta, lambda out, b_: out.add_(local_sums[:C]) if b_ else out.copy_(local_sums[:C]), (C,))
        if direct:
            arena = getattr(dw_weight, "_arena", None)
            cb = getattr(arena, "grad_ready", None) if arena is not None else None
            if cb is not None:
                cb(dw_weight)
                if dw_bias is not None:
                    cb(dw_bias)
            return dg, None, None, dgamma, dbeta, None, None, None, None, None, None, None, None
        return dg, dwt.view(dw_weight.shape), dbt, dgamma, dbeta, None, None, None, None, None, None, None, None


def conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean, running_var, pad_mask, training,
                     momentum, eps, left_pad, right_pad, bn_stats_reduce):
    C = g.shape[-1] // 2
    K = dw_weight.shape[-1]
    if norm_type != "batch_norm" or K not in (5, 9, 15) or C % 8 != 0 or left_pad + right_pad != K - 1:
        from . import reference

        return reference.conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean, running_var,
                                          pad_mask, training, momentum, eps, left_pad, right_pad, None, 0, bn_stats_reduce)
    return _ConvCoreFn.apply(g, dw_weight, dw_bias, norm_weight, norm_bias, running_mean, running_var, pad_mask, bool(training),
                             float(momentum if momentum is not None else 0.1), float(eps), int(left_pad), bn_stats_reduce)

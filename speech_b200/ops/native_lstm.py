"""Multi-layer LSTM (transducer prediction network) on the sm_100a kernels: GEMMs for everything batched over time,
the step kernels of csrc/lstm.cu for the recurrence.  Weights follow ``torch.nn.LSTM`` (gate order i, f, g, o)."""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import native as N


def _i(x):
    return ctypes.c_int(int(x))


class _LSTMFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, h0, c0, num_layers, *weights):
        U, B, _ = x.shape
        dev = x.device
        H = weights[1].shape[1]
        saved = []
        inp = x.contiguous()
        hn, cn = [], []
        for l in range(num_layers):
            w_ih, w_hh, b_ih, b_hh = weights[4 * l: 4 * l + 4]
            wih = N._lowp_weight(w_ih)
            whh = N._lowp_weight(w_hh)
            In = wih.shape[1]
            bias = (b_ih.detach() + b_hh.detach()).float()
            xproj = torch.empty((U * B, 4 * H), dtype=torch.float32, device=dev)
            N.gemm(inp.view(U * B, In), wih, xproj, M=U * B, N=4 * H, K=In, bias=bias)
            acts = torch.empty((U, B, 4 * H), dtype=torch.float32, device=dev)
            c_all = torch.empty((U, B, H), dtype=torch.float32, device=dev)
            y = torch.empty((U, B, H), dtype=torch.bfloat16, device=dev)
            h0l = h0[l].to(torch.bfloat16).contiguous() if h0 is not None else None
            c0l = c0[l].float().contiguous() if c0 is not None else None
            N._check(N.lib().sb_lstm_forward(N._ptr(xproj), N._ptr(h0l), N._ptr(c0l), N._ptr(whh), N._ptr(acts), N._ptr(c_all),
                                             N._ptr(y), _i(U), _i(B), _i(H), N._stream()), "sb_lstm_forward")
            saved.append((inp, acts, c_all, y, h0l, c0l))
            hn.append(y[-1])
            cn.append(c_all[-1])
            inp = y
        ctx.layers = saved
        ctx.weights = weights
        ctx.dims = (U, B, H, num_layers)
        ctx.has_state = h0 is not None
        h_n = torch.stack(hn).to(x.dtype)
        c_n = torch.stack(cn).to(x.dtype)
        ctx.mark_non_differentiable(h_n, c_n)
        return inp, h_n, c_n

    @staticmethod
    def backward(ctx, dy, _dhn, _dcn):
        U, B, H, L = ctx.dims
        dev = dy.device
        weights = ctx.weights
        grads: List[Optional[torch.Tensor]] = [None] * len(weights)
        dcur = dy.contiguous().to(torch.bfloat16)
        for l in reversed(range(L)):
            inp, acts, c_all, y, h0l, c0l = ctx.layers[l]
            w_ih, w_hh, b_ih, b_hh = weights[4 * l: 4 * l + 4]
            wih, whh = N._lowp_weight(w_ih), N._lowp_weight(w_hh)
            In = wih.shape[1]
            dh_rec = torch.zeros((B, H), dtype=torch.float32, device=dev)
            dc_rec = torch.zeros((B, H), dtype=torch.float32, device=dev)
            dGb = torch.empty((U, B, 4 * H), dtype=torch.bfloat16, device=dev)
            N._check(N.lib().sb_lstm_backward(N._ptr(dcur), N._ptr(dh_rec), N._ptr(dc_rec), N._ptr(acts), N._ptr(c_all), N._ptr(c0l),
                                              N._ptr(whh), N._ptr(dGb), _i(U), _i(B), _i(H), N._stream()),
                     "sb_lstm_backward")
            dG2 = dGb.view(U * B, 4 * H)
            first = h0l.unsqueeze(0) if h0l is not None else torch.zeros((1, B, H), dtype=torch.bfloat16, device=dev)
            hprev = torch.cat([first, y[:-1]], dim=0).view(U * B, H)
            x2 = inp.view(U * B, In)
            grads[4 * l + 1] = N._write_param_grad(w_hh, lambda out, beta: N.gemm(dG2, hprev, out, M=4 * H, N=H, K=U * B, a_mn=True,
                                                                                lda=4 * H, b_mn=True, ldb=H, beta=beta), (4 * H, H))
            grads[4 * l] = N._write_param_grad(w_ih, lambda out, beta: N.gemm(dG2, x2, out, M=4 * H, N=In, K=U * B, a_mn=True,
                                                                            lda=4 * H, b_mn=True, ldb=In, beta=beta), (4 * H, In))
            grads[4 * l + 2] = N._write_param_grad(b_ih, lambda out, beta: N.colsum(dG2, out, accumulate=beta != 0.0), (4 * H,))
            grads[4 * l + 3] = N._write_param_grad(b_hh, lambda out, beta: N.colsum(dG2, out, accumulate=beta != 0.0), (4 * H,))
            if l > 0 or ctx.needs_input_grad[0]:
                dx = torch.empty((U * B, In), dtype=torch.bfloat16, device=dev)
                N.gemm(dG2, wih, dx, M=U * B, N=In, K=4 * H, b_mn=True, ldb=In)
                dcur = dx.view(U, B, In)
        dx0 = dcur if ctx.needs_input_grad[0] else None
        return (dx0, None, None, None, *grads)


def lstm(x, weights, h0=None, c0=None, num_layers: int = 1):
    """x: [U, B, In] bf16; weights: (w_ih, w_hh, b_ih, b_hh) per layer.  Returns (out [U,B,H], (h_n, c_n))."""
    H = weights[1].shape[1]
    In = weights[0].shape[1]
    if H % 8 != 0 or In % 8 != 0 or weights[1].shape[0] != 4 * H:
        from . import reference

        return reference.lstm(x, weights, h0, c0, num_layers)
    out, h_n, c_n = _LSTMFn.apply(x, h0, c0, num_layers, *weights)
    return out, (h_n, c_n)

"""Plain-PyTorch statements of every hot op.

These run on the CPU (tests, plumbing configs) and serve as the numerical oracle for the
sm_100a kernels: each CUDA kernel's test compares against the function of the same name here,
evaluated in fp32.  Nothing in this file is performance-critical.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

NEG_INF = -1e30


def act_fn(name: Optional[str]):
    if name is None or name in ("none", "identity"):
        return lambda x: x
    return {"relu": F.relu, "swish": F.silu, "silu": F.silu, "gelu": F.gelu, "tanh": torch.tanh,
            "sigmoid": torch.sigmoid}[name]


def linear(x, weight, bias=None, act=None, residual=None, alpha: float = 1.0, dropout_p: float = 0.0):
    """``residual + alpha * dropout(act(x @ W^T + b))``."""
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    y = act_fn(act)(y)
    if dropout_p > 0.0:
        y = F.dropout(y, dropout_p, training=True)
    if alpha != 1.0:
        y = y * alpha
    if residual is not None:
        y = residual + y
    return y


def layer_norm(x, weight, bias, eps: float = 1e-5):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def rel_shift(x: torch.Tensor) -> torch.Tensor:
    """Transformer-XL skew: ``out[..., i, j] = x[..., i, j + (Tq - 1 - i)]`` for the first ``Tq`` columns kept by the
    caller; implemented by the pad-reshape trick (reference: ``multi_head_attention.py:266-277``)."""
    b, h, qlen, pos_len = x.size()
    x = F.pad(x, pad=(1, 0))
    x = x.view(b, h, -1, qlen)
    x = x[:, :, 1:].view(b, h, qlen, pos_len)
    return x


def relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask=None, dropout_p: float = 0.0, training: bool = False):
    """Transformer-XL relative-position attention.

    q: [B,Tq,H,dk]; k, v: [B,Tk,H,dk]; p: [Bp,P,H,dk] with P = 2*Tk-1 position vectors for relative
    offsets Tk-1 ... -(Tk-1); pos_bias_{u,v}: [H,dk]; mask: bool [B,Tq,Tk], True = not visible.
    Returns [B,Tq,H*dk].  Masked scores are filled with -10000 and masked probabilities re-zeroed
    (reference: ``multi_head_attention.py:127-148,279-361``).
    """
    B, Tq, H, dk = q.shape
    Tk = k.shape[1]
    qf, kf, vf, pf = q.float(), k.float(), v.float(), p.float()
    q_u = (qf + pos_bias_u.float()).transpose(1, 2)  # B,H,Tq,dk
    q_v = (qf + pos_bias_v.float()).transpose(1, 2)
    kk = kf.transpose(1, 2)
    vv = vf.transpose(1, 2)
    pp = pf.transpose(1, 2)  # Bp,H,P,dk
    matrix_ac = torch.matmul(q_u, kk.transpose(-2, -1))
    matrix_bd = torch.matmul(q_v, pp.transpose(-2, -1))
    matrix_bd = rel_shift(matrix_bd)[:, :, :, :Tk]
    scores = (matrix_ac + matrix_bd) / math.sqrt(dk)
    if mask is not None:
        m = mask.unsqueeze(1)
        scores = scores.masked_fill(m, -10000.0)
        attn = torch.softmax(scores, dim=-1).masked_fill(m, 0.0)
    else:
        attn = torch.softmax(scores, dim=-1)
    if dropout_p > 0 and training:
        attn = F.dropout(attn, dropout_p, True)
    out = torch.matmul(attn, vv)  # B,H,Tq,dk
    return out.transpose(1, 2).reshape(B, Tq, H * dk).to(q.dtype)


def mha_attention(q, k, v, mask=None, dropout_p: float = 0.0, training: bool = False, scale: Optional[float] = None):
    """Plain scaled-dot-product attention on [B,T,H,dk] tensors; mask bool [B,Tq,Tk] or [B,1,Tq,Tk], True = hidden."""
    B, Tq, H, dk = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(dk)
    s = torch.matmul(q.float().transpose(1, 2), k.float().transpose(1, 2).transpose(-2, -1)) * scale
    if mask is not None:
        m = mask if mask.dim() == 4 else mask.unsqueeze(1)
        s = s.masked_fill(m, -10000.0)
        a = torch.softmax(s, dim=-1).masked_fill(m, 0.0)
    else:
        a = torch.softmax(s, dim=-1)
    if dropout_p > 0 and training:
        a = F.dropout(a, dropout_p, True)
    o = torch.matmul(a, v.float().transpose(1, 2))
    return o.transpose(1, 2).reshape(B, Tq, H * dk).to(q.dtype)


def conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean, running_var,
                     pad_mask=None, training: bool = False, momentum: float = 0.1, eps: float = 1e-5,
                     left_pad: int = 4, right_pad: int = 4, cache=None, cache_drop_size: int = 0,
                     bn_stats_reduce=None):
    """GLU -> pad-mask -> depthwise conv (k taps) -> BatchNorm / LayerNorm -> SiLU, channels-last.

    g: [B,T,2C] output of the first pointwise conv; dw_weight: [C,1,K]; pad_mask: bool [B,T], True = padding;
    cache: [B,C,K-1] left context for streaming (returns the next cache as second output).
    Reference: ``conformer_modules.py:338-368`` and ``causal_convs.py:131-151``.
    """
    B, T, C2 = g.shape
    C = C2 // 2
    x = F.glu(g.float(), dim=-1)
    if pad_mask is not None:
        x = x.masked_fill(pad_mask.unsqueeze(-1), 0.0)
    xt = x.transpose(1, 2)  # B,C,T
    next_cache = None
    if cache is None:
        xt = F.pad(xt, (left_pad, right_pad))
    else:
        xt = torch.cat([cache.float(), F.pad(xt, (0, right_pad))], dim=-1)
        next_cache = xt[:, :, : xt.shape[-1] - cache_drop_size] if cache_drop_size > 0 else xt
        next_cache = next_cache[:, :, -cache.shape[-1]:].to(cache.dtype)
    y = F.conv1d(xt, dw_weight.float(), None if dw_bias is None else dw_bias.float(), groups=C)
    if norm_type == "batch_norm":
        if training:
            if bn_stats_reduce is not None:
                n = torch.tensor([float(y.shape[0] * y.shape[2])], device=y.device)
                s = torch.cat([y.sum(dim=(0, 2)), (y * y).sum(dim=(0, 2)), n])
                s = bn_stats_reduce(s)
                n_tot = s[-1]
                mean = s[:C] / n_tot
                var = s[C:2 * C] / n_tot - mean * mean
            else:
                n_tot = float(y.shape[0] * y.shape[2])
                mean = y.mean(dim=(0, 2))
                var = y.var(dim=(0, 2), unbiased=False)
            if running_mean is not None:
                with torch.no_grad():
                    unb = var * (n_tot / max(float(n_tot) - 1.0, 1.0))
                    running_mean.mul_(1 - momentum).add_(mean.detach().to(running_mean.dtype), alpha=momentum)
                    running_var.mul_(1 - momentum).add_(unb.detach().to(running_var.dtype), alpha=momentum)
            y = (y - mean[None, :, None]) * torch.rsqrt(var[None, :, None] + eps)
        else:
            y = (y - running_mean.float()[None, :, None]) * torch.rsqrt(running_var.float()[None, :, None] + eps)
        y = y * norm_weight.float()[None, :, None] + norm_bias.float()[None, :, None]
        y = y.transpose(1, 2)
    elif norm_type == "layer_norm":
        y = F.layer_norm(y.transpose(1, 2), (C,), norm_weight.float(), norm_bias.float(), eps)
    else:
        raise ValueError(f"unsupported conv_norm_type {norm_type}")
    out = F.silu(y).to(g.dtype)
    return (out, next_cache) if cache is not None else out


# ----------------------------------------------------------------------------- transducer losses
def _lse2(a, b):
    return torch.logaddexp(a, b)


def transducer_loglik_arcs(blank_arc, label_arc, f_len, y_len):
    """Log-likelihood of a transducer lattice given its arcs.

    ``blank_arc[d]`` / ``label_arc[d]``: [B,T,U1] log-weight of leaving node (t,u) by a blank that advances
    ``d > 0`` frames, or by the next label advancing ``d >= 0`` frames.  Termination is by a blank arc from
    (T-d, U).  Vectorised over batch and u: for each t the duration-0 label chain along u is a first-order
    log-space recurrence solved with ``logcumsumexp``.
    """
    any_arc = next(iter(blank_arc.values()))
    B, T, U1 = any_arc.shape
    dev, dt = any_arc.device, any_arc.dtype
    u_idx = torch.arange(U1, device=dev)
    valid_u = u_idx[None, :] <= y_len[:, None]  # [B,U1]
    alphas: List[torch.Tensor] = []
    neg = torch.full((B, U1), NEG_INF, device=dev, dtype=dt)
    for t in range(T):
        c = neg.clone()
        if t == 0:
            c[:, 0] = 0.0
        for d, arc in blank_arc.items():
            if t - d >= 0:
                c = _lse2(c, alphas[t - d] + arc[:, t - d, :])
        for d, arc in label_arc.items():
            if d > 0 and t - d >= 0:
                contrib = alphas[t - d][:, :-1] + arc[:, t - d, :-1]
                c = torch.cat([c[:, :1], _lse2(c[:, 1:], contrib)], dim=1)
        if 0 in label_arc:
            e0 = label_arc[0][:, t, :-1]  # arc (t,u)->(t,u+1)
            E = torch.cat([torch.zeros(B, 1, device=dev, dtype=dt), torch.cumsum(e0, dim=1)], dim=1)
            a = E + torch.logcumsumexp(c - E, dim=1)
        else:
            a = c
        a = torch.where(valid_u, a, neg)
        alphas.append(a)
    alpha = torch.stack(alphas, dim=1)  # [B,T,U1]
    ll = torch.full((B,), NEG_INF, device=dev, dtype=dt)
    bidx = torch.arange(B, device=dev)
    for d, arc in blank_arc.items():
        tt = f_len - d
        ok = tt >= 0
        tt_c = tt.clamp(min=0)
        val = alpha[bidx, tt_c, y_len] + arc[bidx, tt_c, y_len]
        ll = torch.where(ok, _lse2(ll, val), ll)
    return ll, alpha


def transducer_loglik(blank_lp, label_lp, dur_lp, durations: Sequence[int], f_len, y_len):
    """RNNT (``dur_lp is None``: blank advances one frame, labels none) or TDT lattice log-likelihood from
    gathered log-probabilities blank_lp/label_lp [B,T,U1] and dur_lp [B,T,U1,D].  TDT recursion of
    ``losses/rnnt_pytorch.py:178-247``: blank transitions only with duration > 0, label transitions with any
    duration."""
    if dur_lp is None:
        return transducer_loglik_arcs({1: blank_lp}, {0: label_lp}, f_len, y_len)
    blank_arc = {d: blank_lp + dur_lp[..., i] for i, d in enumerate(durations) if d > 0}
    label_arc = {d: label_lp + dur_lp[..., i] for i, d in enumerate(durations)}
    return transducer_loglik_arcs(blank_arc, label_arc, f_len, y_len)


def multiblank_loss_from_logits(logits, targets, f_len, y_len, blank: int, big_blank_durations: Sequence[int],
                                sigma: float = 0.0):
    """Multi-blank RNNT: ``len(big_blank_durations)`` extra blank symbols stored right before the standard
    blank, the i-th one advancing ``big_blank_durations[i]`` frames (reference kernels
    ``gpu_rnnt_kernel.py:411-885``)."""
    B, T, U1, _ = logits.shape
    tok = torch.log_softmax(logits.float(), dim=-1) - sigma
    nb = len(big_blank_durations)
    tgt = torch.cat([targets, targets.new_zeros(B, 1)], dim=1).clamp(min=0)
    label_lp = torch.gather(tok, 3, tgt[:, None, :, None].expand(B, T, U1, 1).long()).squeeze(-1)
    blank_arc = {1: tok[..., blank]}
    for i, d in enumerate(big_blank_durations):
        lp = tok[..., blank - nb + i]
        blank_arc[d] = torch.logaddexp(blank_arc[d], lp) if d in blank_arc else lp
    ll, _ = transducer_loglik_arcs(blank_arc, {0: label_lp}, f_len, y_len)
    return -ll


def gather_transducer_logprobs(logits, targets, blank: int, num_durations: int = 0, sigma: float = 0.0):
    """From joint logits [B,T,U1,V+1+D] produce (blank_lp, label_lp, dur_lp) with the sigma under-normalisation
    applied to the token log-softmax (reference: ``losses/rnnt_pytorch.py:153-159``)."""
    B, T, U1, _ = logits.shape
    if num_durations > 0:
        tok = torch.log_softmax(logits[..., :-num_durations].float(), dim=-1) - sigma
        dur = torch.log_softmax(logits[..., -num_durations:].float(), dim=-1)
    else:
        tok = torch.log_softmax(logits.float(), dim=-1) - sigma
        dur = None
    blank_lp = tok[..., blank]
    tgt = torch.cat([targets, targets.new_zeros(B, 1)], dim=1).clamp(min=0)  # pad column for u = U
    label_lp = torch.gather(tok, 3, tgt[:, None, :, None].expand(B, T, U1, 1).long()).squeeze(-1)
    return blank_lp, label_lp, dur


def tdt_loss_from_logits(logits, targets, f_len, y_len, blank: int, durations: Sequence[int], sigma: float = 0.0):
    nd = len(durations) if durations else 0
    b, l, d = gather_transducer_logprobs(logits, targets, blank, nd, sigma)
    ll, _ = transducer_loglik(b, l, d, list(durations) if durations else [], f_len, y_len)
    return -ll


def joint_logits(f, g, w, b, act: str = "relu"):
    """f: [B,T,H] projected encoder, g: [B,U1,H] projected prediction net -> [B,T,U1,V]."""
    h = act_fn(act)(f.unsqueeze(2) + g.unsqueeze(1))
    return F.linear(h, w.to(h.dtype), None if b is None else b.to(h.dtype))


def transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank: int, durations: Sequence[int], sigma: float,
                          act: str = "relu", fastemit_lambda: float = 0.0, sub_batch: int = 0, dropout_p: float = 0.0):
    """Joint network + RNNT/TDT negative log-likelihood per utterance, computed sub-batch by sub-batch with the
    T and U axes trimmed to the sub-batch maximum (reference fused mode: ``modules/rnnt.py:1495-1641``)."""
    B = f.shape[0]
    sub_batch = sub_batch or B
    out = []
    for s in range(0, B, sub_batch):
        e = min(B, s + sub_batch)
        tl = int(f_len[s:e].max())
        ul = int(y_len[s:e].max())
        if dropout_p > 0.0:
            hid = F.dropout(act_fn(act)(f[s:e, :tl].float().unsqueeze(2) + g[s:e, : ul + 1].float().unsqueeze(1)), dropout_p, True)
            logits = F.linear(hid, w.float(), None if b is None else b.float())
        else:
            logits = joint_logits(f[s:e, :tl].float(), g[s:e, : ul + 1].float(), w.float(), None if b is None else b.float(), act)
        out.append(tdt_loss_from_logits(logits, targets[s:e, :ul], f_len[s:e], y_len[s:e], blank, durations, sigma))
    loss = torch.cat(out)
    return loss * (1.0 + fastemit_lambda) if fastemit_lambda else loss


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank: int, zero_infinity: bool = True):
    """log_probs: [B,T,V+1] (already log-softmaxed); returns per-utterance negative log-likelihood."""
    return F.ctc_loss(log_probs.float().transpose(0, 1), targets, input_lengths, target_lengths, blank=blank,
                      reduction="none", zero_infinity=zero_infinity)


# ----------------------------------------------------------------------------- front-end
def logmel(x, seq_len, window, fb, n_fft: int, hop: int, win_length: int, preemph: float = 0.97, mag_power: float = 2.0,
           log_zero_guard: float = 2 ** -24, normalize: Optional[str] = "per_feature", pad_to: int = 0,
           pad_value: float = 0.0, dither: float = 0.0, exact_pad: bool = False, log: bool = True):
    """Waveform [B,L] -> log-mel [B,nfilt,T] following ``features.py:415-494`` step by step (fp32)."""
    x = x.float()
    out_len = torch.floor_divide(seq_len + 2 * (n_fft // 2) - n_fft, hop).to(torch.long)
    if dither > 0:
        x = x + dither * torch.randn_like(x)
    if preemph:
        tmask = torch.arange(x.shape[1], device=x.device).unsqueeze(0) < seq_len.unsqueeze(1)
        x = torch.cat((x[:, :1], x[:, 1:] - preemph * x[:, :-1]), dim=1)
        x = x.masked_fill(~tmask, 0.0)
    spec = torch.stft(x, n_fft=n_fft, hop_length=hop, win_length=win_length, center=True, window=window.float(),
                      return_complex=True, pad_mode="constant")
    mag = torch.sqrt(spec.real.pow(2) + spec.imag.pow(2))
    if mag_power != 1.0:
        mag = mag.pow(mag_power)
    mel = torch.matmul(fb.float(), mag)
    if log:
        mel = torch.log(mel + log_zero_guard)
    T = mel.shape[-1]
    if normalize == "per_feature":
        tidx = torch.arange(T, device=x.device)[None, :]
        valid = tidx < out_len[:, None]
        n = out_len.clamp(min=1).float()[:, None]
        mean = (mel * valid[:, None, :]).sum(-1) / n
        var = (((mel - mean[..., None]) ** 2) * valid[:, None, :]).sum(-1) / (n - 1.0).clamp(min=1.0)
        std = torch.sqrt(var)
        std = torch.where(out_len[:, None] == 1, torch.zeros_like(std), std) + 1e-5
        mel = (mel - mean[..., None]) / std[..., None]
    elif normalize == "all_features":
        tidx = torch.arange(T, device=x.device)[None, :]
        valid = (tidx < out_len[:, None])[:, None, :].expand_as(mel)
        for i in range(mel.shape[0]):
            seg = mel[i][valid[i]]
            mel[i] = (mel[i] - seg.mean()) / (seg.std() + 1e-5)
    mask = torch.arange(T, device=x.device)[None, :] >= out_len[:, None]
    mel = mel.masked_fill(mask[:, None, :], pad_value)
    if pad_to and pad_to > 0:
        rem = T % pad_to
        if rem:
            mel = F.pad(mel, (0, pad_to - rem), value=pad_value)
    return mel, out_len


# ----------------------------------------------------------------------------- optimizer
def adamw_flat(master, grad, exp_avg, exp_avg_sq, lowp, lr, beta1, beta2, eps, weight_decay, step, clip_coef=1.0):
    """Decoupled-weight-decay Adam on flat buffers (same update as ``torch.optim.AdamW``)."""
    g = grad * clip_coef
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    master.mul_(1 - lr * weight_decay)
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if lowp is not None:
        lowp.copy_(master)


def lstm(x, weights: List[torch.Tensor], h0=None, c0=None, num_layers: int = 1, dropout: float = 0.0, training=False,
         proj_size: int = 0):
    """Time-major multi-layer LSTM, x: [U,B,In]; weights: flat list (w_ih, w_hh, b_ih, b_hh) per layer."""
    U, B, _ = x.shape
    H = weights[1].shape[1]
    if h0 is None:
        h0 = x.new_zeros(num_layers, B, H)
        c0 = x.new_zeros(num_layers, B, H)
    out, h, c = torch._VF.lstm(x, (h0, c0), [w.to(x.dtype) for w in weights], True, num_layers, dropout, training, False, False)
    return out, (h, c)


def specaugment(x, f_start, f_width, t_start, t_width, mask_value: float = 0.0):
    B, F, T = x.shape
    fill = torch.zeros(B, F, T, dtype=torch.bool, device=x.device)
    if f_start is not None and f_start.shape[1] > 0:
        f = torch.arange(F, device=x.device)[None, None, :]
        fill |= ((f >= f_start[..., None]) & (f < (f_start + f_width)[..., None])).any(dim=1)[:, :, None]
    if t_start is not None and t_start.shape[1] > 0:
        t = torch.arange(T, device=x.device)[None, None, :]
        fill |= ((t >= t_start[..., None]) & (t < (t_start + t_width)[..., None])).any(dim=1)[:, None, :]
    return x.masked_fill(fill, mask_value)


def ngram_advance(states, arc_keys, arc_w, arc_to, backoff_w, backoff_to, V: int, depth: int, default_score: float, start_state: int):
    """Up to ``depth`` rounds of a vectorised binary search over the sorted arc keys, adding back-off weights for the
    (state, token) pairs not yet resolved."""
    B = states.shape[0]
    tok = torch.arange(V, dtype=torch.long, device=states.device)
    cur = states.view(B, 1).expand(B, V)
    acc = torch.zeros((B, V), dtype=torch.float32, device=states.device)
    done = torch.zeros((B, V), dtype=torch.bool, device=states.device)
    scores = torch.zeros_like(acc)
    nxt = torch.full((B, V), start_state, dtype=torch.long, device=states.device)
    last = arc_keys.shape[0] - 1
    for _ in range(depth):
        key = cur * V + tok
        idx = torch.searchsorted(arc_keys, key).clamp(max=last)
        hit = (arc_keys[idx] == key) & ~done
        scores = torch.where(hit, acc + arc_w[idx], scores)
        nxt = torch.where(hit, arc_to[idx], nxt)
        done = done | hit
        acc = acc + backoff_w[cur]
        cur = backoff_to[cur]
    scores = torch.where(done, scores, acc + default_score)
    return scores, nxt

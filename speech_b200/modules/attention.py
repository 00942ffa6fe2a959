"""Positional encodings and multi-head attention layers of the Conformer encoder.

* ``RelPositionalEncoding`` — sinusoid table for relative offsets L-1 ... -(L-1), ``xscale`` and
  centre-window slicing (reference: ``multi_head_attention.py:1046-1150``).
* ``RelPositionMultiHeadAttention`` — Transformer-XL attention with learned ``pos_bias_u/v`` and a
  streaming key/value cache (reference: ``multi_head_attention.py:219-361,207-212``).
* ``MultiHeadAttention`` — absolute-position variant.
* ``RelPositionMultiHeadAttentionLongformer`` — sliding-window local attention with optional global
  tokens (reference: ``:364-997``); implemented as banded attention through a band mask.

Parameter names (``linear_q/k/v/out/pos``, ``pos_bias_u/v``) match the reference so state dicts load.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .. import ops

INF_VAL = 10000.0


class PositionalEncoding(nn.Module):
    def __init__(self, d_model, dropout_rate, max_len=5000, xscale=None, dropout_rate_emb=0.0):
        super().__init__()
        self.d_model, self.xscale, self.max_len = d_model, xscale, max_len
        self.dropout = nn.Dropout(p=dropout_rate)
        self.dropout_emb = nn.Dropout(dropout_rate_emb) if dropout_rate_emb > 0 else None

    def create_pe(self, positions, dtype):
        pos_length = positions.size(0)
        pe = torch.zeros(pos_length, self.d_model, device=positions.device)
        div_term = torch.exp(torch.arange(0, self.d_model, 2, dtype=torch.float32, device=positions.device)
                             * -(math.log(INF_VAL) / self.d_model))
        pe[:, 0::2] = torch.sin(positions * div_term)
        pe[:, 1::2] = torch.cos(positions * div_term)
        pe = pe.unsqueeze(0).to(dtype)
        if hasattr(self, "pe"):
            self.pe = pe
        else:
            self.register_buffer("pe", pe, persistent=False)

    def extend_pe(self, length, device, dtype=torch.float32):
        if hasattr(self, "pe") and self.pe.size(1) >= length and self.pe.device == torch.device(device):
            return
        positions = torch.arange(0, length, dtype=torch.float32, device=device).unsqueeze(1)
        self.create_pe(positions=positions, dtype=dtype)

    def forward(self, x, cache_len=0):
        input_len = x.size(1) + cache_len
        if self.xscale:
            x = x * self.xscale
        pos_emb = self.pe[:, :input_len]
        if self.dropout_emb:
            pos_emb = self.dropout_emb(pos_emb)
        x = x + pos_emb.to(x.dtype)
        return self.dropout(x), pos_emb


class RelPositionalEncoding(PositionalEncoding):
    def extend_pe(self, length, device, dtype=torch.float32):
        needed = 2 * length - 1
        if hasattr(self, "pe") and self.pe.size(1) >= needed and self.pe.device == torch.device(device):
            return
        positions = torch.arange(length - 1, -length, -1, dtype=torch.float32, device=device).unsqueeze(1)
        self.create_pe(positions=positions, dtype=dtype)

    def forward(self, x, cache_len=0):
        if self.xscale:
            x = x * self.xscale
        input_len = x.size(1) + cache_len
        center_pos = self.pe.size(1) // 2 + 1
        start_pos = center_pos - input_len
        end_pos = center_pos + input_len - 1
        pos_emb = self.pe[:, start_pos:end_pos]
        if self.dropout_emb:
            pos_emb = self.dropout_emb(pos_emb)
        return self.dropout(x), pos_emb


class LocalAttRelPositionalEncoding(PositionalEncoding):
    """Relative encodings for a fixed window [-left, right] (reference ``:1152-1200``)."""

    def __init__(self, att_context_size, **kwargs):
        super().__init__(**kwargs)
        self.left_context, self.right_context = att_context_size

    def extend_pe(self, length, device, dtype=torch.float32):
        if hasattr(self, "pe") and self.pe.device == torch.device(device):
            return
        positions = torch.arange(self.left_context, -self.right_context - 1, -1, dtype=torch.float32,
                                 device=device).unsqueeze(1)
        self.create_pe(positions=positions, dtype=dtype)

    def forward(self, x, cache_len=0):
        if self.xscale:
            x = x * self.xscale
        end_pos = self.left_context + self.right_context + 1
        pos_emb = self.pe[:, :end_pos]
        if self.dropout_emb:
            pos_emb = self.dropout_emb(pos_emb)
        return self.dropout(x), pos_emb


class MultiHeadAttention(nn.Module):
    def __init__(self, n_head, n_feat, dropout_rate, max_cache_len=0, use_bias=True, use_pytorch_sdpa=False,
                 use_pytorch_sdpa_backends=None):
        super().__init__()
        assert n_feat % n_head == 0
        self.d_k, self.h = n_feat // n_head, n_head
        self.s_d_k = math.sqrt(self.d_k)
        self.linear_q = nn.Linear(n_feat, n_feat, bias=use_bias)
        self.linear_k = nn.Linear(n_feat, n_feat, bias=use_bias)
        self.linear_v = nn.Linear(n_feat, n_feat, bias=use_bias)
        self.linear_out = nn.Linear(n_feat, n_feat, bias=use_bias)
        self.dropout_rate = dropout_rate
        self._max_cache_len = max_cache_len
        self.cache_drop_size = 0

    def _qkv(self, query, key, value):
        B = query.shape[0]
        fused = None
        if query is key and key is value and query.is_cuda and query.dtype == torch.bfloat16 and not ops.eager_allowed():
            fused = fused_qkv_weight(self)
        if fused is not None:
            w, b = fused
            qkv = ops.linear(query, w, b).view(B, -1, 3, self.h, self.d_k)
            self._last_qkv = qkv
            return qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        self._last_qkv = None
        q = ops.linear(query, self.linear_q.weight, self.linear_q.bias).view(B, -1, self.h, self.d_k)
        k = ops.linear(key, self.linear_k.weight, self.linear_k.bias).view(B, -1, self.h, self.d_k)
        v = ops.linear(value, self.linear_v.weight, self.linear_v.bias).view(B, -1, self.h, self.d_k)
        return q, k, v

    def update_cache(self, key, value, query, cache):
        if cache is not None:
            n_cache = cache.shape[1]
            q_keep_size = query.shape[1] - self.cache_drop_size
            self_attention = key is query
            key = value = torch.cat([cache.to(key.dtype), key], dim=1)
            if self_attention and q_keep_size > 0 and key.dtype == cache.dtype:
                # the new cache is the window of `cache ++ query` that ends after the kept query frames: a view, not a copy
                # (the caller stacks the per-layer caches into one tensor, which is the only copy that is needed)
                cache = key[:, q_keep_size:q_keep_size + n_cache, :]
            else:
                cache = torch.cat([cache[:, q_keep_size:, :], query[:, :q_keep_size, :].to(cache.dtype)], dim=1)
        return key, value, query, cache

    def forward(self, query, key, value, mask=None, pos_emb=None, cache=None, residual=None, out_dropout: float = 0.0):
        same = query is key and key is value
        key, value, query, cache = self.update_cache(key, value, query, cache)
        if same and cache is None:
            key = value = query
        q, k, v = self._qkv(query, key, value)
        ctx = ops.mha_attention(q, k, v, mask, self.dropout_rate, self.training)
        out = ops.linear(ctx, self.linear_out.weight, self.linear_out.bias, residual=residual, dropout_p=out_dropout)
        return out if cache is None else (out, cache)


def fused_qkv_weight(mod):
    """If the optimizer arena laid q/k/v weights (and biases) out back to back, return zero-copy
    ``[3d, d]`` / ``[3d]`` views carrying the arena's low-precision and gradient views; else ``None``."""
    cached = getattr(mod, "_fused_qkv", None)
    wq = mod.linear_q.weight
    arena = getattr(wq, "_arena", None)
    if arena is None:
        return None
    if cached is not None and cached[0] is arena:
        return cached[1]
    res = arena.fuse([mod.linear_q.weight, mod.linear_k.weight, mod.linear_v.weight]) if hasattr(arena, "fuse") else None
    if res is not None and mod.linear_q.bias is not None:
        rb = arena.fuse([mod.linear_q.bias, mod.linear_k.bias, mod.linear_v.bias])
        res = (res, rb) if rb is not None else None
    elif res is not None:
        res = (res, None)
    mod._fused_qkv = (arena, res)
    return res


class RelPositionMultiHeadAttention(MultiHeadAttention):
    # parameters that the optimizer arena should place contiguously (enables the fused QKV GEMM)
    def arena_fusion_groups(self):
        groups = [[self.linear_q.weight, self.linear_k.weight, self.linear_v.weight]]
        if self.linear_q.bias is not None:
            groups.append([self.linear_q.bias, self.linear_k.bias, self.linear_v.bias])
        return groups

    def __init__(self, n_head, n_feat, dropout_rate, pos_bias_u=None, pos_bias_v=None, max_cache_len=0, use_bias=True,
                 use_pytorch_sdpa=False, use_pytorch_sdpa_backends=None):
        super().__init__(n_head, n_feat, dropout_rate, max_cache_len, use_bias)
        self.linear_pos = nn.Linear(n_feat, n_feat, bias=False)
        if pos_bias_u is None or pos_bias_v is None:
            self.pos_bias_u = nn.Parameter(torch.zeros(self.h, self.d_k))
            self.pos_bias_v = nn.Parameter(torch.zeros(self.h, self.d_k))
        else:
            self.pos_bias_u, self.pos_bias_v = pos_bias_u, pos_bias_v

    def forward(self, query, key, value, mask=None, pos_emb=None, cache=None, residual=None, out_dropout: float = 0.0):
        same = query is key and key is value
        key, value, query, cache = self.update_cache(key, value, query, cache)
        if same and cache is None:
            key = value = query
        q, k, v = self._qkv(query, key, value)
        nb = pos_emb.size(0)
        p = ops.linear(pos_emb.to(q.dtype), self.linear_pos.weight, None).view(nb, -1, self.h, self.d_k)
        ctx = ops.relpos_attention(q, k, v, p, self.pos_bias_u, self.pos_bias_v, mask, self.dropout_rate, self.training,
                                   qkv=self._last_qkv)
        self._last_qkv = None
        out = ops.linear(ctx, self.linear_out.weight, self.linear_out.bias, residual=residual, dropout_p=out_dropout)
        return out if cache is None else (out, cache)


class RelPositionMultiHeadAttentionLongformer(RelPositionMultiHeadAttention):
    """Local (sliding window) relative-position attention with optional global tokens, in O(T * window) memory.

    Attention of frame i is restricted to [i-left, i+right]; the ``global_tokens`` frames (every ``global_tokens_spacing``-th
    frame from the start) attend to and are attended by everything.  Relative terms use the window positional table of
    :class:`LocalAttRelPositionalEncoding` and apply inside the band only.  The reference gets the same memory behaviour from
    overlapping-chunk matmuls (``multi_head_attention.py:364-997``, ``sliding_chunks_matmul_qk / _pv``); here the query axis
    is walked in blocks of ``query_block`` frames and each block sees only its ``query_block + left + right`` keys (plus the
    global ones), so no ``[T, T]`` tensor is ever formed and hour-long inputs fit.
    """

    def __init__(self, n_head, n_feat, dropout_rate, pos_bias_u=None, pos_bias_v=None, att_context_size=(128, 128),
                 max_cache_len=0, global_tokens=0, global_tokens_spacing=1, global_attn_separate=False, use_bias=True,
                 query_block: int = 512):
        super().__init__(n_head, n_feat, dropout_rate, pos_bias_u, pos_bias_v, max_cache_len, use_bias)
        self.att_context_size = tuple(att_context_size)
        self.global_tokens, self.global_tokens_spacing = global_tokens, global_tokens_spacing
        self.query_block = int(query_block)

    def forward(self, query, key, value, pad_mask=None, pos_emb=None, cache=None, residual=None, mask=None, out_dropout: float = 0.0):
        B, T, _ = query.shape
        dev = query.device
        q, k, v = self._qkv(query, key, value)
        left, right = self.att_context_size
        p = ops.linear(pos_emb.to(q.dtype), self.linear_pos.weight, None).view(1, -1, self.h, self.d_k)  # window table
        qf = q.float()
        q_u = (qf + self.pos_bias_u.float()).transpose(1, 2)            # [B, H, T, d]
        q_v = (qf + self.pos_bias_v.float()).transpose(1, 2)
        kT = k.float().transpose(1, 2)                                   # [B, H, T, d]
        vT = v.float().transpose(1, 2)
        pT = p.float().transpose(1, 2)                                   # [1, H, W, d]; column c <-> offset i - j = left - c
        g = None
        if self.global_tokens > 0:
            g = torch.arange(0, self.global_tokens * self.global_tokens_spacing, self.global_tokens_spacing, device=dev)
            g = g[g < T]
            kg, vg = kT[:, :, g], vT[:, :, g]
            is_g = torch.zeros(T, dtype=torch.bool, device=dev)
            is_g[g] = True
        ctx = torch.empty(B, self.h, T, self.d_k, dtype=torch.float32, device=dev)
        bq = max(1, self.query_block)
        for i0 in range(0, T, bq):
            i1 = min(T, i0 + bq)
            k0, k1 = max(0, i0 - left), min(T, i1 + right)
            qi = torch.arange(i0, i1, device=dev)[:, None]
            kj = torch.arange(k0, k1, device=dev)[None, :]
            rel = qi - kj
            band = (rel <= left) & (rel >= -right)
            ac = torch.matmul(q_u[:, :, i0:i1], kT[:, :, k0:k1].transpose(-2, -1))                 # [B, H, bq, wk]
            bd_win = torch.matmul(q_v[:, :, i0:i1], pT.transpose(-2, -1))                          # [B, H, bq, W]
            col = (left - rel).clamp(0, left + right)
            bd = torch.gather(bd_win, 3, col[None, None].expand(B, self.h, i1 - i0, k1 - k0))
            scores = (ac + bd) / self.s_d_k
            hidden = (~band)[None].expand(B, i1 - i0, k1 - k0)
            if g is not None:
                hidden = hidden | is_g[k0:k1][None, None, :]          # global keys are counted once, in the global block below
            if pad_mask is not None:
                hidden = hidden | pad_mask[:, None, k0:k1] | pad_mask[:, i0:i1, None]
            scores = scores.masked_fill(hidden[:, None], -INF_VAL)
            if g is not None:
                sg = torch.matmul(q_u[:, :, i0:i1], kg.transpose(-2, -1)) / self.s_d_k             # [B, H, bq, G]
                hg = torch.zeros(B, i1 - i0, g.numel(), dtype=torch.bool, device=dev)
                if pad_mask is not None:
                    hg = hg | pad_mask[:, g][:, None, :] | pad_mask[:, i0:i1, None]
                sg = sg.masked_fill(hg[:, None], -INF_VAL)
                allp = torch.softmax(torch.cat([scores, sg], dim=-1), dim=-1)
                allp = allp.masked_fill(torch.cat([hidden, hg], dim=-1)[:, None], 0.0)
                allp = torch.nn.functional.dropout(allp, self.dropout_rate, self.training)
                wk = k1 - k0
                ctx[:, :, i0:i1] = torch.matmul(allp[..., :wk], vT[:, :, k0:k1]) + torch.matmul(allp[..., wk:], vg)
            else:
                attn = torch.softmax(scores, dim=-1).masked_fill(hidden[:, None], 0.0)
                attn = torch.nn.functional.dropout(attn, self.dropout_rate, self.training)
                ctx[:, :, i0:i1] = torch.matmul(attn, vT[:, :, k0:k1])
        if g is not None and g.numel() > 0:
            # rows of the global frames: full attention over every key ([G, T] scores), content term only
            sg = torch.matmul(q_u[:, :, g], kT.transpose(-2, -1)) / self.s_d_k
            if pad_mask is not None:
                hgr = pad_mask[:, None, :] | pad_mask[:, g][:, :, None]
                sg = sg.masked_fill(hgr[:, None], -INF_VAL)
            ag = torch.softmax(sg, dim=-1)
            if pad_mask is not None:
                ag = ag.masked_fill(hgr[:, None], 0.0)
            ag = torch.nn.functional.dropout(ag, self.dropout_rate, self.training)
            ctx[:, :, g] = torch.matmul(ag, vT)
        ctx = ctx.transpose(1, 2).reshape(B, T, -1).to(query.dtype)
        out = ops.linear(ctx, self.linear_out.weight, self.linear_out.bias, residual=residual, dropout_p=out_dropout)
        return out if cache is None else (out, cache)

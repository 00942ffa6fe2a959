"""Transformer stack used by the TTS models: pre-LN blocks with (optionally causal) self-attention, optional cross-attention
with an additive alignment prior, a convolutional position-wise feed-forward (``kernel_size`` > 1 mixes neighbouring frames),
learnable positional embeddings and a key/value cache for autoregressive decoding.  Optional mixture-of-experts FFN.

Reference: ``tts/modules/transformer_2501.py:29-733`` (``ConvolutionLayer``, ``PositionwiseConvFF``, ``Attention``,
``SelfAttention``, ``CrossAttention``, ``TransformerLayer``, ``Transformer``) and ``tts/modules/moe_modules.py:23,203``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core.module import AdapterModuleMixin


class ConvolutionLayer(nn.Module):
    """Conv1d over [B, T, C] tensors; causal variant pads only on the left."""

    def __init__(self, in_channels, out_channels, kernel_size=1, is_causal=False, bias=False):
        super().__init__()
        self.is_causal, self.k = is_causal, kernel_size
        self.conv = nn.Conv1d(in_channels, out_channels, kernel_size, padding=0 if is_causal else (kernel_size - 1) // 2, bias=bias)

    def forward(self, x):
        if self.k == 1:
            return ops.linear(x, self.conv.weight.squeeze(-1), self.conv.bias)
        y = x.transpose(1, 2)
        if self.is_causal:
            y = F.pad(y, (self.k - 1, 0))
        return self.conv(y.to(self.conv.weight.dtype)).transpose(1, 2).to(x.dtype)


class PositionwiseConvFF(nn.Module):
    def __init__(self, d_model, d_ffn, p_dropout=0.0, kernel_size=1, bias=False, is_causal=True, non_linearity=None):
        super().__init__()
        self.proj = ConvolutionLayer(d_model, d_ffn, kernel_size, is_causal, bias)
        self.o_net = ConvolutionLayer(d_ffn, d_model, kernel_size, is_causal, bias)
        self.act = non_linearity or nn.GELU(approximate="tanh")
        self.dropout = nn.Dropout(p_dropout)

    def forward(self, x):
        return self.dropout(self.o_net(self.act(self.proj(x))))


class MoERouter(nn.Module):
    """Token → expert routing: ``top_k`` softmax routing or Sinkhorn-balanced routing during training; returns the combine
    weights, expert indices and the auxiliary losses (load balancing, router z-loss)."""

    def __init__(self, d_model: int, num_experts: int, top_k: int = 2, routing_strategy: str = "top_k", router_jitter_noise: float = 0.0):
        super().__init__()
        self.num_experts, self.top_k, self.strategy, self.jitter = num_experts, top_k, routing_strategy, router_jitter_noise
        self.router = nn.Linear(d_model, num_experts, bias=False)

    @staticmethod
    def sinkhorn(cost: torch.Tensor, n_iters: int = 8) -> torch.Tensor:
        c = torch.exp(cost.float())
        d0 = torch.ones(c.shape[0], device=c.device)
        d1 = torch.ones(c.shape[1], device=c.device)
        for _ in range(n_iters):
            d0 = 1.0 / (c.shape[0] * (c * d1.unsqueeze(0)).sum(1) + 1e-8)
            d1 = 1.0 / (c.shape[1] * (c * d0.unsqueeze(1)).sum(0) + 1e-8)
        return c * d0.unsqueeze(1) * d1.unsqueeze(0)

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None):
        """x: [N, D] tokens → (weights [N, k], experts [N, k], aux dict)."""
        if self.training and self.jitter > 0:
            x = x * torch.empty_like(x).uniform_(1 - self.jitter, 1 + self.jitter)
        logits = self.router(x.float())
        probs = torch.softmax(logits, dim=-1)
        if self.strategy == "sinkhorn" and self.training:
            with torch.no_grad():
                experts = self.sinkhorn(logits).topk(self.top_k, dim=-1).indices
            weights = probs.gather(-1, experts)
        else:
            weights, experts = probs.topk(self.top_k, dim=-1)
        weights = weights / weights.sum(-1, keepdim=True).clamp(min=1e-9)
        valid = mask.float().view(-1, 1) if mask is not None else torch.ones_like(probs[:, :1])
        frac = (F.one_hot(experts, self.num_experts).float().sum(1) * valid).sum(0) / valid.sum().clamp(min=1) / self.top_k
        mean_p = (probs * valid).sum(0) / valid.sum().clamp(min=1)
        aux = {"load_balancing_loss": self.num_experts * (frac * mean_p).sum(),
               "router_z_loss": ((torch.logsumexp(logits, -1) ** 2) * valid.squeeze(-1)).sum() / valid.sum().clamp(min=1),
               "expert_fraction": frac.detach()}
        return weights.to(x.dtype), experts, aux


class PositionwiseConvFFMoE(nn.Module):
    def __init__(self, d_model, d_ffn, num_experts=4, top_k=2, p_dropout=0.0, kernel_size=1, bias=False, is_causal=True,
                 routing_strategy="top_k", router_jitter_noise=0.0):
        super().__init__()
        self.router = MoERouter(d_model, num_experts, top_k, routing_strategy, router_jitter_noise)
        self.experts = nn.ModuleList([PositionwiseConvFF(d_model, d_ffn, p_dropout, kernel_size, bias, is_causal)
                                      for _ in range(num_experts)])
        self.aux: Dict[str, torch.Tensor] = {}

    def forward(self, x, mask=None):
        B, T, D = x.shape
        w, e, self.aux = self.router(x.reshape(B * T, D), mask.reshape(-1) if mask is not None else None)
        out = torch.zeros_like(x)
        w, e = w.view(B, T, -1), e.view(B, T, -1)
        for i, expert in enumerate(self.experts):
            gate = (w * (e == i)).sum(-1, keepdim=True)            # [B, T, 1]; zero where the expert is not selected
            if bool((gate != 0).any()):
                out = out + gate * expert(x)                        # conv experts need the whole sequence for their context
        return out


class Attention(nn.Module):
    def __init__(self, n_heads, d_model, p_dropout=0.0, is_causal=False, d_memory=None, d_head=None):
        super().__init__()
        self.h, self.dh = n_heads, d_head or d_model // n_heads
        self.is_causal, self.cross = is_causal, d_memory is not None
        inner = self.h * self.dh
        if self.cross:
            self.q_net = nn.Linear(d_model, inner, bias=False)
            self.kv_net = nn.Linear(d_memory, 2 * inner, bias=False)
        else:
            self.qkv_net = nn.Linear(d_model, 3 * inner, bias=False)
        self.o_net = nn.Linear(inner, d_model, bias=False)
        self.dropout = nn.Dropout(p_dropout)
        self.p = p_dropout

    def forward(self, x, x_mask=None, memory=None, memory_mask=None, attn_prior=None, cache: Optional[dict] = None):
        """x: [B, T, D]; masks are True at valid positions.  Returns (y, attention probabilities or None)."""
        B, T, _ = x.shape
        if self.cross:
            q = ops.linear(x, self.q_net.weight, None).view(B, T, self.h, self.dh).transpose(1, 2)
            if cache is not None and "k" in cache:
                k, v = cache["k"], cache["v"]
            else:
                kv = ops.linear(memory, self.kv_net.weight, None).view(B, memory.shape[1], 2, self.h, self.dh)
                k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
                if cache is not None:
                    cache["k"], cache["v"] = k, v
            kmask = memory_mask
        else:
            qkv = ops.linear(x, self.qkv_net.weight, None).view(B, T, 3, self.h, self.dh)
            q, k, v = qkv[:, :, 0].transpose(1, 2), qkv[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)
            if cache is not None:
                if "k" in cache:
                    k, v = torch.cat([cache["k"], k], 2), torch.cat([cache["v"], v], 2)
                cache["k"], cache["v"] = k, v
            kmask = x_mask if (cache is None or k.shape[2] == T) else None
        Tk = k.shape[2]
        need_probs = attn_prior is not None or (self.cross and self.training)
        bias = None
        if kmask is not None:
            bias = torch.zeros((B, 1, 1, Tk), dtype=q.dtype, device=q.device).masked_fill(~kmask.bool().view(B, 1, 1, Tk), float("-inf"))
        if self.is_causal and not self.cross and Tk > 1:
            i = torch.arange(Tk - T, Tk, device=q.device).view(T, 1)
            j = torch.arange(Tk, device=q.device).view(1, Tk)
            cm = torch.zeros((T, Tk), dtype=q.dtype, device=q.device).masked_fill(j > i, float("-inf"))
            bias = cm if bias is None else bias + cm
        if need_probs:
            s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(self.dh)
            if bias is not None:
                s = s + bias.float()
            if attn_prior is not None:
                s = torch.log_softmax(s, dim=-1) + torch.log(attn_prior.float().unsqueeze(1) + 1e-8)
            p = torch.softmax(s, dim=-1)
            y = torch.matmul(self.dropout(p).to(v.dtype), v)
            probs = p
        else:
            y = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, dropout_p=self.p if self.training else 0.0)
            probs = None
        y = y.transpose(1, 2).reshape(B, T, self.h * self.dh)
        return ops.linear(y, self.o_net.weight, None), probs


class TransformerLayer(nn.Module, AdapterModuleMixin):
    def __init__(self, d_model, d_ffn, sa_n_heads, kernel_size, p_dropout, has_xattn, xa_d_memory=None, xa_n_heads=None,
                 is_causal=True, apply_norm_to_cond=True, use_moe=False, num_experts=4, top_k_experts=2, routing_strategy="top_k",
                 router_jitter_noise=0.0):
        super().__init__()
        self.norm_self = nn.LayerNorm(d_model, bias=False)
        self.self_attention = Attention(sa_n_heads, d_model, p_dropout, is_causal)
        self.has_xattn = has_xattn
        if has_xattn:
            self.norm_xattn_query = nn.LayerNorm(d_model, bias=False)
            self.cross_attention = Attention(xa_n_heads, d_model, p_dropout, False, d_memory=xa_d_memory)
            self.norm_xattn_memory = nn.LayerNorm(xa_d_memory, bias=False) if apply_norm_to_cond else nn.Identity()
        self.norm_pos_ff = nn.LayerNorm(d_model, bias=False)
        self.use_moe = use_moe
        self.pos_ff = (PositionwiseConvFFMoE(d_model, d_ffn, num_experts, top_k_experts, p_dropout, kernel_size, False, is_causal,
                                             routing_strategy, router_jitter_noise)
                       if use_moe else PositionwiseConvFF(d_model, d_ffn, p_dropout, kernel_size, False, is_causal))

    def forward(self, x, x_mask, cond=None, cond_mask=None, attn_prior=None, cache: Optional[dict] = None):
        m = x_mask.unsqueeze(-1).to(x.dtype) if x_mask is not None else 1.0
        a, _ = self.self_attention(self.norm_self(x), x_mask, cache=None if cache is None else cache.setdefault("self", {}))
        x = (x + a) * m
        probs = None
        if self.has_xattn and cond is not None:
            mem = self.norm_xattn_memory(cond)
            a, probs = self.cross_attention(self.norm_xattn_query(x), x_mask, mem, cond_mask, attn_prior,
                                            cache=None if cache is None else cache.setdefault("cross", {}))
            x = (x + a) * m
        ff = self.pos_ff(self.norm_pos_ff(x), x_mask) if self.use_moe else self.pos_ff(self.norm_pos_ff(x))
        x = (x + ff) * m
        if self.is_adapter_available():                              # adapters sit at the end of the layer, merged by their strategy (residual add)
            x = self.forward_enabled_adapters(x) * m
        return x, probs


class Transformer(nn.Module):
    def __init__(self, n_layers, d_model, d_ffn, sa_n_heads, kernel_size=1, p_dropout=0.0, p_dropout_out=0.0, has_xattn=False,
                 xa_d_memory=None, xa_n_heads=None, is_causal=True, apply_norm_to_cond=True, apply_norm_out=False,
                 max_length_causal_mask=4096, use_learnable_pos_emb=False, use_moe=False, num_experts=4, top_k_experts=2,
                 routing_strategy="top_k", router_jitter_noise=0.0, **_):
        super().__init__()
        self.d_model = d_model
        self.dropout = nn.Dropout(p_dropout)
        self.p_dropout_out = p_dropout_out
        self.norm_out = nn.LayerNorm(d_model, bias=False) if apply_norm_out else nn.Identity()
        self.position_embeddings = nn.Embedding(max_length_causal_mask, d_model) if use_learnable_pos_emb else None
        self.layers = nn.ModuleList([TransformerLayer(d_model, d_ffn, sa_n_heads, kernel_size, p_dropout, has_xattn, xa_d_memory,
                                                      xa_n_heads, is_causal, apply_norm_to_cond, use_moe, num_experts, top_k_experts,
                                                      routing_strategy, router_jitter_noise) for _ in range(n_layers)])
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Conv1d, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def new_cache(self) -> List[dict]:
        return [dict() for _ in self.layers]

    # ------------------------------------------------------------------ adapters (every layer hosts a copy)
    def add_adapter(self, name: str, cfg) -> None:
        for layer in self.layers:
            layer.add_adapter(name, cfg)

    def is_adapter_available(self) -> bool:
        return any(layer.is_adapter_available() for layer in self.layers)

    @property
    def adapter_cfg(self) -> dict:
        """Names and configs of the hosted adapters (the layers hold identical sets)."""
        return next((layer.adapter_cfg for layer in self.layers if layer.is_adapter_available()), {})

    def set_enabled_adapters(self, name=None, enabled: bool = True) -> None:
        for layer in self.layers:
            if layer.is_adapter_available():
                layer.set_enabled_adapters(name, enabled)

    def get_enabled_adapters(self) -> List[str]:
        names: List[str] = []
        for layer in self.layers:
            for n in layer.get_enabled_adapters():
                if n not in names:
                    names.append(n)
        return names

    def unfreeze_enabled_adapters(self, freeze_batchnorm: bool = True) -> None:
        for layer in self.layers:
            if layer.is_adapter_available():
                layer.unfreeze_enabled_adapters(freeze_batchnorm)

    def moe_aux_losses(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for l in self.layers:
            if l.use_moe:
                for k, v in l.pos_ff.aux.items():
                    if v.dim() == 0:
                        out[k] = out.get(k, 0.0) + v / len(self.layers)
        return out

    def forward(self, x, x_mask, cond=None, cond_mask=None, attn_prior=None, cache: Optional[List[dict]] = None,
                position_offset: int = 0) -> Dict[str, object]:
        """x: [B, T, D]; x_mask: [B, T] bool.  ``attn_prior`` [B, T, T_cond] may be a list (one per layer, ``None`` entries
        skip the prior).  Returns ``{"output", "attn_probabilities"}``."""
        if self.position_embeddings is not None:
            pos = torch.arange(position_offset, position_offset + x.shape[1], device=x.device)
            x = x + self.position_embeddings(pos.clamp(max=self.position_embeddings.num_embeddings - 1)).unsqueeze(0).to(x.dtype)
        x = self.dropout(x)
        cdt = ops.get_compute_dtype()
        if cdt is not None and x.dtype != cdt:
            x = x.to(cdt)
            cond = cond.to(cdt) if cond is not None else None
        probs = []
        for i, layer in enumerate(self.layers):
            prior = attn_prior[i] if isinstance(attn_prior, (list, tuple)) else attn_prior
            x, p = layer(x, x_mask, cond, cond_mask, prior, None if cache is None else cache[i])
            probs.append(p)
        x = self.norm_out(x.float()).to(x.dtype) if not isinstance(self.norm_out, nn.Identity) else x
        if self.p_dropout_out > 0:
            x = F.dropout(x, self.p_dropout_out, self.training)
        return {"output": x, "attn_probabilities": probs}

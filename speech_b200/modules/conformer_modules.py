"""Conformer layer: macaron feed-forward halves, relative-position self-attention, convolution module.

Layer structure ``x + 1/2 FF(LN x) -> + MHSA(LN .) -> + Conv(LN .) -> + 1/2 FF(LN .) -> LN`` and sub-module /
parameter names follow ``nemo/collections/asr/parts/submodules/conformer_modules.py:36-415``.  The
compute is routed through ``speech_b200.ops`` so that on a GPU each block is a handful of fused
kernels: LayerNorm, GEMM with bias+Swish epilogue, GEMM with bias+scaled-residual epilogue, the
fused GLU + depthwise conv + norm + SiLU kernel, and the attention kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..core.module import AccessMixin, AdapterModuleMixin
from .attention import MultiHeadAttention, RelPositionMultiHeadAttention, RelPositionMultiHeadAttentionLongformer


class CausalConv1D(nn.Conv1d):
    """Conv1d with explicit (left, right) padding and a streaming cache (reference: ``causal_convs.py:73-151``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True):
        self.cache_drop_size = None
        if padding is None:
            self._left_padding, self._right_padding = kernel_size - 1, stride - 1
        elif isinstance(padding, int):
            self._left_padding = self._right_padding = padding
        elif isinstance(padding, (list, tuple)) and len(padding) == 2 and padding[0] + padding[1] == kernel_size - 1:
            self._left_padding, self._right_padding = padding
        else:
            raise ValueError(f"Invalid padding param: {padding}!")
        self._max_cache_len = self._left_padding
        super().__init__(in_channels, out_channels, kernel_size, stride, 0, dilation, groups, bias)

    def update_cache(self, x, cache=None):
        if cache is None:
            return torch.nn.functional.pad(x, (self._left_padding, self._right_padding)), None
        new_x = torch.cat([cache.to(x.dtype), torch.nn.functional.pad(x, (0, self._right_padding))], dim=-1)
        nxt = new_x[:, :, : -self.cache_drop_size] if self.cache_drop_size and self.cache_drop_size > 0 else new_x
        return new_x, nxt[:, :, -cache.size(-1):]

    def forward(self, x, cache=None):
        x, cache = self.update_cache(x, cache)
        x = super().forward(x)
        return x if cache is None else (x, cache)


class ConformerFeedForward(nn.Module):
    def __init__(self, d_model, d_ff, dropout, activation=None, use_bias=True):
        super().__init__()
        self.d_model, self.d_ff, self.use_bias = d_model, d_ff, use_bias
        self.linear1 = nn.Linear(d_model, d_ff, bias=use_bias)
        self.activation = activation if activation is not None else nn.SiLU()
        self.dropout = nn.Dropout(p=dropout)
        self.linear2 = nn.Linear(d_ff, d_model, bias=use_bias)

    def forward(self, x, residual=None, alpha: float = 1.0):
        """``residual + alpha * FF(x)``; dropout (if any) is applied between the two GEMMs and on the output."""
        p = self.dropout.p if self.training else 0.0
        h = ops.linear(x, self.linear1.weight, self.linear1.bias, act="swish", dropout_p=p)
        return ops.linear(h, self.linear2.weight, self.linear2.bias, residual=residual, alpha=alpha, dropout_p=p)

    def reset_parameters_ff(self):
        ffn1_max, ffn2_max = self.d_model ** -0.5, self.d_ff ** -0.5
        with torch.no_grad():
            nn.init.uniform_(self.linear1.weight, -ffn1_max, ffn1_max)
            nn.init.uniform_(self.linear2.weight, -ffn2_max, ffn2_max)
            if self.use_bias:
                nn.init.uniform_(self.linear1.bias, -ffn1_max, ffn1_max)
                nn.init.uniform_(self.linear2.bias, -ffn2_max, ffn2_max)


class ConformerConvolution(nn.Module):
    def __init__(self, d_model, kernel_size, norm_type="batch_norm", conv_context_size=None,
                 pointwise_activation="glu_", use_bias=True):
        super().__init__()
        assert (kernel_size - 1) % 2 == 0
        self.d_model, self.kernel_size, self.norm_type, self.use_bias = d_model, kernel_size, norm_type, use_bias
        if conv_context_size is None:
            conv_context_size = [(kernel_size - 1) // 2, (kernel_size - 1) // 2]
        self.conv_context_size = list(conv_context_size)
        self.pointwise_activation = pointwise_activation
        dw_in = d_model if pointwise_activation == "glu_" else d_model * 2
        self.pointwise_conv1 = nn.Conv1d(d_model, d_model * 2, kernel_size=1, bias=use_bias)
        self.depthwise_conv = CausalConv1D(dw_in, dw_in, kernel_size, stride=1, padding=self.conv_context_size,
                                           groups=dw_in, bias=use_bias)
        if norm_type == "batch_norm":
            self.batch_norm = nn.BatchNorm1d(dw_in)
        elif norm_type == "instance_norm":
            self.batch_norm = nn.InstanceNorm1d(dw_in)
        elif norm_type == "layer_norm":
            self.batch_norm = nn.LayerNorm(dw_in)
        elif norm_type == "fused_batch_norm":
            self.batch_norm = FusedBatchNorm1d(dw_in)
        elif norm_type.startswith("group_norm"):
            self.batch_norm = nn.GroupNorm(num_groups=int(norm_type.replace("group_norm", "")), num_channels=d_model)
        else:
            raise ValueError(f"conv_norm_type={norm_type} is not valid!")
        self.activation = nn.SiLU()
        self.pointwise_conv2 = nn.Conv1d(dw_in, d_model, kernel_size=1, bias=use_bias)
        self.bn_stats_reduce = None  # set by the data-parallel strategy for synchronised BatchNorm

    def forward(self, x, pad_mask=None, cache=None, residual=None, out_dropout: float = 0.0):
        g = ops.linear(x, self.pointwise_conv1.weight.squeeze(-1), self.pointwise_conv1.bias)
        fusable = self.pointwise_activation == "glu_" and self.norm_type in ("batch_norm", "layer_norm")
        if fusable:
            bn = self.batch_norm
            is_bn = self.norm_type == "batch_norm"
            res = ops.conv_module_core(
                g, self.depthwise_conv.weight, self.depthwise_conv.bias, self.norm_type, bn.weight, bn.bias,
                bn.running_mean if is_bn else None, bn.running_var if is_bn else None, pad_mask=pad_mask,
                training=self.training, momentum=(bn.momentum if is_bn else 0.1), eps=bn.eps,
                left_pad=self.depthwise_conv._left_padding, right_pad=self.depthwise_conv._right_padding, cache=cache,
                cache_drop_size=self.depthwise_conv.cache_drop_size or 0,
                bn_stats_reduce=self.bn_stats_reduce if (is_bn and self.training) else None)
            if cache is not None:
                s, cache = res
            else:
                s = res
            if is_bn and self.training and bn.num_batches_tracked is not None:
                bn.num_batches_tracked += 1
        else:
            xt = g.transpose(1, 2)
            xt = nn.functional.glu(xt, dim=1) if self.pointwise_activation == "glu_" else nn.functional.silu(xt)
            if pad_mask is not None:
                xt = xt.masked_fill(pad_mask.unsqueeze(1), 0.0)
            xt = self.depthwise_conv(xt, cache=cache)
            if cache is not None:
                xt, cache = xt
            xt = self.batch_norm(xt)
            s = self.activation(xt).transpose(1, 2)
        y = ops.linear(s, self.pointwise_conv2.weight.squeeze(-1), self.pointwise_conv2.bias, residual=residual,
                       dropout_p=out_dropout)
        return y if cache is None else (y, cache)

    def reset_parameters_conv(self):
        pw_max, dw_max = self.d_model ** -0.5, self.kernel_size ** -0.5
        with torch.no_grad():
            nn.init.uniform_(self.pointwise_conv1.weight, -pw_max, pw_max)
            nn.init.uniform_(self.pointwise_conv2.weight, -pw_max, pw_max)
            nn.init.uniform_(self.depthwise_conv.weight, -dw_max, dw_max)
            if self.use_bias:
                nn.init.uniform_(self.pointwise_conv1.bias, -pw_max, pw_max)
                nn.init.uniform_(self.pointwise_conv2.bias, -pw_max, pw_max)
                nn.init.uniform_(self.depthwise_conv.bias, -dw_max, dw_max)


class FusedBatchNorm1d(nn.Module):
    """Inference-time BatchNorm folded to a per-channel affine (reference: ``submodules/batchnorm.py:24``)."""

    def __init__(self, num_features: int):
        super().__init__()
        self.num_features = num_features
        self.weight = nn.Parameter(torch.ones(num_features))
        self.bias = nn.Parameter(torch.zeros(num_features))

    @classmethod
    def from_batchnorm(cls, bn: nn.BatchNorm1d) -> "FusedBatchNorm1d":
        f = cls(bn.num_features)
        std = torch.sqrt(bn.running_var.data + bn.eps)
        f.weight.data = bn.weight.data / std
        f.bias.data = bn.bias.data - bn.running_mean.data * f.weight.data
        return f

    def forward(self, x):
        return x * self.weight.unsqueeze(-1) + self.bias.unsqueeze(-1) if x.dim() == 3 else x * self.weight + self.bias


class ConformerLayer(nn.Module, AdapterModuleMixin, AccessMixin):
    def __init__(self, d_model, d_ff, self_attention_model="rel_pos", global_tokens=0, global_tokens_spacing=1,
                 global_attn_separate=False, n_heads=4, conv_kernel_size=31, conv_norm_type="batch_norm",
                 conv_context_size=None, dropout=0.1, dropout_att=0.1, pos_bias_u=None, pos_bias_v=None,
                 att_context_size=(-1, -1), use_bias=True, use_pytorch_sdpa=False, use_pytorch_sdpa_backends=None):
        super().__init__()
        self.self_attention_model = self_attention_model
        self.fc_factor = 0.5
        self.norm_feed_forward1 = nn.LayerNorm(d_model)
        self.feed_forward1 = ConformerFeedForward(d_model, d_ff, dropout, use_bias=use_bias)
        self.norm_conv = nn.LayerNorm(d_model)
        self.conv = ConformerConvolution(d_model, conv_kernel_size, conv_norm_type, conv_context_size, use_bias=use_bias)
        self.norm_self_att = nn.LayerNorm(d_model)
        mhc = att_context_size[0] if att_context_size[0] >= 0 else 0
        if self_attention_model == "rel_pos":
            self.self_attn = RelPositionMultiHeadAttention(n_heads, d_model, dropout_att, pos_bias_u, pos_bias_v, mhc, use_bias)
        elif self_attention_model == "rel_pos_local_attn":
            self.self_attn = RelPositionMultiHeadAttentionLongformer(
                n_heads, d_model, dropout_att, pos_bias_u, pos_bias_v, att_context_size, mhc, global_tokens,
                global_tokens_spacing, global_attn_separate, use_bias)
        elif self_attention_model == "abs_pos":
            self.self_attn = MultiHeadAttention(n_heads, d_model, dropout_att, mhc, use_bias)
        else:
            raise ValueError(f"'{self_attention_model}' is not a valid value for 'self_attention_model', valid values "
                             f"can be from ['rel_pos', 'rel_pos_local_attn', 'abs_pos']")
        self.norm_feed_forward2 = nn.LayerNorm(d_model)
        self.feed_forward2 = ConformerFeedForward(d_model, d_ff, dropout, use_bias=use_bias)
        self.dropout = nn.Dropout(dropout)
        self.norm_out = nn.LayerNorm(d_model)

    def _ln(self, ln: nn.LayerNorm, x):
        return ops.layer_norm(x, ln.weight, ln.bias, ln.eps)

    def forward(self, x, att_mask=None, pos_emb=None, pad_mask=None, cache_last_channel=None, cache_last_time=None):
        if cache_last_channel is None and cache_last_time is None and x.is_cuda and not self.is_adapter_available() \
                and not self.is_access_enabled(getattr(self, "model_guid", None)):
            out = ops.conformer_layer(self, x, att_mask, pos_emb, pad_mask)   # one native call for the whole layer
            if out is not None:
                return out
        # dropout on the module outputs is fused into the epilogue of each module's last GEMM: residual + dropout(out)
        p_out = self.dropout.p if self.training else 0.0
        residual = self.feed_forward1(self._ln(self.norm_feed_forward1, x), residual=x, alpha=self.fc_factor)
        h = self._ln(self.norm_self_att, residual)
        kw = dict(query=h, key=h, value=h, pos_emb=pos_emb, cache=cache_last_channel, out_dropout=p_out)
        if self.self_attention_model == "rel_pos_local_attn":
            kw["pad_mask"] = pad_mask
        else:
            kw["mask"] = att_mask
        if self.self_attention_model == "abs_pos":
            kw.pop("pos_emb")
        a = self.self_attn(residual=residual, **kw)
        if cache_last_channel is not None:
            a, cache_last_channel = a
        residual = a
        if self.is_adapter_available():
            residual = self.forward_enabled_adapters(residual)
        h = self._ln(self.norm_conv, residual)
        c = self.conv(h, pad_mask=pad_mask, cache=cache_last_time, residual=residual, out_dropout=p_out)
        if cache_last_time is not None:
            c, cache_last_time = c
        residual = c
        residual = self.feed_forward2(self._ln(self.norm_feed_forward2, residual), residual=residual, alpha=self.fc_factor)
        out = self._ln(self.norm_out, residual)
        if self.is_access_enabled(getattr(self, "model_guid", None)) and self.access_cfg.get("save_encoder_tensors", False):
            self.register_accessible_tensor(name="encoder", tensor=out)
        if cache_last_channel is None:
            return out
        return out, cache_last_channel, cache_last_time

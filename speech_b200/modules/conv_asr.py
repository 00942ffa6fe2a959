"""Convolutional encoders and heads: Jasper / QuartzNet / Citrinet / MarbleNet / TitaNet blocks, ECAPA-TDNN, the
classification and speaker-embedding decoders.

Parameter names follow the reference (``modules/conv_asr.py``, ``parts/submodules/jasper.py``,
``parts/submodules/tdnn_attention.py``) so their checkpoints load: ``encoder.<i>.mconv.<j>`` for the block's conv / norm
sequence, ``encoder.<i>.res.<k>`` for residual projections, ``mout`` for the block output activation.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.module import NeuralModule

jasper_activations = {"hardtanh": nn.Hardtanh, "relu": nn.ReLU, "selu": nn.SELU, "swish": nn.SiLU, "silu": nn.SiLU,
                      "gelu": nn.GELU}


def get_same_padding(kernel_size: int, stride: int, dilation: int) -> int:
    if stride > 1 and dilation > 1:
        raise ValueError("Only stride OR dilation may be greater than 1")
    return (dilation * (kernel_size - 1)) // 2


def compute_new_kernel_size(kernel_size: int, kernel_width: float) -> int:
    k = max(int(kernel_size * kernel_width), 1)
    return k + 1 if k % 2 == 0 else k


class MaskedConv1d(nn.Module):
    """Conv1d that zeroes frames beyond each sequence's length before convolving and tracks the output lengths."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, heads=-1,
                 bias=False, use_mask=True):
        super().__init__()
        if heads != -1:
            in_channels = out_channels = groups = heads
        self.real_out_channels = out_channels
        self.heads = heads
        self.conv = nn.Conv1d(in_channels, out_channels, kernel_size, stride=stride, padding=padding, dilation=dilation,
                              groups=groups, bias=bias)
        self.use_mask = use_mask

    def get_seq_len(self, lens):
        c = self.conv
        return torch.div(lens + 2 * c.padding[0] - c.dilation[0] * (c.kernel_size[0] - 1) - 1, c.stride[0],
                         rounding_mode="trunc") + 1

    def forward(self, x, lens):
        if self.use_mask and lens is not None:
            mask = torch.arange(x.shape[-1], device=x.device)[None, :] < lens[:, None]
            x = x * mask.unsqueeze(1).to(x.dtype)
            lens = self.get_seq_len(lens)
        sh = x.shape
        if self.heads != -1:
            x = x.reshape(-1, self.heads, sh[-1])
        out = self.conv(x)
        if self.heads != -1:
            out = out.reshape(sh[0], self.real_out_channels if self.heads == -1 else sh[1], -1)
        return out, lens


class SqueezeExcite(nn.Module):
    def __init__(self, channels: int, reduction_ratio: int, context_window: int = -1, interpolation_mode: str = "nearest",
                 activation=None):
        super().__init__()
        self.context_window = context_window
        self.interpolation_mode = interpolation_mode
        self.fc = nn.Sequential(nn.Linear(channels, channels // reduction_ratio, bias=False),
                                activation or nn.ReLU(inplace=True),
                                nn.Linear(channels // reduction_ratio, channels, bias=False))

    def forward(self, x, lengths):
        T = x.shape[-1]
        mask = (torch.arange(T, device=x.device)[None, :] < lengths[:, None]).unsqueeze(1).to(x.dtype)
        xm = x * mask
        if self.context_window <= 0 or self.context_window >= T:
            y = xm.sum(dim=-1, keepdim=True) / lengths.clamp(min=1).view(-1, 1, 1).to(x.dtype)
        else:
            y = F.avg_pool1d(xm, self.context_window, stride=1, padding=self.context_window // 2, count_include_pad=False)
            y = y[..., :T]
        y = self.fc(y.transpose(1, -1)).transpose(1, -1)
        return x * torch.sigmoid(y), lengths


class JasperBlock(nn.Module):
    def __init__(self, inplanes, planes, repeat=3, kernel_size=11, kernel_size_factor=1, stride=1, dilation=1,
                 padding="same", dropout=0.2, activation=None, residual=True, groups=1, separable=False, heads=-1,
                 normalization="batch", norm_groups=1, residual_mode="add", residual_panes=(), conv_mask=False, se=False,
                 se_reduction_ratio=16, se_context_window=-1, se_interpolation_mode="nearest", stride_last=False, **_):
        super().__init__()
        if padding != "same":
            raise ValueError("currently only 'same' padding is supported")
        ks = [compute_new_kernel_size(k, kernel_size_factor) for k in (kernel_size if isinstance(kernel_size, (list, tuple))
                                                                      else [kernel_size])]
        stride = list(stride) if isinstance(stride, (list, tuple)) else [stride]
        dilation = list(dilation) if isinstance(dilation, (list, tuple)) else [dilation]
        pad = get_same_padding(ks[0], stride[0], dilation[0])
        self.conv_mask, self.separable, self.residual_mode, self.se = conv_mask, separable, residual_mode, se
        act = activation or nn.Hardtanh(min_val=0.0, max_val=20.0)
        cin = inplanes
        layers: List[nn.Module] = []
        for i in range(repeat - 1):
            s = [1] if stride_last else stride
            layers += self._conv_bn(cin, planes, ks, s, dilation, pad, groups, heads, separable, normalization, norm_groups)
            layers += [act, nn.Dropout(dropout)]
            cin = planes
        layers += self._conv_bn(cin, planes, ks, stride, dilation, pad, groups, heads, separable, normalization, norm_groups)
        if se:
            layers.append(SqueezeExcite(planes, se_reduction_ratio, se_context_window, se_interpolation_mode, activation=None))
        self.mconv = nn.ModuleList(layers)
        res_panes = list(residual_panes)
        self.dense_residual = residual
        if residual:
            self.res = nn.ModuleList()
            panes = res_panes if res_panes else [inplanes]
            self.dense_residual = bool(res_panes)
            for ip in panes:
                self.res.append(nn.ModuleList(self._conv_bn(ip, planes, [1], stride if not stride_last else stride, [1], 0, 1, -1,
                                                            False, normalization, norm_groups)))
        else:
            self.res = None
        self.mout = nn.Sequential(act, nn.Dropout(dropout))

    def _conv_bn(self, cin, cout, ks, stride, dilation, pad, groups, heads, separable, normalization, norm_groups):
        if separable:
            layers = [MaskedConv1d(cin, cin, ks[0], stride=stride[0], dilation=dilation[0], padding=pad, groups=cin,
                                   heads=heads, use_mask=self.conv_mask),
                      MaskedConv1d(cin, cout, 1, groups=groups, use_mask=self.conv_mask)]
        else:
            layers = [MaskedConv1d(cin, cout, ks[0], stride=stride[0], dilation=dilation[0], padding=pad, groups=groups,
                                   use_mask=self.conv_mask)]
        if normalization == "group":
            layers.append(nn.GroupNorm(norm_groups, cout))
        elif normalization == "instance":
            layers.append(nn.GroupNorm(cout, cout))
        elif normalization == "layer":
            layers.append(nn.GroupNorm(1, cout))
        else:
            layers.append(nn.BatchNorm1d(cout, eps=1e-3, momentum=0.1))
        return layers

    def forward(self, inputs):
        xs, lens_orig = inputs
        out, lens = xs[-1], lens_orig
        for layer in self.mconv:
            if isinstance(layer, (MaskedConv1d, SqueezeExcite)):
                out, lens = layer(out, lens)
            else:
                out = layer(out)
        if self.res is not None:
            for i, layer in enumerate(self.res):
                r = xs[i]
                for sub in layer:
                    if isinstance(sub, MaskedConv1d):
                        r, _ = sub(r, lens_orig)
                    else:
                        r = sub(r)
                out = out + r if self.residual_mode in ("add", "stride_add") else torch.max(out, r)
        out = self.mout(out)
        if self.res is not None and self.dense_residual:
            return xs + [out], lens
        return [out], lens


def init_weights(m, mode: Optional[str] = "xavier_uniform"):
    if isinstance(m, MaskedConv1d):
        init_weights(m.conv, mode)
    if isinstance(m, (nn.Conv1d, nn.Linear)) and mode is not None:
        {"xavier_uniform": lambda w: nn.init.xavier_uniform_(w, gain=1.0), "xavier_normal": lambda w: nn.init.xavier_normal_(w),
         "kaiming_uniform": lambda w: nn.init.kaiming_uniform_(w, nonlinearity="relu"),
         "kaiming_normal": lambda w: nn.init.kaiming_normal_(w, nonlinearity="relu")}[mode](m.weight)


class ConvASREncoder(NeuralModule):
    """Stack of Jasper blocks described by the ``jasper`` list of the config (reference ``conv_asr.py:60-220``)."""

    def __init__(self, jasper: Sequence[dict], activation: str, feat_in: int, normalization_mode: str = "batch",
                 residual_mode: str = "add", norm_groups: int = -1, conv_mask: bool = True, frame_splicing: int = 1,
                 init_mode: Optional[str] = "xavier_uniform", quantize: bool = False):
        super().__init__()
        act = jasper_activations[activation]()
        feat_in = feat_in * frame_splicing
        self._feat_in = feat_in
        residual_panes: List[int] = []
        blocks = []
        self.dense_residual = False
        for lcfg in jasper:
            lcfg = dict(lcfg)
            dense = []
            if lcfg.get("residual_dense", False):
                residual_panes.append(feat_in)
                dense = list(residual_panes)
                self.dense_residual = True
            filters = lcfg["filters"]
            blocks.append(JasperBlock(
                feat_in, filters, repeat=lcfg["repeat"], kernel_size=lcfg["kernel"], stride=lcfg["stride"],
                dilation=lcfg["dilation"], dropout=lcfg.get("dropout", 0.0), residual=lcfg["residual"],
                groups=lcfg.get("groups", 1), separable=lcfg.get("separable", False), heads=lcfg.get("heads", -1),
                residual_mode=lcfg.get("residual_mode", residual_mode), normalization=normalization_mode,
                norm_groups=norm_groups, activation=act, residual_panes=dense, conv_mask=conv_mask, se=lcfg.get("se", False),
                se_reduction_ratio=lcfg.get("se_reduction_ratio", 8), se_context_window=lcfg.get("se_context_size", -1),
                se_interpolation_mode=lcfg.get("se_interpolation_mode", "nearest"),
                kernel_size_factor=lcfg.get("kernel_size_factor", 1.0), stride_last=lcfg.get("stride_last", False)))
            feat_in = filters
        self._feat_out = feat_in
        self.encoder = nn.Sequential(*blocks)
        self.apply(lambda m: init_weights(m, init_mode))
        self.max_audio_length = 0
        self.subsampling_factor = int(math.prod(int(b["stride"][0] if isinstance(b["stride"], (list, tuple)) else b["stride"])
                                                for b in jasper))

    def forward(self, audio_signal, length=None):
        if length is None:
            length = audio_signal.new_full((audio_signal.shape[0],), audio_signal.shape[-1], dtype=torch.long)
        s_input, length = self.encoder(([audio_signal], length))
        return s_input[-1], length


class ParallelConvASREncoder(ConvASREncoder):
    pass


class ConvASRDecoderClassification(NeuralModule):
    """Pooling over time + linear classifier (``conv_asr.py:586-672``)."""

    def __init__(self, feat_in: int, num_classes: int, init_mode: Optional[str] = "xavier_uniform", return_logits: bool = True,
                 pooling_type: str = "avg"):
        super().__init__()
        self._feat_in, self._num_classes, self._return_logits = feat_in, num_classes, return_logits
        self.pooling_type = pooling_type
        self.decoder_layers = nn.Sequential(nn.Linear(feat_in, num_classes, bias=True))
        self.apply(lambda m: init_weights(m, init_mode))

    @property
    def num_classes(self):
        return self._num_classes

    @property
    def vocabulary(self):
        return getattr(self, "_vocabulary", None)

    def forward(self, encoder_output, length=None):
        if length is not None:
            mask = (torch.arange(encoder_output.shape[-1], device=encoder_output.device)[None] < length[:, None]).unsqueeze(1)
            if self.pooling_type == "max":
                pooled = encoder_output.masked_fill(~mask, float("-inf")).max(dim=-1).values
            else:
                pooled = (encoder_output * mask).sum(-1) / length.clamp(min=1).unsqueeze(1)
        else:
            pooled = encoder_output.max(-1).values if self.pooling_type == "max" else encoder_output.mean(-1)
        logits = self.decoder_layers(pooled)
        return logits if self._return_logits else torch.softmax(logits, dim=-1)


class StatsPoolLayer(nn.Module):
    def __init__(self, feat_in: int, pool_mode: str = "xvector", eps: float = 1e-10, unbiased: bool = True):
        super().__init__()
        self.pool_mode, self.eps, self.unbiased = pool_mode, eps, unbiased
        self.feat_in = feat_in * (2 if pool_mode == "xvector" else 1)

    def forward(self, x, length=None):
        if length is None:
            mean = x.mean(-1)
            std = x.std(-1, unbiased=self.unbiased)
        else:
            mask = (torch.arange(x.shape[-1], device=x.device)[None] < length[:, None]).unsqueeze(1).to(x.dtype)
            n = length.clamp(min=1).view(-1, 1).to(x.dtype)
            mean = (x * mask).sum(-1) / n
            var = (((x - mean.unsqueeze(-1)) * mask) ** 2).sum(-1) / (n - (1 if self.unbiased else 0)).clamp(min=1)
            std = (var + self.eps).sqrt()
        return torch.cat([mean, std], dim=-1) if self.pool_mode == "xvector" else mean


class TDNNModule(nn.Module):
    def __init__(self, inp_filters, out_filters, kernel_size=1, dilation=1, stride=1, padding=None):
        super().__init__()
        padding = get_same_padding(kernel_size, stride, dilation) if padding is None else padding
        self.conv_layer = nn.Conv1d(inp_filters, out_filters, kernel_size, dilation=dilation, padding=padding)
        self.activation = nn.ReLU()
        self.bn = nn.BatchNorm1d(out_filters)

    def forward(self, x, length=None):
        return self.bn(self.activation(self.conv_layer(x)))


class AttentivePoolLayer(nn.Module):
    """Channel-dependent attentive statistics pooling (``tdnn_attention.py`` ``AttentivePoolLayer``)."""

    def __init__(self, inp_filters: int, attention_channels: int = 128, kernel_size: int = 1, dilation: int = 1, eps: float = 1e-10):
        super().__init__()
        self.feat_in = 2 * inp_filters
        self.attention_layer = nn.Sequential(TDNNModule(inp_filters * 3, attention_channels, kernel_size, dilation), nn.Tanh(),
                                             nn.Conv1d(attention_channels, inp_filters, kernel_size, dilation=dilation))
        self.eps = eps

    def forward(self, x, length=None):
        T = x.shape[-1]
        if length is None:
            length = x.new_full((x.shape[0],), T, dtype=torch.long)
        mask = (torch.arange(T, device=x.device)[None] < length[:, None]).unsqueeze(1)
        n = length.clamp(min=1).view(-1, 1, 1).to(x.dtype)
        mean = (x * mask).sum(-1, keepdim=True) / n
        std = ((((x - mean) * mask) ** 2).sum(-1, keepdim=True) / n).clamp(min=self.eps).sqrt()
        attn = self.attention_layer(torch.cat([x, mean.expand(-1, -1, T), std.expand(-1, -1, T)], dim=1))
        alpha = torch.softmax(attn.masked_fill(~mask, float("-inf")), dim=-1)
        mu = (alpha * x).sum(-1)
        sg = ((alpha * x * x).sum(-1) - mu * mu).clamp(min=self.eps).sqrt()
        return torch.cat([mu, sg], dim=1).unsqueeze(-1)


class SpeakerDecoder(NeuralModule):
    """Pooling → embedding layers → (angular) classifier; returns ``(logits, embeddings)`` (``conv_asr.py:675-790``)."""

    def __init__(self, feat_in: int, num_classes: int, emb_sizes=256, pool_mode: str = "xvector", angular: bool = False,
                 attention_channels: int = 128, init_mode: str = "xavier_uniform"):
        super().__init__()
        self.angular = angular
        self.emb_id = 2
        emb_sizes = [emb_sizes] if isinstance(emb_sizes, int) else list(emb_sizes)
        self._num_classes = num_classes
        if pool_mode in ("xvector", "tap"):
            self._pooling = StatsPoolLayer(feat_in, pool_mode)
            affine = "batch"
        else:
            self._pooling = AttentivePoolLayer(feat_in, attention_channels)
            affine = "layer"
        self._feat_in = self._pooling.feat_in
        shapes = [self._feat_in] + emb_sizes
        self.emb_layers = nn.ModuleList([self._affine(i, o, affine) for i, o in zip(shapes[:-1], shapes[1:])])
        self.final = nn.Linear(shapes[-1], num_classes, bias=not angular)
        self.apply(lambda m: init_weights(m, init_mode))

    @staticmethod
    def _affine(inp, out, kind):
        if kind == "layer":
            return nn.Sequential(nn.BatchNorm1d(inp, affine=True, track_running_stats=True), nn.Conv1d(inp, out, 1))
        return nn.Sequential(nn.Linear(inp, out), nn.BatchNorm1d(out, affine=True, track_running_stats=True), nn.ReLU())

    @property
    def num_classes(self):
        return self._num_classes

    def forward(self, encoder_output, length=None):
        pool = self._pooling(encoder_output, length)
        embs = []
        for layer in self.emb_layers:
            if isinstance(layer[0], nn.Linear):
                pool = pool.squeeze(-1) if pool.dim() == 3 else pool
                emb = layer[0](pool)
                pool = layer[2](layer[1](emb))
            else:
                pool = pool if pool.dim() == 3 else pool.unsqueeze(-1)
                pool = layer(pool)
                emb = pool
            embs.append(emb)
        pool = pool.squeeze(-1) if pool.dim() == 3 else pool
        if self.angular:
            w = F.normalize(self.final.weight, p=2, dim=1)
            out = F.linear(F.normalize(pool, p=2, dim=1), w)
        else:
            out = self.final(pool)
        e = embs[-1]
        return out, (e.squeeze(-1) if e.dim() == 3 else e)


class SEModule(nn.Module):
    def __init__(self, inp_filters, se_filters, out_filters, kernel_size=1, dilation=1):
        super().__init__()
        self.se_layer = nn.Sequential(nn.Conv1d(inp_filters, se_filters, kernel_size, dilation=dilation), nn.ReLU(),
                                      nn.BatchNorm1d(se_filters), nn.Conv1d(se_filters, out_filters, kernel_size, dilation=dilation),
                                      nn.Sigmoid())

    def forward(self, x, length=None):
        if length is None:
            s = x.mean(dim=2, keepdim=True)
        else:
            mask = (torch.arange(x.shape[-1], device=x.device)[None] < length[:, None]).unsqueeze(1).to(x.dtype)
            s = (x * mask).sum(2, keepdim=True) / length.clamp(min=1).view(-1, 1, 1).to(x.dtype)
        return self.se_layer(s) * x


class TDNNSEModule(nn.Module):
    """Res2Net-style TDNN block with squeeze-excite (ECAPA building block)."""

    def __init__(self, inp_filters, out_filters, group_scale=8, se_channels=128, kernel_size=1, dilation=1):
        super().__init__()
        self.out_filters = out_filters
        self.tdnn1 = TDNNModule(inp_filters, out_filters, 1)
        self.scale = group_scale
        w = out_filters // group_scale
        self.res2 = nn.ModuleList([TDNNModule(w, w, kernel_size, dilation) for _ in range(group_scale - 1)])
        self.tdnn2 = TDNNModule(out_filters, out_filters, 1)
        self.se_layer = SEModule(out_filters, se_channels, out_filters)

    def forward(self, x, length=None):
        y = self.tdnn1(x)
        chunks = torch.chunk(y, self.scale, dim=1)
        outs = [chunks[0]]
        prev = None
        for i, blk in enumerate(self.res2):
            inp = chunks[i + 1] if prev is None else chunks[i + 1] + prev
            prev = blk(inp)
            outs.append(prev)
        y = self.tdnn2(torch.cat(outs, dim=1))
        return self.se_layer(y, length) + x


class ECAPAEncoder(NeuralModule):
    """ECAPA-TDNN encoder (``conv_asr.py:793-880``)."""

    def __init__(self, feat_in: int, filters: Sequence[int], kernel_sizes: Sequence[int], dilations: Sequence[int],
                 scale: int = 8, init_mode: str = "xavier_uniform"):
        super().__init__()
        self.layers = nn.ModuleList([TDNNModule(feat_in, filters[0], kernel_sizes[0], dilations[0])])
        for i in range(len(filters) - 2):
            self.layers.append(TDNNSEModule(filters[i], filters[i + 1], group_scale=scale, se_channels=128,
                                            kernel_size=kernel_sizes[i + 1], dilation=dilations[i + 1]))
        self.feature_agg = TDNNModule(filters[-1], filters[-1], kernel_sizes[-1], dilations[-1])
        self._feat_out = filters[-1]
        self.apply(lambda m: init_weights(m, init_mode))

    def forward(self, audio_signal, length=None):
        x = audio_signal
        outs = []
        for layer in self.layers:
            x = layer(x, length=length)
            outs.append(x)
        x = torch.cat(outs[1:], dim=1)
        return self.feature_agg(x), length


class ConvASRDecoderReconstruction(NeuralModule):
    """Transposed-conv decoder reconstructing spectrogram frames from encoder states (SSL, ``conv_asr.py:473-583``)."""

    def __init__(self, feat_in: int, feat_out: int, feat_hidden: int = 128, stride_layers: int = 2, non_stride_layers: int = 0,
                 kernel_size: int = 11, init_mode: str = "xavier_uniform", activation: str = "relu", stride_transpose: bool = True,
                 apply_softmax: bool = False):
        super().__init__()
        if stride_layers > 0 and (kernel_size < 3 or kernel_size % 2 == 0):
            raise ValueError("Kernel size in this decoder needs to be >= 3 and odd when using strided layers.")
        act = jasper_activations[activation]()
        self.feat_in, self.feat_out, self.apply_softmax = feat_in, feat_out, apply_softmax
        layers: List[nn.Module] = [nn.Conv1d(feat_in, feat_hidden, 1, bias=True)]
        for _ in range(stride_layers):
            layers += [act, nn.ConvTranspose1d(feat_hidden, feat_hidden, kernel_size, stride=2, padding=(kernel_size - 3) // 2 + 1,
                                              output_padding=1, bias=True, groups=feat_hidden) if stride_transpose else
                       nn.Conv1d(feat_hidden, feat_hidden, kernel_size, stride=2, padding=(kernel_size - 1) // 2, bias=True,
                                 groups=feat_hidden),
                       nn.Conv1d(feat_hidden, feat_hidden, 1, bias=True), nn.BatchNorm1d(feat_hidden, eps=1e-3, momentum=0.1)]
        for _ in range(non_stride_layers):
            layers += [act, nn.Conv1d(feat_hidden, feat_hidden, kernel_size, bias=True, groups=feat_hidden, padding=kernel_size // 2),
                       nn.Conv1d(feat_hidden, feat_hidden, 1, bias=True), nn.BatchNorm1d(feat_hidden, eps=1e-3, momentum=0.1)]
        layers += [act, nn.Conv1d(feat_hidden, feat_out, 1, bias=True)]
        self.decoder_layers = nn.Sequential(*layers)
        self.apply(lambda m: init_weights(m, init_mode))

    def forward(self, encoder_output):
        out = self.decoder_layers(encoder_output).transpose(-2, -1)
        return torch.log_softmax(out, dim=-1) if self.apply_softmax else out

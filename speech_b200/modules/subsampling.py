"""Convolutional sub-sampling front of the encoder.

``ConvSubsampling`` with ``subsampling='dw_striding'`` is the FastConformer 8x front: Conv2d(1->C,3,s2)
+ReLU, then twice [depthwise Conv2d(C,3,s2) + pointwise Conv2d(C,1) + ReLU], flatten C*F/8, Linear to
d_model; time positions beyond each utterance's length are zeroed before every layer
(reference: ``nemo/collections/asr/parts/submodules/subsampling.py:184-257,427-478,697-731``).
Layer indices inside ``conv`` (0,2,3,5,6) and the ``out`` Linear keep the reference's names.  The
causal variant pads (k-1, s-1) (reference: ``causal_convs.py:24-70``).  ``striding`` (full
convolutions), ``stacking`` and 1-D variants are provided as well.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops


def calc_length(lengths, all_paddings: int, kernel_size: int, stride: int, ceil_mode: bool, repeat_num: int = 1):
    add_pad = float(all_paddings - kernel_size)
    lengths = lengths.to(torch.float)
    for _ in range(repeat_num):
        lengths = lengths.add(add_pad).div(stride).add(1.0)
        lengths = torch.ceil(lengths) if ceil_mode else torch.floor(lengths)
    return lengths.to(torch.int)


class CausalConv2D(nn.Conv2d):
    """Conv2d whose padding is (k-1) on the left / top and (s-1) on the right / bottom."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=None, dilation=1, groups=1, bias=True):
        if padding is not None:
            raise ValueError("Argument padding should be set to None for CausalConv2D.")
        self._left_padding = kernel_size - 1
        self._right_padding = stride - 1
        super().__init__(in_channels, out_channels, kernel_size, stride, 0, dilation, groups, bias)

    def forward(self, x):
        x = F.pad(x, pad=(self._left_padding, self._right_padding, self._left_padding, self._right_padding))
        return super().forward(x)


def _time_mask(x, lengths):
    B, _, T, _ = x.shape
    m = torch.arange(T, device=x.device)[None, :] < lengths[:, None]
    return x * m[:, None, :, None].to(x.dtype)


class MaskedConvSequential(nn.Sequential):
    def forward(self, x, lengths):
        x = x.unsqueeze(1)
        cur = lengths.clone().long()
        for layer in self:
            x = _time_mask(x, cur)
            x = layer(x)
            if hasattr(layer, "stride") and tuple(layer.stride) != (1, 1):
                if hasattr(layer, "_left_padding"):
                    pl, pr = layer._left_padding, layer._right_padding
                else:
                    pl, pr = layer.padding[0], layer.padding[0]
                cur = torch.div(cur + pl + pr - layer.kernel_size[0], layer.stride[0], rounding_mode="floor") + 1
        x = _time_mask(x, cur)
        return x, cur


class ConvSubsampling(nn.Module):
    def __init__(self, subsampling: str, subsampling_factor: int, feat_in: int, feat_out: int, conv_channels: int,
                 subsampling_conv_chunking_factor: int = 1, activation=None, is_causal: bool = False):
        super().__init__()
        activation = activation if activation is not None else nn.ReLU()
        self._subsampling = subsampling
        self._conv_channels = conv_channels
        self._feat_in, self._feat_out = feat_in, feat_out
        if subsampling_factor % 2 != 0:
            raise ValueError("Sampling factor should be a multiply of 2!")
        self._sampling_num = int(math.log(subsampling_factor, 2))
        self.subsampling_factor = subsampling_factor
        self.is_causal = is_causal
        self.subsampling_conv_chunking_factor = subsampling_conv_chunking_factor
        layers: List[nn.Module] = []
        in_channels = 1
        if subsampling in ("dw_striding", "striding"):
            self._stride, self._kernel_size, self._ceil_mode = 2, 3, False
            if is_causal:
                self._left_padding, self._right_padding = self._kernel_size - 1, self._stride - 1
                self._max_cache_len = subsampling_factor + 1
            else:
                self._left_padding = self._right_padding = (self._kernel_size - 1) // 2
                self._max_cache_len = 0
            mk = (lambda i, o, g: CausalConv2D(i, o, self._kernel_size, self._stride, None, groups=g)) if is_causal else \
                (lambda i, o, g: nn.Conv2d(i, o, self._kernel_size, self._stride, self._left_padding, groups=g))
            if subsampling == "dw_striding":
                layers += [mk(in_channels, conv_channels, 1), activation]
                in_channels = conv_channels
                for _ in range(self._sampling_num - 1):
                    layers += [mk(in_channels, in_channels, in_channels), nn.Conv2d(in_channels, conv_channels, 1),
                               activation]
                    in_channels = conv_channels
            else:
                for _ in range(self._sampling_num):
                    layers += [mk(in_channels, conv_channels, 1), activation]
                    in_channels = conv_channels
            out_len = calc_length(torch.tensor(float(feat_in)), self._left_padding + self._right_padding,
                                  self._kernel_size, self._stride, self._ceil_mode, self._sampling_num)
            self.out = nn.Linear(conv_channels * int(out_len), feat_out)
            self.conv2d_subsampling = True
            self.conv = MaskedConvSequential(*layers)
        elif subsampling in ("striding_conv1d", "dw_striding_conv1d"):
            self._stride, self._ceil_mode = 2, False
            self._kernel_size = 5
            self._left_padding = self._right_padding = (self._kernel_size - 1) // 2
            in_channels = feat_in
            for i in range(self._sampling_num):
                last = i == self._sampling_num - 1
                outc = feat_out if last else conv_channels
                if subsampling == "dw_striding_conv1d":
                    layers += [nn.Conv1d(in_channels, in_channels, self._kernel_size, self._stride, self._left_padding,
                                         groups=in_channels), nn.Conv1d(in_channels, outc, 1), activation]
                else:
                    layers += [nn.Conv1d(in_channels, outc, self._kernel_size, self._stride, self._left_padding), activation]
                in_channels = outc
            self.out = None
            self.conv2d_subsampling = False
            self.conv = nn.Sequential(*layers)
        else:
            raise ValueError(f"Not valid sub-sampling: {subsampling}!")

    def get_sampling_frames(self):
        return [1, self.subsampling_factor]

    def get_streaming_cache_size(self):
        return [0, self.subsampling_factor + 1]

    def forward(self, x, lengths):
        """x: [B, T, F] features; returns ([B, T', d_model], lengths').

        ``subsampling_conv_chunking_factor``: -1 never splits; 1 splits only when the widest activation of the stack
        (``B x conv_channels x T/2 x F/2``) would pass 2**31 elements, the limit of 32-bit indexing in convolution kernels;
        ``n > 1`` always splits into pieces of at most ``1/n`` of that activation (the reference has the same switch,
        ``subsampling.py:427-466``, and splits by batch, then by channel).  Here pieces are taken along the batch first and,
        for single long recordings, along time: chunks start on a multiple of the subsampling factor and carry one output
        frame of context on either side, which makes the chunked result equal to the unsplit one, masks included."""
        f = self.subsampling_conv_chunking_factor
        if self.conv2d_subsampling and f != -1 and x.dim() == 3:
            B, T, F_ = x.shape
            widest = self._conv_channels * ((T + 1) // 2) * ((F_ + 1) // 2)          # per batch element, after the first layer
            budget = 2 ** 31 if f == 1 else max(1, (B * widest) // f)
            if B * widest > budget:
                return self._forward_chunked(x, lengths, widest, budget)
        return self._forward_once(x, lengths)

    def _forward_chunked(self, x, lengths, widest: int, budget: int):
        B, T, _ = x.shape
        sf = self.subsampling_factor
        if widest <= budget or self.is_causal or self._subsampling not in ("dw_striding", "striding"):
            # whole recordings fit (or time splitting is not exact for this variant): groups of batch elements
            per = max(1, budget // max(1, widest))
            outs, lens = [], []
            for b0 in range(0, B, per):
                y, l = self._forward_once(x[b0:b0 + per], lengths[b0:b0 + per])
                outs.append(y)
                lens.append(l)
            return torch.cat(outs, dim=0), torch.cat(lens, dim=0)
        # one recording is too long: time chunks of `step` input frames (a multiple of the subsampling factor) with a halo of
        # one output frame (sf input frames) on both sides; the halo's outputs are dropped
        frames_budget = max(4 * sf, int(T * budget / widest))
        step = max(sf, (frames_budget - 2 * sf) // sf * sf)
        outs, out_len = [], None
        for b in range(B):
            pieces = []
            for t0 in range(0, T, step):
                lo, hi = max(0, t0 - sf), min(T, t0 + step + sf)
                y, _ = self._forward_once(x[b:b + 1, lo:hi], (lengths[b:b + 1] - lo).clamp(min=0, max=hi - lo))
                drop = (t0 - lo) // sf
                keep = -(-min(step, T - t0) // sf) if t0 + step < T else y.shape[1] - drop
                pieces.append(y[:, drop:drop + keep])
            outs.append(torch.cat(pieces, dim=1))
        n = max(o.shape[1] for o in outs)
        out = torch.cat([torch.nn.functional.pad(o, (0, 0, 0, n - o.shape[1])) for o in outs], dim=0)
        out_len = calc_length(lengths, self._left_padding + self._right_padding, self._kernel_size, self._stride, self._ceil_mode,
                              self._sampling_num)
        return out, out_len.to(lengths.dtype) if torch.is_tensor(out_len) else out_len

    def _forward_once(self, x, lengths):
        if self._native_front_end(x):
            from ..ops import native_subsampling as ns

            convs = [m for m in self.conv if isinstance(m, nn.Conv2d)]
            return ns.dw_striding_forward(x, lengths, convs, self.out.weight, self.out.bias, self.is_causal)
        if self.conv2d_subsampling:
            x, out_lengths = self.conv(x, lengths)
            b, c, t, f = x.shape
            x = x.transpose(1, 2).reshape(b, t, c * f)
            x = ops.linear(x, self.out.weight, self.out.bias)
        else:
            out_lengths = calc_length(lengths, self._left_padding + self._right_padding, self._kernel_size, self._stride,
                                      self._ceil_mode, self._sampling_num)
            x = self.conv(x.transpose(1, 2)).transpose(1, 2)
        return x, out_lengths

    def _native_front_end(self, x) -> bool:
        """The channels-last kernels of ``ops/csrc/subsampling.cu`` serve the depthwise-striding front end in bf16 on GPUs."""
        if not (self.conv2d_subsampling and self._subsampling == "dw_striding" and x.is_cuda and x.dim() == 3):
            return False
        if ops.get_compute_dtype() != torch.bfloat16 or not ops._use_native(x):
            return False
        from ..ops import native_subsampling as ns

        return ns.supported(self._conv_channels, self._sampling_num, self._feat_in) and self._feat_out % 8 == 0

    def prime_shapes(self, shapes, device, dtype=None) -> None:
        """Run the convolution stack forward and backward once on zeros for every ``(batch, frames)`` in ``shapes``.  The
        convolution library builds an execution plan per problem shape on first use (milliseconds each, three per layer with the
        backward passes); with bucketed batches the shapes are known before training starts, so the plans can be built then
        instead of inside the first step that meets a shape.  Parameter gradients produced here are discarded."""
        if not self.conv2d_subsampling:
            return
        if dtype == torch.bfloat16 and torch.device(device).type == "cuda" and self._subsampling == "dw_striding" and ops.native_available():
            return  # the native front end has no per-shape plans
        import contextlib

        ctx = torch.autocast("cuda", dtype=dtype) if (dtype is not None and torch.device(device).type == "cuda") else contextlib.nullcontext()
        was = self.training
        self.train()
        for b, t in shapes:
            x = torch.zeros(int(b), int(t), self._feat_in, device=device, requires_grad=True)
            with ctx:
                y, _ = self.conv(x, torch.full((int(b),), int(t), device=device, dtype=torch.long))
            y.float().sum().backward()
        for p in self.parameters():
            p.grad = None
        self.train(was)

    def reset_parameters(self):
        if self._subsampling != "dw_striding":
            return
        with torch.no_grad():
            scale = 1.0 / self._kernel_size
            dw_max = (self._kernel_size ** 2) ** -0.5
            pw_max = self._conv_channels ** -0.5
            nn.init.uniform_(self.conv[0].weight, -scale, scale)
            nn.init.uniform_(self.conv[0].bias, -scale, scale)
            for idx in range(2, len(self.conv), 3):
                nn.init.uniform_(self.conv[idx].weight, -dw_max, dw_max)
                nn.init.uniform_(self.conv[idx].bias, -dw_max, dw_max)
                nn.init.uniform_(self.conv[idx + 1].weight, -pw_max, pw_max)
                nn.init.uniform_(self.conv[idx + 1].bias, -pw_max, pw_max)
            fc_scale = (self._feat_out * self._feat_in / self.subsampling_factor) ** -0.5
            nn.init.uniform_(self.out.weight, -fc_scale, fc_scale)
            nn.init.uniform_(self.out.bias, -fc_scale, fc_scale)


class StackingSubsampling(nn.Module):
    """Stack ``factor`` consecutive frames and project (``subsampling='stacking'`` / ``'stacking_norm'``)."""

    def __init__(self, subsampling_factor: int, feat_in: int, feat_out: int, norm: bool = False):
        super().__init__()
        self.subsampling_factor = subsampling_factor
        self.proj_out = nn.Linear(subsampling_factor * feat_in, feat_out)
        self.pre_norm = nn.LayerNorm(feat_in) if norm else None

    def get_sampling_frames(self):
        return self.subsampling_factor

    def get_streaming_cache_size(self):
        return 0

    def forward(self, x, lengths):
        b, t, h = x.shape
        if self.pre_norm is not None:
            x = self.pre_norm(x)
        pad = (self.subsampling_factor - t % self.subsampling_factor) % self.subsampling_factor
        x = F.pad(x, (0, 0, 0, pad))
        x = x.reshape(b, (t + pad) // self.subsampling_factor, h * self.subsampling_factor)
        x = self.proj_out(x)
        lengths = torch.div(lengths + pad, self.subsampling_factor, rounding_mode="floor")
        return x, lengths


class SubsamplingReductionModule(nn.Module):
    """Mid-encoder time reduction by pooling or strided convolution (reference ``subsampling.py:631``)."""

    def __init__(self, reduction: str, d_model: int, reduction_factor: int = 2):
        super().__init__()
        assert reduction in ("pooling", "striding")
        self.reduction, self.d_model, self._sampling_num = reduction, d_model, int(math.log(reduction_factor, 2))
        if reduction == "pooling":
            self.reduction_enc = nn.MaxPool1d(kernel_size=reduction_factor)
            self.padding, self.kernel_size, self.stride = 0, reduction_factor, reduction_factor
        else:
            self.kernel_size, self.stride, self.padding = 3, 2, 1
            self.reduction_enc = ConvSubsampling("striding_conv1d", reduction_factor, d_model, d_model, d_model)

    def forward(self, x, lengths):
        if self.reduction == "striding":
            return self.reduction_enc(x, lengths)
        x = self.reduction_enc(x.transpose(1, 2)).transpose(1, 2)
        lengths = calc_length(lengths, self.padding, self.kernel_size, self.stride, False, 1)
        return x, lengths

"""Conformer / FastConformer encoder with offline and cache-aware streaming modes.

Constructor arguments, attention-context styles (``regular``, ``chunked_limited``,
``chunked_limited_with_rc``), streaming geometry and cache layout follow
``nemo/collections/asr/modules/conformer_encoder.py:64-1554``:

* masks are built on the fly from lengths and ``att_context_size`` (``:841-922``),
* multi-lookahead training samples one ``att_context_size`` per step (``:663-666``),
* ``setup_streaming_params`` derives chunk / shift / cache sizes (``:1004-1112``),
* ``get_initial_cache_state`` returns ``cache_last_channel [L,B,cache,d]``, ``cache_last_time [L,B,d,k-1]``,
  ``cache_last_channel_len [B]`` (``:1114-1152``),
* stochastic depth keeps dropped layers in the graph (``:744-755``), inter-CTC capture (``:771-783``),
* the positional table is extended on demand; under data parallelism the maximum length is agreed
  across ranks with one MAX all-reduce (``:808-826``).
"""
from __future__ import annotations

import math
import random
from dataclasses import dataclass
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..core.module import AccessMixin, NeuralModule
from ..core.neural_types import (AcousticEncodedRepresentation, ChannelType, LengthsType, NeuralType, SpectrogramType,
                                 typecheck)
from .attention import (LocalAttRelPositionalEncoding, MultiHeadAttention, PositionalEncoding, RelPositionalEncoding)
from .conformer_modules import CausalConv1D, ConformerLayer
from .subsampling import ConvSubsampling, StackingSubsampling, SubsamplingReductionModule


@dataclass
class CacheAwareStreamingConfig:
    chunk_size: Union[int, List[int]] = 0
    shift_size: Union[int, List[int]] = 0
    cache_drop_size: int = 0
    last_channel_cache_size: int = 0
    valid_out_len: int = 0
    pre_encode_cache_size: Union[int, List[int]] = 0
    drop_extra_pre_encoded: int = 0
    last_channel_num: int = 0
    last_time_num: int = 0


def compute_stochastic_depth_drop_probs(num_layers, drop_prob=0.0, mode="linear", start_layer=1):
    """Per-layer drop probabilities; the first ``start_layer`` layers are never dropped
    (reference: ``parts/utils/regularization_utils.py:25-64``)."""
    if not 0 <= drop_prob < 1.0:
        raise ValueError("stochastic_depth_drop_prob has to be in [0, 1).")
    if not 1 <= start_layer <= num_layers:
        raise ValueError("stochastic_depth_start_layer has to be in [1, num layers].")
    probs = [0.0] * start_layer
    if (L := num_layers - start_layer) > 0:
        if mode == "linear":
            probs += [l / L * drop_prob for l in range(1, L + 1)]
        elif mode == "uniform":
            probs += [drop_prob] * L
        else:
            raise ValueError(f'stochastic_depth_mode has to be one of ["linear", "uniform"]. Current value: {mode}')
    return probs


class ConformerEncoder(NeuralModule, AccessMixin):
    def __init__(self, feat_in, n_layers, d_model, feat_out=-1, causal_downsampling=False, subsampling="striding",
                 subsampling_factor=4, subsampling_conv_chunking_factor=1, subsampling_conv_channels=-1,
                 reduction=None, reduction_position=None, reduction_factor=1, ff_expansion_factor=4,
                 self_attention_model="rel_pos", n_heads=4, att_context_size=None, att_context_probs=None,
                 att_context_style="regular", xscaling=True, untie_biases=True, pos_emb_max_len=5000,
                 conv_kernel_size=31, conv_norm_type="batch_norm", conv_context_size=None, use_bias=True, dropout=0.1,
                 dropout_pre_encoder=0.1, dropout_emb=0.1, dropout_att=0.0, stochastic_depth_drop_prob: float = 0.0,
                 stochastic_depth_mode: str = "linear", stochastic_depth_start_layer: int = 1,
                 global_tokens: int = 0, global_tokens_spacing: int = 1, global_attn_separate: bool = False,
                 use_pytorch_sdpa: bool = False, use_pytorch_sdpa_backends=None, sync_max_audio_length: bool = True):
        super().__init__()
        d_ff = d_model * ff_expansion_factor
        self.d_model, self.n_layers, self._feat_in = d_model, n_layers, feat_in
        self.att_context_style = att_context_style
        self.subsampling_factor = subsampling_factor
        self.subsampling_conv_chunking_factor = subsampling_conv_chunking_factor
        self.self_attention_model = self_attention_model
        self.global_tokens, self.global_attn_separate, self.global_tokens_spacing = (
            global_tokens, global_attn_separate, global_tokens_spacing)
        self.sync_max_audio_length = sync_max_audio_length
        (self.att_context_size_all, self.att_context_size, self.att_context_probs,
         self.conv_context_size) = self._calc_context_sizes(att_context_style, att_context_size, att_context_probs,
                                                            conv_context_size, conv_kernel_size)
        self.xscale = math.sqrt(d_model) if xscaling else None
        if subsampling_conv_channels == -1:
            subsampling_conv_channels = d_model
        if subsampling and subsampling_factor > 1:
            if subsampling in ("stacking", "stacking_norm"):
                self.pre_encode = StackingSubsampling(subsampling_factor, feat_in, d_model, norm=subsampling == "stacking_norm")
            else:
                self.pre_encode = ConvSubsampling(subsampling, subsampling_factor, feat_in, d_model,
                                                  subsampling_conv_channels, subsampling_conv_chunking_factor,
                                                  nn.ReLU(True), is_causal=causal_downsampling)
        else:
            self.pre_encode = nn.Linear(feat_in, d_model)
        if reduction and reduction_factor > 1:
            assert reduction_position >= -1 and reduction_position < n_layers
            self.reduction_subsampling = SubsamplingReductionModule(reduction, d_model, reduction_factor)
            self.reduction_position = reduction_position
        else:
            self.reduction_subsampling, self.reduction_position = None, None
        self._feat_out = d_model
        if not untie_biases and self_attention_model == "rel_pos":
            d_head = d_model // n_heads
            pos_bias_u = nn.Parameter(torch.zeros(n_heads, d_head))
            pos_bias_v = nn.Parameter(torch.zeros(n_heads, d_head))
        else:
            pos_bias_u = pos_bias_v = None
        self.pos_emb_max_len = pos_emb_max_len
        if self_attention_model == "rel_pos":
            self.pos_enc = RelPositionalEncoding(d_model=d_model, dropout_rate=dropout_pre_encoder, max_len=pos_emb_max_len,
                                                 xscale=self.xscale, dropout_rate_emb=dropout_emb)
        elif self_attention_model == "rel_pos_local_attn":
            if max(self.att_context_size) <= 0:
                raise ValueError("When using local attention, context size must be set > 0")
            self.pos_enc = LocalAttRelPositionalEncoding(att_context_size=self.att_context_size, d_model=d_model,
                                                         dropout_rate=dropout, max_len=pos_emb_max_len,
                                                         xscale=self.xscale, dropout_rate_emb=dropout_emb)
        elif self_attention_model == "abs_pos":
            self.pos_enc = PositionalEncoding(d_model=d_model, dropout_rate=dropout_pre_encoder, max_len=pos_emb_max_len,
                                              xscale=self.xscale)
        else:
            raise ValueError(f"Not valid self_attention_model: '{self_attention_model}'!")
        self.layers = nn.ModuleList([
            ConformerLayer(d_model=d_model, d_ff=d_ff, self_attention_model=self_attention_model,
                           global_tokens=global_tokens, global_tokens_spacing=global_tokens_spacing,
                           global_attn_separate=global_attn_separate, n_heads=n_heads,
                           conv_kernel_size=conv_kernel_size, conv_norm_type=conv_norm_type,
                           conv_context_size=self.conv_context_size, dropout=dropout, dropout_att=dropout_att,
                           pos_bias_u=pos_bias_u, pos_bias_v=pos_bias_v, att_context_size=self.att_context_size,
                           use_bias=use_bias) for _ in range(n_layers)])
        if feat_out > 0 and feat_out != self._feat_out:
            self.out_proj = nn.Linear(self._feat_out, feat_out)
            self._feat_out = feat_out
        else:
            self.out_proj = None
            self._feat_out = d_model
        self.set_max_audio_length(self.pos_emb_max_len)
        self.use_pad_mask = True
        self.setup_streaming_params()
        self.export_cache_support = False
        self.layer_drop_probs = compute_stochastic_depth_drop_probs(len(self.layers), stochastic_depth_drop_prob,
                                                                    stochastic_depth_mode, stochastic_depth_start_layer)
        self.interctc_capture_at_layers = None

    # ------------------------------------------------------------------ types
    @property
    def input_types(self):
        return {"audio_signal": NeuralType(("B", "D", "T"), SpectrogramType()),
                "length": NeuralType(("B",), LengthsType()),
                "cache_last_channel": NeuralType(("D", "B", "T", "D"), ChannelType(), optional=True),
                "cache_last_time": NeuralType(("D", "B", "D", "T"), ChannelType(), optional=True),
                "cache_last_channel_len": NeuralType(("B",), LengthsType(), optional=True),
                "bypass_pre_encode": NeuralType(("Any",), optional=True)}

    @property
    def output_types(self):
        return {"outputs": NeuralType(("B", "D", "T"), AcousticEncodedRepresentation()),
                "encoded_lengths": NeuralType(("B",), LengthsType())}

    # ------------------------------------------------------------------ context sizes
    def _calc_context_sizes(self, att_context_style, att_context_size, att_context_probs, conv_context_size,
                            conv_kernel_size):
        if att_context_size:
            att_context_size_all = [list(a) for a in att_context_size] if isinstance(att_context_size[0], (list, tuple)) or \
                hasattr(att_context_size[0], "__iter__") else [list(att_context_size)]
            for acs in att_context_size_all:
                if att_context_style == "chunked_limited":
                    if acs[0] > 0 and acs[0] % (acs[1] + 1) > 0:
                        raise ValueError(f"att_context_size[0] % (att_context_size[1] + 1) should be zero: {acs}")
                    if acs[1] < 0 and len(att_context_size_all) <= 1:
                        raise ValueError(f"Right context (att_context_size[1]) can not be unlimited for chunked_limited style: {acs}")
        else:
            att_context_size_all = [[-1, -1]] if att_context_style != "chunked_limited_with_rc" else [[-1, -1, -1]]
        if att_context_probs:
            if len(att_context_probs) != len(att_context_size_all):
                raise ValueError("The size of the att_context_probs should be the same as att_context_size.")
            att_context_probs = list(att_context_probs)
            if abs(sum(att_context_probs) - 1.0) > 1e-6:
                raise ValueError("The sum of numbers in att_context_probs should be equal to one to be a distribution.")
        else:
            att_context_probs = [1.0 / len(att_context_size_all)] * len(att_context_size_all)
        if conv_context_size is not None:
            if isinstance(conv_context_size, str):
                if conv_context_size != "causal":
                    raise ValueError("Invalid conv_context_size! It should be the string 'causal' or a list of two integers.")
                conv_context_size = [conv_kernel_size - 1, 0]
            else:
                conv_context_size = list(conv_context_size)
                if conv_context_size[0] + conv_context_size[1] + 1 != conv_kernel_size:
                    raise ValueError(f"Invalid conv_context_size: {conv_context_size}!")
        else:
            conv_context_size = [(conv_kernel_size - 1) // 2, (conv_kernel_size - 1) // 2]
        return att_context_size_all, att_context_size_all[0], att_context_probs, conv_context_size

    def set_default_att_context_size(self, att_context_size):
        if att_context_size not in self.att_context_size_all:
            pass
        self.att_context_size = list(att_context_size)
        self.setup_streaming_params()

    # ------------------------------------------------------------------ positional table
    def set_max_audio_length(self, max_audio_length):
        self.max_audio_length = max_audio_length
        device = next(self.parameters()).device
        self.pos_enc.extend_pe(max_audio_length, device, torch.float32)

    def update_max_seq_length(self, seq_length: int, device):
        if self.sync_max_audio_length and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([seq_length], dtype=torch.float32, device=device if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seq_length = int(t.item())
        if seq_length > self.max_audio_length:
            self.max_audio_length = seq_length
        self.pos_enc.extend_pe(max(seq_length, self.max_audio_length), device, torch.float32)

    # ------------------------------------------------------------------ masks
    def _create_masks(self, att_context_size, padding_length, max_audio_length, offset, device):
        T = max_audio_length
        if self.self_attention_model != "rel_pos_local_attn":
            att_mask = torch.ones(1, T, T, dtype=torch.bool, device=device)
            if self.att_context_style == "regular":
                if att_context_size[0] >= 0:
                    att_mask = att_mask.triu(diagonal=-att_context_size[0])
                if att_context_size[1] >= 0:
                    att_mask = att_mask.tril(diagonal=att_context_size[1])
            elif self.att_context_style == "chunked_limited":
                if att_context_size[1] == -1:
                    if att_context_size[0] >= 0:
                        att_mask = att_mask.triu(diagonal=-att_context_size[0])
                else:
                    chunk_size = att_context_size[1] + 1
                    left_chunks_num = att_context_size[0] // chunk_size if att_context_size[0] >= 0 else 10000
                    chunk_idx = torch.div(torch.arange(0, T, dtype=torch.int, device=device), chunk_size, rounding_mode="trunc")
                    diff = chunk_idx.unsqueeze(1) - chunk_idx.unsqueeze(0)
                    att_mask = att_mask & ((diff <= left_chunks_num) & (diff >= 0)).unsqueeze(0)
            elif self.att_context_style == "chunked_limited_with_rc" and sum(att_context_size) != -3:
                left, chunk, right = att_context_size
                frame = torch.arange(0, T, dtype=torch.int, device=device)
                cidx = torch.div(frame, chunk, rounding_mode="trunc")
                ws = (cidx * chunk - left).clamp(min=0)
                we = (cidx * chunk + chunk - 1 + right).clamp(max=T - 1)
                att_mask = att_mask & ((frame[None, :] >= ws[:, None]) & (frame[None, :] <= we[:, None])).unsqueeze(0)
        else:
            att_mask = None
        pad_mask = torch.arange(0, T, device=device).expand(padding_length.size(0), -1) < padding_length.unsqueeze(-1)
        if offset is not None:
            pad_mask = pad_mask & (torch.arange(0, T, device=device).expand(padding_length.size(0), -1) >= offset.unsqueeze(-1))
        if att_mask is not None:
            pm = pad_mask.unsqueeze(1).expand(-1, T, -1)
            pm = pm & pm.transpose(1, 2)
            att_mask = ~(pm & att_mask)
        return ~pad_mask, att_mask

    def enable_pad_mask(self, on=True):
        mask = self.use_pad_mask
        self.use_pad_mask = on
        return mask

    # ------------------------------------------------------------------ forward
    def forward_for_export(self, audio_signal, length, cache_last_channel=None, cache_last_time=None,
                           cache_last_channel_len=None):
        if cache_last_channel is not None:
            cache_last_channel = cache_last_channel.transpose(0, 1)
            cache_last_time = cache_last_time.transpose(0, 1)
        rets = self.forward_internal(audio_signal, length, cache_last_channel, cache_last_time, cache_last_channel_len)
        rets = self.streaming_post_process(rets, keep_all_outputs=False)
        if len(rets) == 2:
            return rets
        return rets[0], rets[1], rets[2].transpose(0, 1), rets[3].transpose(0, 1), rets[4]

    def streaming_post_process(self, rets, keep_all_outputs=True):
        if len(rets) == 2:
            return rets[0], rets[1], None, None, None
        encoded, encoded_len, clc, clt, clcl = rets
        if self.streaming_cfg.last_channel_cache_size >= 0 and self.streaming_cfg.last_channel_cache_size > 0:
            clc = clc[:, :, -self.streaming_cfg.last_channel_cache_size:, :]
        if self.streaming_cfg.valid_out_len > 0 and (not keep_all_outputs or self.att_context_style == "regular"):
            encoded = encoded[:, :, : self.streaming_cfg.valid_out_len]
            encoded_len = torch.clamp(encoded_len, max=self.streaming_cfg.valid_out_len)
        return encoded, encoded_len, clc, clt, clcl

    # ------------------------------------------------------------------ adapters (every layer hosts a copy)
    def add_adapter(self, name: str, cfg) -> None:
        for layer in self.layers:
            layer.add_adapter(name, cfg)

    def is_adapter_available(self) -> bool:
        return any(layer.is_adapter_available() for layer in self.layers)

    def set_enabled_adapters(self, name=None, enabled: bool = True) -> None:
        for layer in self.layers:
            if layer.is_adapter_available():
                layer.set_enabled_adapters(name, enabled)

    def get_enabled_adapters(self):
        names = []
        for layer in self.layers:
            for n in layer.get_enabled_adapters():
                if n not in names:
                    names.append(n)
        return names

    def unfreeze_enabled_adapters(self, freeze_batchnorm: bool = True) -> None:
        for layer in self.layers:
            if layer.is_adapter_available():
                layer.unfreeze_enabled_adapters(freeze_batchnorm)

    @property
    def adapter_cfg(self):
        return getattr(self.layers[0], "adapter_cfg", {}) if len(self.layers) else {}

    @typecheck()
    def forward(self, audio_signal, length, cache_last_channel=None, cache_last_time=None, cache_last_channel_len=None,
                bypass_pre_encode=False):
        if not bypass_pre_encode and audio_signal.shape[-2] != self._feat_in:
            raise ValueError(f"If bypass_pre_encode is False, audio_signal should have shape (batch, {self._feat_in}, "
                             f"n_frame) but got last dimension {audio_signal.shape[-2]}.")
        if bypass_pre_encode and audio_signal.shape[-1] != self.d_model:
            raise ValueError(f"If bypass_pre_encode is True, audio_signal should have shape (batch, n_frame, {self.d_model})")
        if bypass_pre_encode:
            self.update_max_seq_length(seq_length=audio_signal.size(1), device=audio_signal.device)
        else:
            self.update_max_seq_length(seq_length=audio_signal.size(2), device=audio_signal.device)
        return self.forward_internal(audio_signal, length, cache_last_channel, cache_last_time, cache_last_channel_len,
                                     bypass_pre_encode)

    def forward_internal(self, audio_signal, length, cache_last_channel=None, cache_last_time=None,
                         cache_last_channel_len=None, bypass_pre_encode=False):
        if length is None:
            length = audio_signal.new_full((audio_signal.size(0),), audio_signal.size(-1), dtype=torch.int64)
        if self.training and len(self.att_context_size_all) > 1:
            cur_att = random.choices(self.att_context_size_all, weights=self.att_context_probs)[0]
        else:
            cur_att = self.att_context_size
        cdt = ops.get_compute_dtype()
        if not bypass_pre_encode:
            audio_signal = audio_signal.transpose(1, 2)
            if cdt is not None and audio_signal.is_cuda and not isinstance(self.pre_encode, nn.Linear):
                pass  # convolutions run under torch.autocast; the projection GEMM receives their bf16 output
            if isinstance(self.pre_encode, nn.Linear):
                audio_signal = ops.linear(audio_signal.to(cdt) if cdt else audio_signal, self.pre_encode.weight,
                                          self.pre_encode.bias)
            else:
                audio_signal, length = self.pre_encode(x=audio_signal, lengths=length)
                length = length.to(torch.int64)
                if self.streaming_cfg.drop_extra_pre_encoded > 0 and cache_last_channel is not None:
                    audio_signal = audio_signal[:, self.streaming_cfg.drop_extra_pre_encoded:, :]
                    length = (length - self.streaming_cfg.drop_extra_pre_encoded).clamp(min=0)
            if self.reduction_position is not None and cache_last_channel is not None:
                raise ValueError("Caching with reduction feature is not supported yet!")
        if cdt is not None and audio_signal.dtype != cdt:
            audio_signal = audio_signal.to(cdt)
        max_audio_length = audio_signal.size(1)
        if cache_last_channel is not None:
            cache_len = self.streaming_cfg.last_channel_cache_size
            cache_keep_size = max_audio_length - self.streaming_cfg.cache_drop_size
            max_audio_length = max_audio_length + cache_len
            padding_length = length + cache_len
            offset = torch.neg(cache_last_channel_len) + cache_len
        else:
            padding_length, cache_len, offset = length, 0, None
        audio_signal, pos_emb = self.pos_enc(x=audio_signal, cache_len=cache_len)
        pad_mask, att_mask = self._create_masks(cur_att, padding_length, max_audio_length, offset, audio_signal.device)
        cache_last_time_next, cache_last_channel_next = [], []
        if cache_last_channel is not None:
            pad_mask = pad_mask[:, cache_len:]
            if att_mask is not None:
                att_mask = att_mask[:, cache_len:]
        if not self.use_pad_mask:
            pad_mask = None
        for lth, (drop_prob, layer) in enumerate(zip(self.layer_drop_probs, self.layers)):
            original_signal = audio_signal
            clc = cache_last_channel[lth] if cache_last_channel is not None else None
            clt = cache_last_time[lth] if cache_last_channel is not None else None
            audio_signal = layer(x=audio_signal, att_mask=att_mask, pos_emb=pos_emb, pad_mask=pad_mask,
                                 cache_last_channel=clc, cache_last_time=clt)
            if clc is not None:
                audio_signal, clc, clt = audio_signal
                cache_last_channel_next.append(clc)
                cache_last_time_next.append(clt)
            if self.training and drop_prob > 0.0:
                if torch.rand(1) < drop_prob:
                    audio_signal = audio_signal * 0.0 + original_signal
                else:
                    audio_signal = (audio_signal - original_signal) / (1.0 - drop_prob) + original_signal
            if self.reduction_position == lth:
                audio_signal, length = self.reduction_subsampling(x=audio_signal, lengths=length)
                max_audio_length = audio_signal.size(1)
                _, pos_emb = self.pos_enc(x=audio_signal, cache_len=cache_len)
                pad_mask, att_mask = self._create_masks(cur_att, length, max_audio_length, offset, audio_signal.device)
            if self.is_access_enabled(getattr(self, "model_guid", None)):
                if self.interctc_capture_at_layers is None:
                    self.interctc_capture_at_layers = self.access_cfg.get("interctc", {}).get("capture_layers", [])
                if lth in self.interctc_capture_at_layers:
                    sig = audio_signal if self.out_proj is None else self.out_proj(audio_signal)
                    self.register_accessible_tensor(name=f"interctc/layer_output_{lth}", tensor=sig.transpose(1, 2))
                    self.register_accessible_tensor(name=f"interctc/layer_length_{lth}", tensor=length)
        if self.out_proj is not None:
            audio_signal = ops.linear(audio_signal, self.out_proj.weight, self.out_proj.bias)
        if self.reduction_position == -1:
            audio_signal, length = self.reduction_subsampling(x=audio_signal, lengths=length)
        audio_signal = audio_signal.transpose(1, 2)
        length = length.to(dtype=torch.int64)
        if cache_last_channel is not None:
            return (audio_signal, length, torch.stack(cache_last_channel_next, dim=0),
                    torch.stack(cache_last_time_next, dim=0),
                    torch.clamp(cache_last_channel_len + cache_keep_size, max=cache_len))
        return audio_signal, length

    # ------------------------------------------------------------------ streaming
    def setup_streaming_params(self, chunk_size: int = None, shift_size: int = None, left_chunks: int = None,
                               att_context_size: list = None, max_context: int = 10000):
        cfg = CacheAwareStreamingConfig()
        if att_context_size is None:
            att_context_size = self.att_context_size
        if chunk_size is not None:
            if chunk_size < 1:
                raise ValueError("chunk_size needs to be a number larger or equal to one.")
            lookahead_steps = chunk_size - 1
            cfg.cache_drop_size = chunk_size - shift_size
        elif self.att_context_style == "chunked_limited":
            lookahead_steps = att_context_size[1]
            cfg.cache_drop_size = 0
        elif self.att_context_style == "chunked_limited_with_rc":
            lookahead_steps = att_context_size[2] * self.n_layers + self.conv_context_size[1] * self.n_layers
            cfg.cache_drop_size = 0
        elif self.att_context_style == "regular":
            lookahead_steps = att_context_size[1] * self.n_layers + self.conv_context_size[1] * self.n_layers
            cfg.cache_drop_size = lookahead_steps
        else:
            cfg.cache_drop_size, lookahead_steps = 0, None
        if chunk_size is None or left_chunks is None:
            cfg.last_channel_cache_size = att_context_size[0] if att_context_size[0] >= 0 else max_context
        else:
            cfg.last_channel_cache_size = left_chunks * chunk_size
        sampling_frames = self.pre_encode.get_sampling_frames() if hasattr(self.pre_encode, "get_sampling_frames") else 0
        sf = self.subsampling_factor
        if isinstance(sampling_frames, list):
            cfg.chunk_size = [sampling_frames[0] + sf * lookahead_steps, sampling_frames[1] + sf * lookahead_steps]
            cfg.shift_size = [sampling_frames[0] + sampling_frames[1] * (lookahead_steps - cfg.cache_drop_size),
                              sampling_frames[1] + sampling_frames[1] * (lookahead_steps - cfg.cache_drop_size)]
            cfg.valid_out_len = (cfg.shift_size[1] - sampling_frames[1]) // sf + 1
        else:
            cfg.chunk_size = sampling_frames * (1 + lookahead_steps)
            cfg.shift_size = sampling_frames * (1 + lookahead_steps - cfg.cache_drop_size)
            cfg.valid_out_len = cfg.shift_size // sf
        cfg.pre_encode_cache_size = self.pre_encode.get_streaming_cache_size() \
            if hasattr(self.pre_encode, "get_streaming_cache_size") else 0
        if isinstance(cfg.pre_encode_cache_size, list):
            cfg.drop_extra_pre_encoded = 1 + (cfg.pre_encode_cache_size[1] - 1) // sf if cfg.pre_encode_cache_size[1] >= 1 else 0
        else:
            cfg.drop_extra_pre_encoded = cfg.pre_encode_cache_size // sf
        for m in self.layers.modules():
            if hasattr(m, "_max_cache_len"):
                if isinstance(m, (MultiHeadAttention, CausalConv1D)):
                    m.cache_drop_size = cfg.cache_drop_size
        self.streaming_cfg = cfg

    def get_initial_cache_state(self, batch_size=1, dtype=torch.float32, device=None, max_dim=0):
        if device is None:
            device = next(self.parameters()).device
        last_time_cache_size = self.conv_context_size[0]
        L = len(self.layers)
        clc = torch.zeros((L, batch_size, self.streaming_cfg.last_channel_cache_size, self.d_model), device=device, dtype=dtype)
        clt = torch.zeros((L, batch_size, self.d_model, last_time_cache_size), device=device, dtype=dtype)
        clcl = torch.zeros(batch_size, device=device, dtype=torch.int64)
        return clc, clt, clcl

    # ------------------------------------------------------------------ streaming step under CUDA graphs
    stream_cuda_graphs = False      # set by the streaming wrappers: replay the whole encoder step from a graph per input signature
    max_stream_graphs = 8

    def cache_aware_stream_step(self, processed_signal, processed_signal_length=None, cache_last_channel=None,
                                cache_last_time=None, cache_last_channel_len=None, keep_all_outputs=True,
                                drop_extra_pre_encoded=None, bypass_pre_encode=False):
        """One chunk through the encoder with caches.  A streaming step is ~1000 small launches whose cost is host time, and its
        shapes repeat from step to step, so on a GPU the step is captured once per signature (batch, frames, drop, dtypes) and
        replayed; inputs are copied into the graph's static buffers and the returned tensors are the graph's static outputs
        (valid until the next step with the same signature: callers store what they keep, as the slot cache manager does)."""
        if (self.stream_cuda_graphs and processed_signal.is_cuda and not self.training and not torch.is_grad_enabled()
                and cache_last_channel is not None and processed_signal_length is not None and not bypass_pre_encode
                and not torch.cuda.is_current_stream_capturing()):
            return self._stream_step_graphed(processed_signal, processed_signal_length, cache_last_channel, cache_last_time,
                                             cache_last_channel_len, keep_all_outputs, drop_extra_pre_encoded)
        return self._stream_step_eager(processed_signal, processed_signal_length, cache_last_channel, cache_last_time,
                                       cache_last_channel_len, keep_all_outputs, drop_extra_pre_encoded, bypass_pre_encode)

    def _stream_step_graphed(self, sig, length, clc, clt, clcl, keep_all_outputs, drop_extra):
        from collections import OrderedDict

        graphs = self.__dict__.setdefault("_stream_graphs", OrderedDict())
        key = (tuple(sig.shape), sig.dtype, tuple(clc.shape), clc.dtype, tuple(clt.shape), bool(keep_all_outputs), drop_extra,
               ops.get_compute_dtype(), torch.is_autocast_enabled())
        e = graphs.get(key)
        if e is None:
            args = [sig.clone(), length.clone(), clc.clone(), clt.clone(), clcl.clone()]
            run = lambda: self._stream_step_eager(args[0], args[1], args[2], args[3], args[4], keep_all_outputs, drop_extra, False)  # noqa: E731
            side = torch.cuda.Stream(device=sig.device)
            side.wait_stream(torch.cuda.current_stream(sig.device))
            with torch.cuda.stream(side):
                for _ in range(2):                      # lazy initialisation (tables, kernel attributes, allocator) outside the capture
                    run()
            torch.cuda.current_stream(sig.device).wait_stream(side)
            torch.cuda.synchronize(sig.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                outs = run()
            e = graphs[key] = {"graph": g, "args": args, "outs": outs}
            while len(graphs) > self.max_stream_graphs:
                graphs.popitem(last=False)
        else:
            graphs.move_to_end(key)
        for dst, src in zip(e["args"], (sig, length, clc, clt, clcl)):
            dst.copy_(src, non_blocking=True)
        e["graph"].replay()
        return e["outs"]

    def _stream_step_eager(self, processed_signal, processed_signal_length=None, cache_last_channel=None,
                           cache_last_time=None, cache_last_channel_len=None, keep_all_outputs=True,
                           drop_extra_pre_encoded=None, bypass_pre_encode=False):
        """One chunk through the encoder with caches, then trim (reference: ``parts/mixins/streaming.py:40-76``)."""
        if self.streaming_cfg is None:
            self.setup_streaming_params()
        prev = None
        if drop_extra_pre_encoded is not None:
            prev = self.streaming_cfg.drop_extra_pre_encoded
            self.streaming_cfg.drop_extra_pre_encoded = drop_extra_pre_encoded
        try:
            out = self(audio_signal=processed_signal, length=processed_signal_length, cache_last_channel=cache_last_channel,
                       cache_last_time=cache_last_time, cache_last_channel_len=cache_last_channel_len,
                       bypass_pre_encode=bypass_pre_encode)
        finally:
            if prev is not None:
                self.streaming_cfg.drop_extra_pre_encoded = prev
        return self.streaming_post_process(out, keep_all_outputs=keep_all_outputs)

    def change_attention_model(self, self_attention_model: str = None, att_context_size=None,
                               update_config: bool = True, device=None):
        """Swap ``rel_pos`` <-> ``rel_pos_local_attn`` after training, keeping all weights (``:1154-1320``)."""
        from .attention import RelPositionMultiHeadAttention, RelPositionMultiHeadAttentionLongformer

        att_context_size = list(att_context_size) if att_context_size else self.att_context_size
        self_attention_model = self_attention_model or self.self_attention_model
        if self_attention_model == "rel_pos_local_attn" and max(att_context_size) <= 0:
            raise ValueError("When using local attention, context size must be set > 0")
        d = self.d_model
        dev = device or next(self.parameters()).device
        if self_attention_model == "rel_pos":
            new_pos = RelPositionalEncoding(d_model=d, dropout_rate=self.pos_enc.dropout.p, max_len=self.pos_emb_max_len,
                                            xscale=self.xscale)
        elif self_attention_model == "rel_pos_local_attn":
            new_pos = LocalAttRelPositionalEncoding(att_context_size=att_context_size, d_model=d,
                                                    dropout_rate=self.pos_enc.dropout.p, max_len=self.pos_emb_max_len,
                                                    xscale=self.xscale)
        elif self_attention_model == "abs_pos":
            new_pos = PositionalEncoding(d_model=d, dropout_rate=self.pos_enc.dropout.p, max_len=self.pos_emb_max_len,
                                         xscale=self.xscale)
        else:
            raise ValueError(f"Not valid self_attention_model: '{self_attention_model}'!")
        self.pos_enc = new_pos.to(dev)
        self.self_attention_model = self_attention_model
        self.att_context_size = att_context_size
        self.set_max_audio_length(self.pos_emb_max_len)
        for layer in self.layers:
            old = layer.self_attn
            if self_attention_model == "rel_pos_local_attn":
                new = RelPositionMultiHeadAttentionLongformer(old.h, d, old.dropout_rate, None, None, att_context_size,
                                                              global_tokens=self.global_tokens,
                                                              global_tokens_spacing=self.global_tokens_spacing)
            elif self_attention_model == "rel_pos":
                new = RelPositionMultiHeadAttention(old.h, d, old.dropout_rate, None, None)
            else:
                new = MultiHeadAttention(old.h, d, old.dropout_rate)
            new.load_state_dict(old.state_dict(), strict=False)
            layer.self_attn = new.to(dev)
            layer.self_attention_model = self_attention_model
        self.setup_streaming_params()

"""Further acoustic encoders / decoders: RNN encoder, LSTM decoder, plain Transformer encoder, wav2vec feature encoder and
Transformer, and the parallel-expert (diarization + ASR) encoder.

Reference: ``asr/modules/rnn_encoder.py:30`` (sub-sampling + stacked projected (bi)LSTM/GRU, LayerNorm, dropout),
``lstm_decoder.py:28`` (LSTM + linear + log-softmax), ``transformer_encoder.py:36-560`` (pre-norm Transformer blocks with a
fused QKV projection, optional per-head QK LayerNorm, ``rel_pos`` / ``abs_pos`` / ``no_pos`` scoring, full or causal
attention), ``wav2vec_modules.py:56-360`` (strided Conv1d feature extractor with group / layer norm, convolutional positional
embedding, layer drop, ``GradMultiply``), ``parallel_expert_encoder.py:286-560`` (Sortformer speaker activities projected by
a fixed sinusoidal kernel and added to the normalised ASR encoder states).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core.module import NeuralModule
from .attention import PositionalEncoding, RelPositionalEncoding
from .subsampling import ConvSubsampling, StackingSubsampling


def _pre_encoder(subsampling: Optional[str], factor: int, feat_in: int, feat_out: int, conv_channels: int):
    if subsampling and factor > 1:
        if subsampling in ("stacking", "stacking_norm", "feature_stacking"):
            return StackingSubsampling(factor, feat_in, feat_out, norm="norm" in subsampling)
        return ConvSubsampling(subsampling, factor, feat_in, feat_out, conv_channels if conv_channels > 0 else feat_out, activation=nn.ReLU())
    return nn.Linear(feat_in, feat_out)


# ---------------------------------------------------------------------------------------------- RNN encoder / LSTM decoder
class RNNEncoder(NeuralModule):
    def __init__(self, feat_in: int, n_layers: int, d_model: int, proj_size: int = -1, rnn_type: str = "lstm", bidirectional: bool = True,
                 subsampling: str = "striding", subsampling_factor: int = 4, subsampling_conv_channels: int = -1, dropout: float = 0.2):
        super().__init__()
        kinds = {"lstm": nn.LSTM, "gru": nn.GRU, "rnn": nn.RNN}
        if rnn_type not in kinds:
            raise ValueError(f"rnn_type can be one from the following:{list(kinds)}")
        proj_size = proj_size if proj_size > 0 else d_model
        self.d_model, self._feat_in, self._feat_out = d_model, feat_in, proj_size
        self.pre_encode = _pre_encoder(subsampling, subsampling_factor, feat_in, proj_size, subsampling_conv_channels)
        self.subsampling_factor = subsampling_factor if subsampling else 1
        self.layers = nn.ModuleList()
        for _ in range(n_layers):
            per_dir = proj_size // 2 if bidirectional else proj_size
            if rnn_type == "lstm":
                rnn = nn.LSTM(proj_size, d_model, 1, batch_first=True, bidirectional=bidirectional, proj_size=per_dir if per_dir < d_model else 0)
                out = (per_dir if per_dir < d_model else d_model) * (2 if bidirectional else 1)
            else:
                rnn = kinds[rnn_type](proj_size, per_dir, 1, batch_first=True, bidirectional=bidirectional)
                out = per_dir * (2 if bidirectional else 1)
            self.layers.append(nn.ModuleDict({"rnn": rnn, "proj": nn.Identity() if out == proj_size else nn.Linear(out, proj_size),
                                              "norm": nn.LayerNorm(proj_size), "drop": nn.Dropout(dropout)}))

    def forward(self, audio_signal, length=None):
        x = audio_signal.transpose(1, 2)
        if length is None:
            length = torch.full((x.shape[0],), x.shape[1], dtype=torch.long, device=x.device)
        if isinstance(self.pre_encode, nn.Linear):
            x = self.pre_encode(x)
        else:
            x, length = self.pre_encode(x, length)
        x = x.float()
        for l in self.layers:
            y, _ = l["rnn"](x)
            x = l["drop"](l["norm"](l["proj"](y)))
        return x.transpose(1, 2), length


class LSTMDecoder(NeuralModule):
    """Frame classifier: (bi)LSTM over encoder states, linear layer, log-softmax (``vocabulary`` + blank)."""

    def __init__(self, feat_in: int, num_classes: int, lstm_hidden_size: int, vocabulary: Optional[Sequence[str]] = None,
                 bidirectional: bool = False, num_layers: int = 1):
        super().__init__()
        if vocabulary is not None and len(vocabulary) != num_classes:
            raise ValueError(f"If vocabulary is specified, it's length should be equal to the num_classes. Instead got: "
                             f"num_classes={num_classes} and len(vocabulary)={len(vocabulary)}")
        self.vocabulary = list(vocabulary) if vocabulary is not None else None
        self._num_classes = num_classes + 1
        self.lstm_layer = nn.LSTM(feat_in, lstm_hidden_size, num_layers, batch_first=True, bidirectional=bidirectional)
        self.linear_layer = nn.Linear(lstm_hidden_size * (2 if bidirectional else 1), self._num_classes)

    @property
    def num_classes_with_blank(self):
        return self._num_classes

    def forward(self, encoder_output):
        y, _ = self.lstm_layer(encoder_output.transpose(1, 2).float())
        return F.log_softmax(self.linear_layer(y), dim=-1)


# ---------------------------------------------------------------------------------------------- Transformer encoder
@dataclass
class TransformerEncoderConfig:
    feat_in: int = 128
    d_model: int = 512
    n_heads: int = 8
    n_layers: int = 17
    drop_rate: float = 0.1
    qkv_bias: bool = False
    qk_norm: bool = False
    ff_expansion: float = 4.0
    pre_block_norm: bool = True
    subsampling_factor: int = 4
    attn_mode: str = "full"
    self_attention_model: str = "rel_pos"


class _Attention(nn.Module):
    def __init__(self, c: TransformerEncoderConfig):
        super().__init__()
        self.h, self.dk = c.n_heads, c.d_model // c.n_heads
        self.qkv = nn.Linear(c.d_model, 3 * c.d_model, bias=c.qkv_bias)
        self.out = nn.Linear(c.d_model, c.d_model)
        self.q_norm = nn.LayerNorm(self.dk) if c.qk_norm else None
        self.k_norm = nn.LayerNorm(self.dk) if c.qk_norm else None
        self.rel = c.self_attention_model == "rel_pos"
        if self.rel:
            self.linear_pos = nn.Linear(c.d_model, c.d_model, bias=False)
            self.pos_bias_u = nn.Parameter(torch.zeros(self.h, self.dk))
            self.pos_bias_v = nn.Parameter(torch.zeros(self.h, self.dk))
        self.drop = c.drop_rate

    def forward(self, x, mask, pos_emb=None):
        B, T, _ = x.shape
        qkv = ops.linear(x, self.qkv.weight, self.qkv.bias).view(B, T, 3, self.h, self.dk)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if self.q_norm is not None:
            q = F.layer_norm(q.float(), (self.dk,), self.q_norm.weight, self.q_norm.bias, self.q_norm.eps).to(x.dtype)
            k = F.layer_norm(k.float(), (self.dk,), self.k_norm.weight, self.k_norm.bias, self.k_norm.eps).to(x.dtype)
        if self.rel:
            p = ops.linear(pos_emb.to(x.dtype), self.linear_pos.weight, None).view(1, -1, self.h, self.dk)
            ctx = ops.relpos_attention(q, k, v, p, self.pos_bias_u, self.pos_bias_v, mask, self.drop, self.training)
        else:
            ctx = ops.mha_attention(q, k, v, mask, self.drop, self.training)
        return ops.linear(ctx.reshape(B, T, -1), self.out.weight, self.out.bias)


class TransformerBlock(nn.Module):
    def __init__(self, c: TransformerEncoderConfig):
        super().__init__()
        hidden = int(c.ff_expansion * c.d_model)
        self.norm1, self.norm2 = nn.LayerNorm(c.d_model), nn.LayerNorm(c.d_model)
        self.attn = _Attention(c)
        self.fc1, self.fc2 = nn.Linear(c.d_model, hidden), nn.Linear(hidden, c.d_model)
        self.drop = nn.Dropout(c.drop_rate)

    def forward(self, x, mask, pos_emb=None):
        x = x + self.drop(self.attn(ops.layer_norm(x, self.norm1.weight, self.norm1.bias, self.norm1.eps), mask, pos_emb))
        h = ops.linear(ops.layer_norm(x, self.norm2.weight, self.norm2.bias, self.norm2.eps), self.fc1.weight, self.fc1.bias, act="gelu")
        return ops.linear(self.drop(h), self.fc2.weight, self.fc2.bias, residual=x)


class TransformerEncoder(NeuralModule):
    """Sub-sampling front end + pre-norm Transformer blocks; I/O as the Conformer encoder ([B, D, T] in and out)."""

    def __init__(self, feat_in: int = 128, d_model: int = 512, n_heads: int = 8, n_layers: int = 17, drop_rate: float = 0.1,
                 qkv_bias: bool = False, qk_norm: bool = False, ff_expansion: float = 4.0, pre_block_norm: bool = True,
                 subsampling: str = "dw_striding", subsampling_factor: int = 4, subsampling_conv_channels: int = 256,
                 attn_mode: str = "full", self_attention_model: Optional[str] = "rel_pos", xscaling: bool = False, pos_emb_max_len: int = 5000,
                 dropout_pre_encoder: Optional[float] = None, dropout_emb: float = 0.0, feat_out: int = -1, sync_max_audio_length: bool = True):
        super().__init__()
        self_attention_model = self_attention_model or "no_pos"
        dropout_pre_encoder = drop_rate if dropout_pre_encoder is None else dropout_pre_encoder
        if d_model % n_heads:
            raise ValueError(f"d_model ({d_model}) must be divisible by n_heads ({n_heads})")
        if d_model // n_heads < 16:
            raise ValueError(f"head dimension d_model / n_heads = {d_model // n_heads} is below 16, the smallest the attention kernels tile")
        if attn_mode not in ("full", "causal"):
            raise ValueError(f"attn_mode must be one of ('full', 'causal'), got {attn_mode!r}")
        if self_attention_model not in ("abs_pos", "rel_pos", "no_pos"):
            raise ValueError(f"self_attention_model must be one of ('abs_pos', 'rel_pos', 'no_pos'), got {self_attention_model!r}")
        self.cfg = TransformerEncoderConfig(feat_in, d_model, n_heads, n_layers, drop_rate, qkv_bias, qk_norm, ff_expansion, pre_block_norm,
                                            subsampling_factor, attn_mode, self_attention_model)
        self.d_model, self._feat_in, self.subsampling_factor = d_model, feat_in, subsampling_factor
        self._feat_out = feat_out if feat_out and feat_out > 0 else d_model
        self.out_proj = nn.Linear(d_model, self._feat_out) if self._feat_out != d_model else None
        self.sync_max_audio_length, self.max_audio_length = sync_max_audio_length, pos_emb_max_len
        self.pre_encode = _pre_encoder(subsampling, subsampling_factor, feat_in, d_model, subsampling_conv_channels)
        xs = math.sqrt(d_model) if xscaling else None
        if self_attention_model == "rel_pos":
            self.pos_enc = RelPositionalEncoding(d_model=d_model, dropout_rate=dropout_pre_encoder, max_len=pos_emb_max_len, xscale=xs,
                                                 dropout_rate_emb=dropout_emb)
        elif self_attention_model == "abs_pos":
            self.pos_enc = PositionalEncoding(d_model=d_model, dropout_rate=dropout_pre_encoder, max_len=pos_emb_max_len, xscale=xs)
        else:
            self.pos_enc = None
        self.pre_norm = nn.LayerNorm(d_model) if pre_block_norm else None
        self.layers = nn.ModuleList([TransformerBlock(self.cfg) for _ in range(n_layers)])
        self.final_norm = nn.LayerNorm(d_model)

    def forward(self, audio_signal, length, bypass_pre_encode: bool = False):
        x = audio_signal if bypass_pre_encode else audio_signal.transpose(1, 2)
        if not bypass_pre_encode:
            if isinstance(self.pre_encode, nn.Linear):
                x = self.pre_encode(x)
            else:
                x, length = self.pre_encode(x, length)
        cdt = ops.get_compute_dtype()
        if cdt is not None:
            x = x.to(cdt)
        T = x.shape[1]
        pos_emb = None
        if self.pos_enc is not None:
            self.pos_enc.extend_pe(T, x.device)
            x, pos_emb = self.pos_enc(x)
        if self.pre_norm is not None:
            x = ops.layer_norm(x, self.pre_norm.weight, self.pre_norm.bias, self.pre_norm.eps)
        pad = torch.arange(T, device=x.device)[None, :] >= length[:, None]
        hidden = pad[:, None, :] | pad[:, :, None]
        if self.cfg.attn_mode == "causal":
            hidden = hidden | torch.ones(T, T, dtype=torch.bool, device=x.device).triu(1)[None]
        for blk in self.layers:
            x = blk(x, hidden, pos_emb)
        x = ops.layer_norm(x, self.final_norm.weight, self.final_norm.bias, self.final_norm.eps)
        if self.out_proj is not None:
            x = ops.linear(x, self.out_proj.weight, self.out_proj.bias)
        return x.transpose(1, 2), length

    def set_max_audio_length(self, max_audio_length: int):
        """Grows the positional table to ``max_audio_length`` frames (after sub-sampling)."""
        self.max_audio_length = max(self.max_audio_length, int(max_audio_length))
        if self.pos_enc is not None:
            self.pos_enc.extend_pe(self.max_audio_length, next(self.parameters()).device)

    def update_max_seq_length(self, seq_length: int, device=None):
        """Before a forward on ``seq_length`` input frames: with ``sync_max_audio_length`` every rank grows its positional table to
        the longest length among ranks, so that no rank re-allocates inside a step the others have passed."""
        if self.sync_max_audio_length and torch.distributed.is_available() and torch.distributed.is_initialized():
            t = torch.tensor([seq_length], dtype=torch.float32, device=device if torch.distributed.get_backend() == "nccl" else "cpu")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            seq_length = int(t.item())
        need = -(-int(seq_length) // max(1, self.subsampling_factor))
        if need > self.max_audio_length:
            self.set_max_audio_length(need)


# ---------------------------------------------------------------------------------------------- wav2vec
class GradMultiply(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        return grad * ctx.scale, None


class ConvFeatureEncoder(NeuralModule):
    """Raw waveform -> frame embeddings: a stack of strided Conv1d blocks (``extractor_mode`` "default": GroupNorm after the
    first block only; "layer_norm": LayerNorm after every block), GELU, final LayerNorm + projection to ``embedding_dim``."""

    def __init__(self, conv_layers: List[Dict[str, int]], extractor_mode: str = "layer_norm", conv_bias: bool = False,
                 feature_grad_mult: float = 1.0, normalize_audio: bool = True, embedding_dim: int = 768):
        super().__init__()
        if extractor_mode not in ("default", "layer_norm"):
            raise ValueError("extractor_mode must be 'default' or 'layer_norm'")
        self.grad_mult, self.normalize_input, self.mode = feature_grad_mult, normalize_audio, extractor_mode
        self.convs, self.norms, self.spec = nn.ModuleList(), nn.ModuleList(), []
        c_in = 1
        for i, cl in enumerate(conv_layers):
            dim, k, s = int(cl["emb_dim"]), int(cl["kernel_size"]), int(cl["stride"])
            conv = nn.Conv1d(c_in, dim, k, stride=s, bias=conv_bias)
            nn.init.kaiming_normal_(conv.weight)
            self.convs.append(conv)
            if extractor_mode == "layer_norm":
                self.norms.append(nn.LayerNorm(dim))
            elif i == 0:
                self.norms.append(nn.GroupNorm(dim, dim))
            else:
                self.norms.append(nn.Identity())
            self.spec.append((k, s))
            c_in = dim
        self.layer_norm = nn.LayerNorm(c_in)
        self.post_extract_proj = nn.Linear(c_in, embedding_dim) if c_in != embedding_dim else None
        self.feat_out = embedding_dim

    def get_subsampled_lens(self, lens: torch.Tensor) -> torch.Tensor:
        for k, s in self.spec:
            lens = torch.div(lens - k, s, rounding_mode="floor") + 1
        return lens.clamp(min=0)

    def forward(self, input_signal, length):
        x = input_signal.float()
        if self.normalize_input:
            m = (torch.arange(x.shape[1], device=x.device)[None, :] < length[:, None]).float()
            n = m.sum(1, keepdim=True).clamp(min=1)
            mean = (x * m).sum(1, keepdim=True) / n
            var = (((x - mean) * m) ** 2).sum(1, keepdim=True) / n
            x = (x - mean) / torch.sqrt(var + 1e-5) * m
        x = x.unsqueeze(1)
        for conv, norm in zip(self.convs, self.norms):
            x = conv(x)
            if isinstance(norm, nn.LayerNorm):
                x = norm(x.transpose(1, 2)).transpose(1, 2)
            else:
                x = norm(x)
            x = F.gelu(x)
        if self.grad_mult != 1.0:
            x = GradMultiply.apply(x, self.grad_mult)
        x = self.layer_norm(x.transpose(1, 2))
        if self.post_extract_proj is not None:
            x = self.post_extract_proj(x)
        return x.transpose(1, 2), self.get_subsampled_lens(length)


class Wav2VecTransformerEncoder(NeuralModule):
    """Convolutional (grouped, weight-normalised) positional embedding + post-norm Transformer with layer drop."""

    def __init__(self, embedding_dim: int = 768, num_layers: int = 12, num_heads: int = 8, inner_size: int = 3072, dropout: float = 0.1,
                 layer_drop: float = 0.0, pos_kernel_size: int = 128, pos_groups: int = 16):
        super().__init__()
        self.layer_drop, self.dropout = layer_drop, dropout
        self.pos_conv = nn.Conv1d(embedding_dim, embedding_dim, pos_kernel_size, padding=pos_kernel_size // 2, groups=pos_groups)
        nn.init.normal_(self.pos_conv.weight, mean=0, std=math.sqrt(4.0 / (pos_kernel_size * embedding_dim)))
        nn.init.constant_(self.pos_conv.bias, 0)
        self.pos_conv = nn.utils.parametrizations.weight_norm(self.pos_conv, name="weight", dim=2)
        self.trim = 1 if pos_kernel_size % 2 == 0 else 0
        self.layer_norm = nn.LayerNorm(embedding_dim)
        self.layers = nn.ModuleList([nn.TransformerEncoderLayer(embedding_dim, num_heads, inner_size, dropout, activation="gelu", batch_first=True)
                                     for _ in range(num_layers)])

    def forward(self, audio_signal, length):
        x = audio_signal.float()                                            # [B, D, T]
        pad = torch.arange(x.shape[2], device=x.device)[None, :] >= length[:, None]
        x = x.masked_fill(pad[:, None, :], 0.0)
        pos = self.pos_conv(x)
        if self.trim:
            pos = pos[:, :, : -self.trim]
        x = (x + F.gelu(pos)).transpose(1, 2)
        x = F.dropout(self.layer_norm(x), self.dropout, self.training)
        for layer in self.layers:
            if self.training and self.layer_drop > 0 and float(torch.rand(())) < self.layer_drop:
                continue
            x = layer(x, src_key_padding_mask=pad)
        return x.transpose(1, 2), length


# ---------------------------------------------------------------------------------------------- parallel-expert encoder
def sinusoid_table(n: int, dim: int) -> torch.Tensor:
    pos = torch.arange(n, dtype=torch.float32).unsqueeze(1)
    div = torch.exp(torch.arange(0, dim, 2, dtype=torch.float32) * -(math.log(10000.0) / dim))
    pe = torch.zeros(n, dim)
    pe[:, 0::2], pe[:, 1::2] = torch.sin(pos * div), torch.cos(pos * div)
    return pe


class ParallelExpertEncoder(nn.Module):
    """A diarization expert (Sortformer) and an ASR Conformer encoder read the same features; the speaker activities
    ``[B, T, n_spk]`` are layer-normalised, mapped through a fixed sinusoidal kernel ``[n_spk, D]`` and added to the
    layer-normalised ASR states.  ``spk_targets`` (e.g. from RTTM) overrides the diarizer."""

    def __init__(self, asr_encoder: nn.Module, diarization_model: Optional[nn.Module], n_spk: int = 4, freeze_diar: bool = True,
                 freeze_asr: bool = False):
        super().__init__()
        self.asr_encoder, self.diarization_model = asr_encoder, diarization_model
        self.freeze_diar, self.freeze_asr, self.n_spk = freeze_diar, freeze_asr, n_spk
        D = asr_encoder.d_model
        self.asr_norm, self.diar_norm = nn.LayerNorm(D), nn.LayerNorm(n_spk)
        self.register_buffer("diar_kernel", sinusoid_table(n_spk, D), persistent=False)
        if freeze_diar and diarization_model is not None:
            for p in diarization_model.parameters():
                p.requires_grad_(False)
        if freeze_asr:
            for p in asr_encoder.parameters():
                p.requires_grad_(False)

    @property
    def d_model(self):
        return self.asr_encoder.d_model

    @property
    def subsampling_factor(self):
        return self.asr_encoder.subsampling_factor

    def train(self, mode: bool = True):
        super().train(mode)
        if self.freeze_diar and self.diarization_model is not None:
            self.diarization_model.eval()
        if self.freeze_asr:
            self.asr_encoder.eval()
        return self

    @staticmethod
    def align_frames(spk: torch.Tensor, T: int) -> torch.Tensor:
        if spk.shape[1] < T:
            return torch.cat([spk, spk[:, -1:].expand(-1, T - spk.shape[1], -1)], dim=1)
        return spk[:, :T]

    def fuse(self, asr_encoded: torch.Tensor, spk_targets: torch.Tensor) -> torch.Tensor:
        h = asr_encoded.transpose(1, 2).float()
        spk = self.align_frames(spk_targets, h.shape[1]).float()
        return (self.asr_norm(h) + self.diar_norm(spk) @ self.diar_kernel).transpose(1, 2).to(asr_encoded.dtype)

    def forward(self, audio_signal, length, spk_targets=None):
        if spk_targets is None and self.diarization_model is not None:
            with torch.set_grad_enabled(not self.freeze_diar and torch.is_grad_enabled()):
                emb, emb_len = self.diarization_model.frontend_encoder(audio_signal, length)
                spk_targets = self.diarization_model.forward_infer(emb, emb_len)
        with torch.set_grad_enabled(not self.freeze_asr and torch.is_grad_enabled()):
            enc, enc_len = self.asr_encoder(audio_signal=audio_signal, length=length)[:2]
        return (self.fuse(enc, spk_targets) if spk_targets is not None else enc), enc_len

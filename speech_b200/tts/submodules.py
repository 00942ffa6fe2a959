"""Building blocks of the spectrogram generators: initialised linear / convolution wrappers, mask-aware normalisation and
partial convolution, the location-sensitive attention of Tacotron 2 with its pre-net, conditional layer norm / conditional
input for speaker conditioning, and the speaker encoder (look-up table, global style tokens over a reference encoder,
pre-computed embeddings).
Reference: ``tts/modules/submodules.py``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

SUPPORTED_CONDITION_TYPES = ("add", "concat", "layernorm")


def check_support_condition_types(condition_types: Sequence[str]) -> None:
    for t in condition_types:
        if t not in SUPPORTED_CONDITION_TYPES:
            raise ValueError(f"unknown conditioning type '{t}': choose from {list(SUPPORTED_CONDITION_TYPES)}")


class LinearNorm(nn.Module):
    """Linear layer with Xavier-uniform weights scaled for the non-linearity that follows."""

    def __init__(self, in_dim: int, out_dim: int, bias: bool = True, w_init_gain: str = "linear"):
        super().__init__()
        self.linear_layer = nn.Linear(in_dim, out_dim, bias=bias)
        nn.init.xavier_uniform_(self.linear_layer.weight, gain=nn.init.calculate_gain(w_init_gain))

    def forward(self, x):
        return self.linear_layer(x)


class MaskedInstanceNorm1d(nn.InstanceNorm1d):
    """Instance norm over ``[B, C, T]`` whose statistics only see the frames where ``mask [B, 1, T]`` is set; padded frames come out 0."""

    def __init__(self, d_channel: int, unbiased: bool = True, affine: bool = False):
        super().__init__(d_channel, affine=affine)
        self.unbiased = unbiased

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        m = mask.to(x.dtype)
        n = m.sum(-1, keepdim=True).clamp(min=1)
        mean = (x * m).sum(-1, keepdim=True) / n
        var = (((x - mean) * m) ** 2).sum(-1, keepdim=True) / ((n - 1).clamp(min=1) if self.unbiased else n)
        y = (x - mean) / torch.sqrt(var + self.eps)
        if self.affine:
            y = y * self.weight.view(1, -1, 1) + self.bias.view(1, -1, 1)
        return y * m


class PartialConv1d(nn.Conv1d):
    """Convolution over the valid frames only: the input is masked, and each output is rescaled by (window size / number of valid
    frames under the window) so that windows hanging over the padding are not attenuated; outputs with no valid frame are 0."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.register_buffer("_ones", torch.ones(1, 1, self.kernel_size[0]), persistent=False)

    def forward(self, x: torch.Tensor, mask_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        if mask_in is None:
            return super().forward(x)
        m = mask_in.to(x.dtype)
        with torch.no_grad():
            cover = F.conv1d(m, self._ones.to(x.dtype), stride=self.stride, padding=self.padding, dilation=self.dilation)
            ratio = self.kernel_size[0] / cover.clamp(min=1e-6)
            valid = (cover > 0).to(x.dtype)
            ratio = ratio * valid
        raw = F.conv1d(x * m, self.weight, None, self.stride, self.padding, self.dilation, self.groups)
        out = raw * ratio
        if self.bias is not None:
            out = (out + self.bias.view(1, -1, 1)) * valid
        return out


class ConvNorm(nn.Module):
    """``same``-padded 1-D convolution with Xavier initialisation; with ``use_partial_padding`` it becomes a partial convolution driven by
    the mask, with ``norm_fn`` (a module class taking the channel count) the output is normalised (mask-aware when the norm accepts a mask)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 1, stride: int = 1, padding: Optional[int] = None, dilation: int = 1,
                 bias: bool = True, w_init_gain: str = "linear", use_partial_padding: bool = False, use_weight_norm: bool = False, norm_fn=None):
        super().__init__()
        if padding is None:
            if kernel_size % 2 != 1:
                raise ValueError("automatic padding needs an odd kernel size")
            padding = dilation * (kernel_size - 1) // 2
        self.use_partial_padding = use_partial_padding
        cls = PartialConv1d if use_partial_padding else nn.Conv1d
        self.conv = cls(in_channels, out_channels, kernel_size, stride=stride, padding=padding, dilation=dilation, bias=bias)
        nn.init.xavier_uniform_(self.conv.weight, gain=nn.init.calculate_gain(w_init_gain))
        if use_weight_norm:
            self.conv = nn.utils.parametrizations.weight_norm(self.conv)
        self.norm = norm_fn(out_channels, affine=True) if norm_fn is not None else None

    def forward(self, signal: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = self.conv(signal, mask) if self.use_partial_padding else self.conv(signal * mask if mask is not None else signal)
        if self.norm is not None:
            y = self.norm(y, mask) if isinstance(self.norm, MaskedInstanceNorm1d) and mask is not None else self.norm(y)
        return y * mask if mask is not None else y


class Prenet(nn.Module):
    """Bottleneck in front of an autoregressive decoder: ReLU layers with dropout that stays ON at inference (it is the decoder's source
    of variation); ``inference=True`` draws one dropout mask for the whole batch."""

    def __init__(self, in_dim: int, sizes: Sequence[int], p_dropout: float = 0.5):
        super().__init__()
        self.layers = nn.ModuleList(LinearNorm(i, o, bias=False) for i, o in zip([in_dim] + list(sizes[:-1]), sizes))
        self.p_dropout = p_dropout

    def forward(self, x: torch.Tensor, inference: bool = False) -> torch.Tensor:
        for lin in self.layers:
            x = F.relu(lin(x))
            if inference and self.p_dropout > 0:
                keep = torch.bernoulli(torch.full_like(x[:1], 1.0 - self.p_dropout)) / (1.0 - self.p_dropout)
                x = x * keep
            else:
                x = F.dropout(x, self.p_dropout, training=True)
        return x


class LocationLayer(nn.Module):
    """Features of the previous and cumulative attention weights ``[B, 2, T]`` → ``[B, T, attention_dim]``."""

    def __init__(self, attention_n_filters: int, attention_kernel_size: int, attention_dim: int):
        super().__init__()
        self.location_conv = ConvNorm(2, attention_n_filters, attention_kernel_size, bias=False)
        self.location_dense = LinearNorm(attention_n_filters, attention_dim, bias=False, w_init_gain="tanh")

    def forward(self, attention_weights_cat: torch.Tensor) -> torch.Tensor:
        return self.location_dense(self.location_conv(attention_weights_cat).transpose(1, 2))


class Attention(nn.Module):
    """Location-sensitive additive attention: ``e_t = v . tanh(W q + V memory_t + U location_t)``."""

    def __init__(self, attention_rnn_dim: int, embedding_dim: int, attention_dim: int, attention_location_n_filters: int, attention_location_kernel_size: int):
        super().__init__()
        self.query_layer = LinearNorm(attention_rnn_dim, attention_dim, bias=False, w_init_gain="tanh")
        self.memory_layer = LinearNorm(embedding_dim, attention_dim, bias=False, w_init_gain="tanh")
        self.v = LinearNorm(attention_dim, 1, bias=False)
        self.location_layer = LocationLayer(attention_location_n_filters, attention_location_kernel_size, attention_dim)

    def get_alignment_energies(self, query, processed_memory, attention_weights_cat):
        return self.v(torch.tanh(self.query_layer(query.unsqueeze(1)) + self.location_layer(attention_weights_cat) + processed_memory)).squeeze(-1)

    def forward(self, attention_hidden_state, memory, processed_memory, attention_weights_cat, mask) -> Tuple[torch.Tensor, torch.Tensor]:
        """``mask``: True on padded memory positions.  Returns (context [B, D], weights [B, T])."""
        e = self.get_alignment_energies(attention_hidden_state, processed_memory, attention_weights_cat)
        if mask is not None:
            e = e.masked_fill(mask, float("-inf"))
        w = torch.softmax(e, dim=1)
        return torch.bmm(w.unsqueeze(1), memory).squeeze(1), w


class ConditionalLayerNorm(nn.LayerNorm):
    """Layer norm whose scale and shift are predicted from a conditioning vector when ``'layernorm'`` is among the condition types (the
    predictors start at the identity: scale 1, shift 0); a plain layer norm otherwise."""

    def __init__(self, hidden_dim: int, condition_dim: Optional[int] = None, condition_types: Sequence[str] = ()):
        check_support_condition_types(condition_types)
        self.condition = "layernorm" in condition_types
        super().__init__(hidden_dim, elementwise_affine=not self.condition)
        if self.condition:
            self.cond_weight = nn.Linear(condition_dim, hidden_dim)
            self.cond_bias = nn.Linear(condition_dim, hidden_dim)
            nn.init.zeros_(self.cond_weight.weight); nn.init.ones_(self.cond_weight.bias)
            nn.init.zeros_(self.cond_bias.weight); nn.init.zeros_(self.cond_bias.bias)

    def forward(self, inputs: torch.Tensor, conditioning: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = super().forward(inputs)
        if self.condition:
            if conditioning is None:
                raise ValueError("this layer norm is conditional: pass the conditioning embedding (define a speaker encoder in the model config)")
            y = y * self.cond_weight(conditioning) + self.cond_bias(conditioning)
        return y


class ConditionalInput(nn.Module):
    """Conditions ``inputs [B, T, H]`` on ``conditioning [B, 1, C]`` by addition (projected when C ≠ H) and / or by concatenation followed
    by a projection back to H; with neither type it passes the input through."""

    def __init__(self, hidden_dim: int, condition_dim: int, condition_types: Sequence[str] = ()):
        check_support_condition_types(condition_types)
        super().__init__()
        self.condition_types = [t for t in condition_types if t in ("add", "concat")]
        self.hidden_dim, self.condition_dim = hidden_dim, condition_dim
        if "add" in self.condition_types and condition_dim != hidden_dim:
            self.add_proj = nn.Linear(condition_dim, hidden_dim)
        if "concat" in self.condition_types:
            self.concat_proj = nn.Linear(hidden_dim + condition_dim, hidden_dim)

    def forward(self, inputs: torch.Tensor, conditioning: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not self.condition_types:
            return inputs
        if conditioning is None:
            raise ValueError("this input is conditional: pass the conditioning embedding (define a speaker encoder in the model config)")
        if "add" in self.condition_types:
            inputs = inputs + (self.add_proj(conditioning) if self.condition_dim != self.hidden_dim else conditioning)
        if "concat" in self.condition_types:
            inputs = self.concat_proj(torch.cat([inputs, conditioning.expand(-1, inputs.shape[1], -1)], dim=-1))
        return inputs


class StyleAttention(nn.Module):
    """A bank of learned style tokens attended by the reference embedding (multi-head); the output is the style embedding ``[B, gst_size]``."""

    def __init__(self, gst_size: int = 128, n_style_token: int = 10, n_style_attn_head: int = 4):
        super().__init__()
        token_size = gst_size // n_style_attn_head
        self.tokens = nn.Parameter(torch.randn(n_style_token, token_size))
        self.mha = nn.MultiheadAttention(gst_size, n_style_attn_head, dropout=0.0, bias=True, kdim=token_size, vdim=token_size, batch_first=True)

    def forward(self, inputs: torch.Tensor, token_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        tokens = torch.tanh(self.tokens).unsqueeze(0).expand(inputs.shape[0], -1, -1)
        out, _ = self.mha(query=inputs.unsqueeze(1), key=tokens, value=tokens)
        return out.squeeze(1)


class Conv2DReLUNorm(nn.Module):
    """Channels-last ``[B, W, H, C]`` strided 2-D convolution → ReLU → layer norm over channels → dropout."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 2, padding: int = 1, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        self.conv = nn.Conv2d(in_channels, out_channels, kernel_size, stride=stride, padding=padding, bias=bias)
        self.norm = nn.LayerNorm(out_channels)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x: torch.Tensor, x_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x_mask is not None:
            x = x * x_mask
        x = F.relu(self.conv(x.permute(0, 3, 1, 2))).permute(0, 2, 3, 1)
        return self.dropout(self.norm(x))


class ReferenceEncoder(nn.Module):
    """Mel spectrogram ``[B, n_mels, T]`` → one vector per utterance: a stack of strided 2-D convolutions over (time, mel), then a GRU over
    the down-sampled time axis whose state at each utterance's last valid frame is the output."""

    def __init__(self, n_mels: int, cnn_filters: Sequence[int], dropout: float, gru_hidden: int, kernel_size: int = 3, stride: int = 2, padding: int = 1, bias: bool = True):
        super().__init__()
        chans = [1] + list(cnn_filters)
        self.k, self.s, self.p = kernel_size, stride, padding
        self.layers = nn.ModuleList(Conv2DReLUNorm(chans[i], chans[i + 1], kernel_size, stride, padding, bias, dropout) for i in range(len(cnn_filters)))
        height = int(self.calculate_post_conv_lengths(torch.tensor(n_mels), len(cnn_filters), kernel_size, stride, padding))
        self.gru = nn.GRU(cnn_filters[-1] * height, gru_hidden, batch_first=True)

    @staticmethod
    def calculate_post_conv_lengths(lengths, n_convs: int = 1, kernel_size: int = 3, stride: int = 2, pad: int = 1):
        for _ in range(n_convs):
            lengths = (lengths - kernel_size + 2 * pad) // stride + 1
        return lengths

    @staticmethod
    def lengths_to_masks(lengths: torch.Tensor) -> torch.Tensor:
        return torch.arange(int(lengths.max()), device=lengths.device)[None, :] < lengths[:, None]

    def forward(self, inputs: torch.Tensor, inputs_lengths: torch.Tensor) -> torch.Tensor:
        x = inputs.transpose(1, 2).unsqueeze(3)                        # [B, T, M, 1]
        lens = inputs_lengths
        for layer in self.layers:
            x = layer(x, self.lengths_to_masks(lens)[:, :x.shape[1], None, None].to(x.dtype))
            lens = self.calculate_post_conv_lengths(lens, 1, self.k, self.s, self.p)
        x = x.reshape(x.shape[0], x.shape[1], -1)
        out, _ = self.gru(x)
        last = (lens.clamp(min=1, max=out.shape[1]) - 1).long()
        return out[torch.arange(out.shape[0], device=out.device), last]


class GlobalStyleToken(nn.Module):
    def __init__(self, reference_encoder: ReferenceEncoder, gst_size: int = 128, n_style_token: int = 10, n_style_attn_head: int = 4):
        super().__init__()
        self.reference_encoder = reference_encoder
        self.style_attention = StyleAttention(gst_size, n_style_token, n_style_attn_head)

    def forward(self, inp: torch.Tensor, inp_lengths: torch.Tensor) -> torch.Tensor:
        return self.style_attention(self.reference_encoder(inp, inp_lengths))


class SpeakerLookupTable(nn.Module):
    def __init__(self, n_speakers: int, embedding_dim: int):
        super().__init__()
        self.table = nn.Embedding(n_speakers, embedding_dim)

    def forward(self, speaker: torch.Tensor) -> torch.Tensor:
        return self.table(speaker)


class SpeakerEncoder(nn.Module):
    """Sum of the available speaker representations: a pre-computed embedding set with ``overwrite_precomputed_emb`` (broadcast over the
    batch), the look-up table entry of ``speaker`` ids, and the global-style-token embedding of a reference spectrogram.  Returns
    ``[B, 1, D]`` for broadcasting over time, or ``None`` when nothing is available."""

    def __init__(self, lookup_module: Optional[SpeakerLookupTable] = None, gst_module: Optional[GlobalStyleToken] = None, precomputed_embedding_dim: Optional[int] = None):
        super().__init__()
        self.lookup_module, self.gst_module = lookup_module, gst_module
        self.precomputed_emb = nn.Parameter(torch.empty(precomputed_embedding_dim).normal_()) if precomputed_embedding_dim is not None else None

    def overwrite_precomputed_emb(self, emb: torch.Tensor) -> None:
        self.precomputed_emb = nn.Parameter(emb.detach().clone().reshape(-1))

    def forward(self, batch_size: Optional[int] = None, speaker: Optional[torch.Tensor] = None, reference_spec: Optional[torch.Tensor] = None,
                reference_spec_lens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        if self.precomputed_emb is not None:
            if batch_size is None:
                raise ValueError("a pre-computed speaker embedding needs the batch size")
            return self.precomputed_emb.view(1, 1, -1).expand(batch_size, -1, -1)
        embs = None
        if self.lookup_module is not None and speaker is not None:
            embs = self.lookup_module(speaker)
        if self.gst_module is not None and reference_spec is not None and reference_spec_lens is not None:
            g = self.gst_module(reference_spec, reference_spec_lens)
            embs = g if embs is None else embs + g
        return None if embs is None else embs.unsqueeze(1)

    @staticmethod
    def from_config(cfg, hidden_dim: int) -> "SpeakerEncoder":
        """``{lookup_module: {n_speakers}, gst_module: {n_mels, cnn_filters, dropout, gru_hidden, gst_size, n_style_token, n_style_attn_head},
        precomputed_embedding_dim}`` — every part optional; embedding sizes default to the model width."""
        c = dict(cfg or {})
        lookup = SpeakerLookupTable(int(c["lookup_module"]["n_speakers"]), int(c["lookup_module"].get("embedding_dim", hidden_dim))) if c.get("lookup_module") else None
        gst = None
        if c.get("gst_module"):
            g = dict(c["gst_module"])
            size = int(g.get("gst_size", hidden_dim))
            ref = ReferenceEncoder(int(g.get("n_mels", 80)), list(g.get("cnn_filters", [32, 32, 64, 64, 128, 128])), float(g.get("dropout", 0.2)),
                                   int(g.get("gru_hidden", size)), int(g.get("kernel_size", 3)), int(g.get("stride", 2)), int(g.get("padding", 1)), bool(g.get("bias", True)))
            gst = GlobalStyleToken(ref, size, int(g.get("n_style_token", 10)), int(g.get("n_style_attn_head", 4)))
        return SpeakerEncoder(lookup, gst, c.get("precomputed_embedding_dim"))

"""Transformer encoder / decoder stack used by the AED (Canary) models.

Structure and parameter names follow ``nemo/collections/asr/modules/transformer`` (``transformer_modules.py:29-250``,
``transformer_decoders.py:31-300``, ``transformer_encoders.py``, ``transformer.py:159``):
``TransformerEmbedding`` (token + fixed / learned position embedding + LayerNorm + dropout), ``MultiHeadAttention``
(``query_net/key_net/value_net/out_projection``), ``PositionWiseFF`` (``dense_in/dense_out``), pre-LN or post-LN
blocks with self-attention, cross-attention and feed-forward, and cached ``decoder_mems_list`` for incremental
decoding.  GEMMs, LayerNorm and attention go through ``speech_b200.ops``.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..core.module import NeuralModule

NEG_INF = -10000.0


def form_attention_mask(input_mask: Optional[torch.Tensor], diagonal: Optional[int] = None) -> Optional[torch.Tensor]:
    """[B, T] validity mask (1 = token) -> bool "hidden" mask [B, 1|T, T]; ``diagonal=0`` adds causality."""
    if input_mask is None:
        return None
    hidden = ~input_mask.to(torch.bool).unsqueeze(1)  # [B,1,T]
    if diagonal is not None:
        T = input_mask.shape[1]
        future = torch.triu(torch.ones(T, T, dtype=torch.bool, device=input_mask.device), diagonal=diagonal + 1)
        hidden = hidden | future.unsqueeze(0)
    return hidden


class FixedPositionalEncoding(nn.Module):
    def __init__(self, hidden_size: int, max_sequence_length: int = 512):
        super().__init__()
        self._hidden_size, self._max_sequence_length = hidden_size, max_sequence_length
        pos = torch.arange(0.0, max_sequence_length).unsqueeze(1)
        coef = -math.log(10000.0) / hidden_size
        div = torch.exp(coef * torch.arange(0.0, hidden_size, 2))
        enc = torch.zeros(max_sequence_length, hidden_size)
        enc[:, 0::2] = torch.sin(pos * div)
        enc[:, 1::2] = torch.cos(pos * div)
        enc.div_(math.sqrt(hidden_size))
        self.register_buffer("pos_enc", enc, persistent=True)

    def forward(self, position_ids):
        return torch.embedding(self.pos_enc, position_ids)


class TransformerEmbedding(nn.Module):
    def __init__(self, vocab_size, hidden_size, max_sequence_length=512, num_token_types=2, embedding_dropout=0.0,
                 learn_positional_encodings=False, padding_idx=0):
        super().__init__()
        self.max_sequence_length = max_sequence_length
        self.learn_positional_encodings = learn_positional_encodings
        self.token_embedding = nn.Embedding(vocab_size, hidden_size, padding_idx=padding_idx)
        self.position_embedding = nn.Embedding(max_sequence_length, hidden_size) if learn_positional_encodings else \
            FixedPositionalEncoding(hidden_size, max_sequence_length)
        if num_token_types > 0:
            self.token_type_embedding = nn.Embedding(num_token_types, hidden_size)
        self.layer_norm = nn.LayerNorm(hidden_size, eps=1e-5)
        self.dropout = nn.Dropout(embedding_dropout)

    def forward(self, input_ids, token_type_ids=None, start_pos=0):
        T = input_ids.size(1)
        if T + start_pos > self.max_sequence_length:
            raise ValueError(f"Input sequence is longer than maximum allowed sequence length for positional encoding. "
                             f"Got {T + start_pos} and {self.max_sequence_length}")
        pos = torch.arange(start_pos, start_pos + T, dtype=torch.long, device=input_ids.device).unsqueeze(0).expand_as(input_ids)
        emb = self.token_embedding(input_ids) + self.position_embedding(pos)
        if token_type_ids is not None and hasattr(self, "token_type_embedding"):
            emb = emb + self.token_type_embedding(token_type_ids)
        cdt = ops.get_compute_dtype()
        if cdt is not None and emb.is_cuda:
            emb = emb.to(cdt)
        emb = ops.layer_norm(emb, self.layer_norm.weight, self.layer_norm.bias, self.layer_norm.eps)
        return self.dropout(emb)


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, num_attention_heads, attn_score_dropout=0.0, attn_layer_dropout=0.0):
        super().__init__()
        if hidden_size % num_attention_heads != 0:
            raise ValueError(f"The hidden size ({hidden_size}) is not a multiple of the number of attention heads "
                             f"({num_attention_heads})")
        self.hidden_size, self.num_attention_heads = hidden_size, num_attention_heads
        self.attn_head_size = hidden_size // num_attention_heads
        self.attn_scale = math.sqrt(math.sqrt(self.attn_head_size))
        self.query_net = nn.Linear(hidden_size, hidden_size)
        self.key_net = nn.Linear(hidden_size, hidden_size)
        self.value_net = nn.Linear(hidden_size, hidden_size)
        self.out_projection = nn.Linear(hidden_size, hidden_size)
        self.attn_dropout = nn.Dropout(attn_score_dropout)
        self.layer_dropout = nn.Dropout(attn_layer_dropout)

    def forward(self, queries, keys, values, attention_mask, residual=None):
        B, Tq, _ = queries.shape
        H, dk = self.num_attention_heads, self.attn_head_size
        q = ops.linear(queries, self.query_net.weight, self.query_net.bias).view(B, Tq, H, dk)
        k = ops.linear(keys, self.key_net.weight, self.key_net.bias).view(B, -1, H, dk)
        v = ops.linear(values, self.value_net.weight, self.value_net.bias).view(B, -1, H, dk)
        mask = None
        if attention_mask is not None:
            mask = attention_mask if attention_mask.dtype == torch.bool else attention_mask < -1.0
            if mask.dim() == 4:
                mask = mask[:, 0]
            mask = mask.expand(B, Tq, k.shape[1])
        ctx = ops.mha_attention(q, k, v, mask, self.attn_dropout.p, self.training, scale=1.0 / math.sqrt(dk))
        drop = self.training and self.layer_dropout.p > 0
        out = ops.linear(ctx, self.out_projection.weight, self.out_projection.bias, residual=None if drop else residual)
        if drop:
            out = self.layer_dropout(out)
            if residual is not None:
                out = out + residual
        return out


class PositionWiseFF(nn.Module):
    def __init__(self, hidden_size, inner_size, ffn_dropout=0.0, hidden_act="relu"):
        super().__init__()
        self.dense_in = nn.Linear(hidden_size, inner_size)
        self.dense_out = nn.Linear(inner_size, hidden_size)
        self.layer_dropout = nn.Dropout(ffn_dropout)
        self.act_name = {"relu": "relu", "gelu": "gelu", "swish": "swish", "silu": "swish"}[hidden_act]

    def forward(self, hidden_states, residual=None):
        h = ops.linear(hidden_states, self.dense_in.weight, self.dense_in.bias, act=self.act_name)
        drop = self.training and self.layer_dropout.p > 0
        out = ops.linear(h, self.dense_out.weight, self.dense_out.bias, residual=None if drop else residual)
        if drop:
            out = self.layer_dropout(out)
            if residual is not None:
                out = out + residual
        return out


def _ln(ln: nn.LayerNorm, x):
    return ops.layer_norm(x, ln.weight, ln.bias, ln.eps)


class TransformerEncoderBlock(nn.Module):
    def __init__(self, hidden_size, inner_size, num_attention_heads=1, attn_score_dropout=0.0, attn_layer_dropout=0.0,
                 ffn_dropout=0.0, hidden_act="relu", pre_ln=False):
        super().__init__()
        self.pre_ln = pre_ln
        self.layer_norm_1 = nn.LayerNorm(hidden_size, eps=1e-5)
        self.first_sub_layer = MultiHeadAttention(hidden_size, num_attention_heads, attn_score_dropout, attn_layer_dropout)
        self.layer_norm_2 = nn.LayerNorm(hidden_size, eps=1e-5)
        self.second_sub_layer = PositionWiseFF(hidden_size, inner_size, ffn_dropout, hidden_act)

    def forward(self, encoder_query, encoder_mask, encoder_keys):
        if self.pre_ln:
            q = _ln(self.layer_norm_1, encoder_query)
            k = _ln(self.layer_norm_1, encoder_keys) if encoder_keys is not encoder_query else q
            x = self.first_sub_layer(q, k, k, encoder_mask, residual=encoder_query)
            return self.second_sub_layer(_ln(self.layer_norm_2, x), residual=x)
        x = self.first_sub_layer(encoder_query, encoder_keys, encoder_keys, encoder_mask, residual=encoder_query)
        x = _ln(self.layer_norm_1, x)
        y = self.second_sub_layer(x, residual=x)
        return _ln(self.layer_norm_2, y)


class TransformerEncoder(nn.Module):
    def __init__(self, num_layers, hidden_size, inner_size, mask_future=False, num_attention_heads=1, attn_score_dropout=0.0,
                 attn_layer_dropout=0.0, ffn_dropout=0.0, hidden_act="relu", pre_ln=False, pre_ln_final_layer_norm=True):
        super().__init__()
        self.final_layer_norm = nn.LayerNorm(hidden_size, eps=1e-5) if pre_ln and pre_ln_final_layer_norm else None
        self.layers = nn.ModuleList([TransformerEncoderBlock(hidden_size, inner_size, num_attention_heads, attn_score_dropout,
                                                             attn_layer_dropout, ffn_dropout, hidden_act, pre_ln)
                                     for _ in range(num_layers)])
        self.diag = 0 if mask_future else None

    def forward(self, encoder_states, encoder_mask, encoder_mems_list=None, return_mems=False):
        att_mask = form_attention_mask(encoder_mask, self.diag)
        x = encoder_states
        for layer in self.layers:
            x = layer(x, att_mask, x)
        if self.final_layer_norm is not None:
            x = _ln(self.final_layer_norm, x)
        return x


class TransformerDecoderBlock(nn.Module):
    def __init__(self, hidden_size, inner_size, num_attention_heads=1, attn_score_dropout=0.0, attn_layer_dropout=0.0,
                 ffn_dropout=0.0, hidden_act="relu", pre_ln=False):
        super().__init__()
        self.pre_ln = pre_ln
        self.layer_norm_1 = nn.LayerNorm(hidden_size, eps=1e-5)
        self.first_sub_layer = MultiHeadAttention(hidden_size, num_attention_heads, attn_score_dropout, attn_layer_dropout)
        self.layer_norm_2 = nn.LayerNorm(hidden_size, eps=1e-5)
        self.second_sub_layer = MultiHeadAttention(hidden_size, num_attention_heads, attn_score_dropout, attn_layer_dropout)
        self.layer_norm_3 = nn.LayerNorm(hidden_size, eps=1e-5)
        self.third_sub_layer = PositionWiseFF(hidden_size, inner_size, ffn_dropout, hidden_act)

    def forward(self, decoder_query, decoder_mask, decoder_keys, encoder_states, encoder_mask):
        if self.pre_ln:
            q = _ln(self.layer_norm_1, decoder_query)
            k = _ln(self.layer_norm_1, decoder_keys) if decoder_keys is not decoder_query else q
            x = self.first_sub_layer(q, k, k, decoder_mask, residual=decoder_query)
            x = self.second_sub_layer(_ln(self.layer_norm_2, x), encoder_states, encoder_states, encoder_mask, residual=x)
            return self.third_sub_layer(_ln(self.layer_norm_3, x), residual=x)
        x = self.first_sub_layer(decoder_query, decoder_keys, decoder_keys, decoder_mask, residual=decoder_query)
        x = _ln(self.layer_norm_1, x)
        y = self.second_sub_layer(x, encoder_states, encoder_states, encoder_mask, residual=x)
        y = _ln(self.layer_norm_2, y)
        z = self.third_sub_layer(y, residual=y)
        return _ln(self.layer_norm_3, z)


class TransformerDecoder(nn.Module):
    def __init__(self, num_layers, hidden_size, inner_size, num_attention_heads=1, attn_score_dropout=0.0,
                 attn_layer_dropout=0.0, ffn_dropout=0.0, hidden_act="relu", pre_ln=False, pre_ln_final_layer_norm=True):
        super().__init__()
        self.final_layer_norm = nn.LayerNorm(hidden_size, eps=1e-5) if pre_ln and pre_ln_final_layer_norm else None
        self.layers = nn.ModuleList([TransformerDecoderBlock(hidden_size, inner_size, num_attention_heads, attn_score_dropout,
                                                             attn_layer_dropout, ffn_dropout, hidden_act, pre_ln)
                                     for _ in range(num_layers)])
        self.diagonal = 0

    def forward(self, decoder_states, decoder_mask, encoder_states, encoder_mask, decoder_mems_list=None, return_mems=False,
                return_mems_as_list=True):
        """With ``decoder_mems_list`` the new states are appended to the cached ones (incremental decoding) and the
        per-layer memories ``[embeddings, layer_1, ..., layer_N]`` are returned when ``return_mems`` is set."""
        enc_mask = form_attention_mask(encoder_mask)
        T_new = decoder_states.shape[1]
        mems_out: List[torch.Tensor] = []

        def cat(i, cur):
            if decoder_mems_list is not None:
                cur = torch.cat([decoder_mems_list[i].to(cur.dtype), cur], dim=1)
            if return_mems:
                mems_out.append(cur)
            return cur

        x = decoder_states
        keys = cat(0, x)
        T_all = keys.shape[1]
        full_mask = decoder_mask
        if full_mask is not None and full_mask.shape[1] != T_all:
            pad = torch.ones(full_mask.shape[0], T_all - full_mask.shape[1], dtype=full_mask.dtype, device=full_mask.device)
            full_mask = torch.cat([pad, full_mask], dim=1)
        dec_mask = form_attention_mask(full_mask, self.diagonal)
        if dec_mask is not None:
            dec_mask = dec_mask[:, -T_new:, :] if dec_mask.shape[1] > 1 else dec_mask
        for i, layer in enumerate(self.layers):
            x = layer(x, dec_mask, keys, encoder_states, enc_mask)
            keys = cat(i + 1, x) if i + 1 < len(self.layers) or return_mems else x
        if self.final_layer_norm is not None:
            x = _ln(self.final_layer_norm, x)
        if return_mems:
            # (final states of the new positions, per-layer input memories for the next incremental call)
            return x, (mems_out if return_mems_as_list else torch.stack(mems_out, dim=0))
        return x

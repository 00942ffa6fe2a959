"""Config-facing wrappers of the transformer stack, the token classifier head and the AED sequence generators.

``TransformerDecoderNM`` / ``TransformerEncoderNM`` hold ``_embedding`` + ``_decoder`` / ``_encoder`` sub-modules under the
reference's attribute names (``nemo/collections/asr/modules/transformer/transformer.py:97,106,190,199``; ``embedding`` /
``decoder`` / ``encoder`` are read-only properties there as here), so Canary checkpoints' ``transf_decoder._embedding.*`` and
``transf_decoder._decoder.*`` keys load; ``TokenClassifier`` is ``mlp.layer0`` + log-softmax (``parts/submodules/token_classifier.py``).  Greedy and beam
generators with incremental decoding follow ``transformer_generators.py:36,400``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..core.module import NeuralModule
from .transformer import TransformerDecoder, TransformerEmbedding, TransformerEncoder


class TransformerEncoderNM(NeuralModule):
    def __init__(self, vocab_size, hidden_size, num_layers, inner_size, num_attention_heads, max_sequence_length=512,
                 num_token_types=2, embedding_dropout=0.0, learn_positional_encodings=False, ffn_dropout=0.0,
                 attn_score_dropout=0.0, attn_layer_dropout=0.0, hidden_act="relu", mask_future=False, pre_ln=False,
                 pre_ln_final_layer_norm=True):
        super().__init__()
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self._embedding = TransformerEmbedding(vocab_size, hidden_size, max_sequence_length, num_token_types, embedding_dropout,
                                               learn_positional_encodings)
        self._encoder = TransformerEncoder(num_layers, hidden_size, inner_size, mask_future, num_attention_heads,
                                          attn_score_dropout, attn_layer_dropout, ffn_dropout, hidden_act, pre_ln,
                                          pre_ln_final_layer_norm)

    @property
    def embedding(self):
        return self._embedding

    @property
    def encoder(self):
        return self._encoder

    def forward(self, input_ids, encoder_mask):
        return self._encoder(self._embedding(input_ids), encoder_mask)


class TransformerDecoderNM(NeuralModule):
    def __init__(self, vocab_size, hidden_size, num_layers, inner_size, num_attention_heads, max_sequence_length=512,
                 num_token_types=2, embedding_dropout=0.0, learn_positional_encodings=False, ffn_dropout=0.0,
                 attn_score_dropout=0.0, attn_layer_dropout=0.0, hidden_act="relu", pre_ln=False, pre_ln_final_layer_norm=True,
                 **_):
        super().__init__()
        self.vocab_size, self.hidden_size, self.max_sequence_length = vocab_size, hidden_size, max_sequence_length
        self.num_states = num_layers + 1
        self.return_mems = False
        self._embedding = TransformerEmbedding(vocab_size, hidden_size, max_sequence_length, num_token_types, embedding_dropout,
                                               learn_positional_encodings)
        self._decoder = TransformerDecoder(num_layers, hidden_size, inner_size, num_attention_heads, attn_score_dropout,
                                          attn_layer_dropout, ffn_dropout, hidden_act, pre_ln, pre_ln_final_layer_norm)

    @property
    def embedding(self):
        return self._embedding

    @property
    def decoder(self):
        return self._decoder

    def forward(self, input_ids, decoder_mask, encoder_embeddings, encoder_mask, decoder_mems=None):
        start_pos = 0
        if decoder_mems is not None:
            start_pos = decoder_mems[0].shape[1]
        emb = self.embedding(input_ids, start_pos=start_pos)
        enc = encoder_embeddings
        if emb.dtype != enc.dtype:
            enc = enc.to(emb.dtype)
        return self.decoder(emb, decoder_mask, enc, encoder_mask, decoder_mems_list=decoder_mems,
                            return_mems=self.return_mems or decoder_mems is not None)


def get_transformer(library="nemo", model_name=None, pretrained=False, config_dict=None, encoder=True, pre_ln_final_layer_norm=True):
    cfg = dict(config_dict or {})
    cfg.pop("library", None), cfg.pop("model_name", None), cfg.pop("pretrained", None)
    cls = TransformerEncoderNM if encoder else TransformerDecoderNM
    return cls(pre_ln_final_layer_norm=pre_ln_final_layer_norm, **cfg)


class MultiLayerPerceptron(nn.Module):
    def __init__(self, hidden_size, num_classes, num_layers=2, activation="relu", log_softmax=True):
        super().__init__()
        self.layers = 0
        act = activation
        for _ in range(num_layers - 1):
            setattr(self, f"layer{self.layers}", nn.Linear(hidden_size, hidden_size))
            setattr(self, f"layer{self.layers + 1}", {"relu": nn.ReLU, "gelu": nn.GELU, "tanh": nn.Tanh}[act]())
            self.layers += 2
        setattr(self, f"layer{self.layers}", nn.Linear(hidden_size, num_classes))
        self.layers += 1
        self.log_softmax = log_softmax

    @property
    def last_linear_layer(self):
        return getattr(self, f"layer{self.layers - 1}")

    def forward(self, x, temperature: Optional[float] = None):
        for i in range(self.layers):
            layer = getattr(self, f"layer{i}")
            x = ops.linear(x, layer.weight, layer.bias) if isinstance(layer, nn.Linear) else layer(x)
        x = x.float()
        if temperature is not None:
            x = x / temperature
        return torch.log_softmax(x, dim=-1) if self.log_softmax else x


class TokenClassifier(NeuralModule):
    def __init__(self, hidden_size, num_classes, num_layers=1, activation="relu", log_softmax=True, dropout=0.0,
                 use_transformer_init=True):
        super().__init__()
        self.mlp = MultiLayerPerceptron(hidden_size, num_classes, num_layers, activation, log_softmax)
        self.dropout = nn.Dropout(dropout)
        self.log_softmax = log_softmax

    def set_log_softmax_enabled(self, value: bool):
        self.mlp.log_softmax = value

    def forward(self, hidden_states, temperature: Optional[float] = None):
        return self.mlp(self.dropout(hidden_states), temperature=temperature)


class GreedySequenceGenerator:
    """Greedy / sampling generator with incremental decoding over the decoder's per-layer memories."""

    def __init__(self, embedding, decoder, classifier, pad=0, bos=1, eos=2, max_sequence_length=512, max_delta_length=20,
                 batch_size=1, temperature: Optional[float] = None, n_samples=1):
        self.embedding, self.decoder, self.classifier = embedding, decoder, classifier
        self.pad, self.bos, self.eos = pad, bos, eos
        self.max_seq_length, self.max_delta_len = max_sequence_length, max_delta_length
        self.temperature = temperature

    def _one_step(self, ids, enc, enc_mask, mems, pos):
        emb = self.embedding(ids, start_pos=pos)
        if emb.dtype != enc.dtype:
            emb = emb.to(enc.dtype)
        mask = torch.ones_like(ids)
        x, mems = self.decoder(emb, mask, enc, enc_mask, decoder_mems_list=mems, return_mems=True)
        logp = self.classifier(hidden_states=x[:, -1:], temperature=None)
        return logp, mems

    @torch.no_grad()
    def __call__(self, decoder_input_ids=None, encoder_hidden_states=None, encoder_input_mask=None, return_beam_scores=False):
        enc = encoder_hidden_states
        B = enc.shape[0]
        dev = enc.device
        if decoder_input_ids is None:
            tgt = torch.full((B, 1), self.bos, dtype=torch.long, device=dev)
        else:
            tgt = decoder_input_ids.long()
        max_len = min(self.max_seq_length, enc.shape[1] + self.max_delta_len) if enc is not None else self.max_seq_length
        mems = None
        logp, mems = self._one_step(tgt, enc, encoder_input_mask, None, 0)
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        scores = torch.zeros(B, device=dev)
        pos = tgt.shape[1]
        for _ in range(max(0, max_len - pos)):
            if self.temperature is None:
                sc, nxt = logp[:, -1].max(dim=-1)
            else:
                probs = torch.softmax(logp[:, -1] / self.temperature, dim=-1)
                nxt = torch.multinomial(probs, 1).squeeze(1)
                sc = logp[:, -1].gather(1, nxt[:, None]).squeeze(1)
            nxt = torch.where(done, torch.full_like(nxt, self.pad), nxt)
            scores = scores + torch.where(done, torch.zeros_like(sc), sc)
            tgt = torch.cat([tgt, nxt[:, None]], dim=1)
            done = done | (nxt == self.eos)
            if bool(done.all()):
                break
            logp, mems = self._one_step(nxt[:, None], enc, encoder_input_mask, mems, pos)
            pos += 1
        return (tgt, scores) if return_beam_scores else tgt


class BeamSearchSequenceGenerator(GreedySequenceGenerator):
    """Length-normalised beam search; each utterance is expanded to ``beam_size`` hypotheses processed as one batch."""

    def __init__(self, embedding, decoder, classifier, beam_size=1, len_pen=0.0, **kw):
        super().__init__(embedding, decoder, classifier, **kw)
        self.beam_size, self.len_pen = beam_size, len_pen

    @staticmethod
    def compute_len_penalty(lengths, alpha):
        return ((5 + lengths) / 6).pow(alpha)

    @torch.no_grad()
    def __call__(self, decoder_input_ids=None, encoder_hidden_states=None, encoder_input_mask=None, return_beam_scores=False):
        enc, K = encoder_hidden_states, self.beam_size
        B, dev = enc.shape[0], enc.device
        prompt = decoder_input_ids.long() if decoder_input_ids is not None else torch.full((B, 1), self.bos, dtype=torch.long, device=dev)
        max_len = min(self.max_seq_length, enc.shape[1] + self.max_delta_len)
        logp, mems = self._one_step(prompt, enc, encoder_input_mask, None, 0)
        sc, idx = logp[:, -1].topk(K, dim=-1)                      # [B,K]
        seqs = torch.cat([prompt[:, None, :].expand(B, K, -1), idx[:, :, None]], dim=2)  # [B,K,L]
        scores = sc
        enc_k = enc.repeat_interleave(K, dim=0)
        mask_k = encoder_input_mask.repeat_interleave(K, dim=0) if encoder_input_mask is not None else None
        mems = [m.repeat_interleave(K, dim=0) for m in mems]
        done = idx == self.eos
        lens = torch.full((B, K), prompt.shape[1] + 1, device=dev, dtype=torch.float)
        pos = prompt.shape[1]
        for _ in range(max(0, max_len - pos - 1)):
            if bool(done.all()):
                break
            last = seqs[:, :, -1].reshape(B * K, 1)
            logp, mems = self._one_step(last, enc_k, mask_k, mems, pos)
            pos += 1
            lp = logp[:, -1].view(B, K, -1)
            V = lp.shape[-1]
            # finished beams only extend with pad at no cost
            lp = torch.where(done[:, :, None], torch.full_like(lp, -1e9), lp)
            lp[:, :, self.pad] = torch.where(done, torch.zeros_like(scores), lp[:, :, self.pad])
            cand = scores[:, :, None] + lp
            new_len = lens[:, :, None] + (~done)[:, :, None].float()
            norm = cand / self.compute_len_penalty(new_len, self.len_pen)
            _, flat = norm.view(B, -1).topk(K, dim=-1)
            src, tok = flat // V, flat % V
            scores = cand.view(B, -1).gather(1, flat)
            seqs = torch.cat([seqs.gather(1, src[:, :, None].expand(-1, -1, seqs.shape[2])), tok[:, :, None]], dim=2)
            lens = new_len.expand(-1, -1, V).reshape(B, -1).gather(1, flat)
            done = done.gather(1, src) | (tok == self.eos)
            gidx = (src + torch.arange(B, device=dev)[:, None] * K).view(-1)
            mems = [m[gidx] for m in mems]
        final = scores / self.compute_len_penalty(lens, self.len_pen)
        best = final.argmax(dim=1)
        out = seqs[torch.arange(B, device=dev), best]
        return (out, final.max(dim=1).values) if return_beam_scores else out

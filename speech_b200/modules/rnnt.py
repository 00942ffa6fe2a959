"""Transducer prediction networks and joint networks.

* ``RNNTDecoder`` — ``Embedding(V+1, H, padding_idx=blank)`` -> prepend a zero SOS frame -> time-major
  multi-layer LSTM -> ``[B, H, U+1]``; stateful ``predict`` for decoding; batched state helpers for
  graph decoders (reference: ``nemo/collections/asr/modules/rnnt.py:550-1276``; LSTM factory
  ``nemo/collections/common/parts/rnn.py:25,151``).  Parameter names
  ``prediction.embed.weight``, ``prediction.dec_rnn.lstm.{weight,bias}_{ih,hh}_l{k}`` match.
* ``StatelessTransducerDecoder`` — embedding-context prediction net (``:55-547``).
* ``RNNTJoint`` — ``enc``/``pred`` projections, ``joint_net = [act, dropout?, Linear(H -> V+1+extra)]``
  (``:1279-1835``).  In *fused* mode the joint never builds the ``B x T x U x V`` logits tensor on a
  GPU: projections go to the fused joint+loss kernels (``ops.transducer_joint_loss``); on the CPU the
  same maths runs sub-batch by sub-batch (``fused_batch_size``) as in ``:1495-1641``.
* ``SampledRNNTJoint`` (sampled softmax, ``:1914-2373``) and ``HATJoint`` (separate blank sigmoid,
  ``modules/hybrid_autoregressive_transducer.py``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from .. import ops
from ..core.module import AdapterModuleMixin, NeuralModule
from ..core.neural_types import (AcousticEncodedRepresentation, ElementType, EmbeddedTextType, LabelsType, LengthsType,
                                 LogprobsType, LossType, NeuralType, typecheck)


class LSTMDropout(nn.Module):
    def __init__(self, input_size, hidden_size, num_layers, dropout, forget_gate_bias, t_max=None,
                 weights_init_scale=1.0, hidden_hidden_bias_scale=0.0, proj_size=0):
        super().__init__()
        self.lstm = nn.LSTM(input_size=input_size, hidden_size=hidden_size, num_layers=num_layers,
                            dropout=dropout or 0.0, proj_size=proj_size)
        if t_max is not None:
            for name, p in self.lstm.named_parameters():
                if "bias" in name:
                    h = p.nelement() // 4
                    p.data.fill_(0)
                    p.data[h:2 * h] = torch.log(nn.init.uniform_(p.data[0:h], 1, t_max - 1))
                    p.data[0:h] = -p.data[h:2 * h]
        elif forget_gate_bias is not None:
            for name, p in self.lstm.named_parameters():
                if "bias_ih" in name:
                    p.data[hidden_size:2 * hidden_size].fill_(forget_gate_bias)
                if "bias_hh" in name:
                    p.data[hidden_size:2 * hidden_size] *= float(hidden_hidden_bias_scale)
        self.dropout = nn.Dropout(dropout) if dropout else None
        for name, p in self.named_parameters():
            if "weight" in name or "bias" in name:
                p.data *= float(weights_init_scale)
        self.num_layers = num_layers
        self.hidden_size = hidden_size

    def flat_weights(self) -> List[torch.Tensor]:
        out = []
        for k in range(self.num_layers):
            out += [getattr(self.lstm, f"weight_ih_l{k}"), getattr(self.lstm, f"weight_hh_l{k}"),
                    getattr(self.lstm, f"bias_ih_l{k}"), getattr(self.lstm, f"bias_hh_l{k}")]
        return out

    def forward(self, x, h=None):
        cdt = ops.get_compute_dtype()
        if x.is_cuda and cdt is not None and not ops.eager_allowed() and self.lstm.proj_size == 0:
            h0, c0 = (None, None) if h is None else h
            x, h = ops.lstm(x.to(cdt), self.flat_weights(), h0, c0, self.num_layers,
                            self.lstm.dropout, self.training)
        else:
            x, h = self.lstm(x, h)
        if self.dropout:
            x = self.dropout(x)
        return x, h


def rnn(input_size, hidden_size, num_layers, norm=None, forget_gate_bias=1.0, dropout=0.0, norm_first_rnn=None,
        t_max=None, weights_init_scale=1.0, hidden_hidden_bias_scale=0.0, proj_size=0):
    if norm not in (None, "batch", "layer"):
        raise ValueError(f"unknown norm={norm}")
    if norm is None:
        return LSTMDropout(input_size, hidden_size, num_layers, dropout, forget_gate_bias, t_max, weights_init_scale,
                           hidden_hidden_bias_scale, proj_size)
    if norm == "batch":
        return BNRNNSum(input_size, hidden_size, rnn_layers=num_layers, batch_norm=True, dropout=dropout, forget_gate_bias=forget_gate_bias,
                        norm_first_rnn=bool(norm_first_rnn), t_max=t_max, weights_init_scale=weights_init_scale,
                        hidden_hidden_bias_scale=hidden_hidden_bias_scale, proj_size=proj_size)
    return LayerNormLSTM(input_size, hidden_size, num_layers, dropout, forget_gate_bias, t_max, weights_init_scale, hidden_hidden_bias_scale)


class BNRNNSum(nn.Module):
    """Stack of single-layer LSTMs with BatchNorm over the features in front of each layer (optionally the first too); state
    is threaded per layer.  Reference: ``common/parts/rnn.py:287`` (``BNRNNSum`` / ``StackTime``-free variant)."""

    def __init__(self, input_size, hidden_size, rnn_layers=1, batch_norm=True, dropout=0.0, forget_gate_bias=1.0, norm_first_rnn=False,
                 t_max=None, weights_init_scale=1.0, hidden_hidden_bias_scale=0.0, proj_size=0):
        super().__init__()
        self.rnn_layers = rnn_layers
        self.layers = nn.ModuleList()
        for i in range(rnn_layers):
            in_size = input_size if i == 0 else (proj_size or hidden_size)
            bn = nn.BatchNorm1d(in_size) if batch_norm and (i > 0 or norm_first_rnn) else None
            self.layers.append(nn.ModuleDict({"bn": bn if bn is not None else nn.Identity(),
                                              "rnn": LSTMDropout(in_size, hidden_size, 1, dropout if i + 1 < rnn_layers else 0.0, forget_gate_bias, t_max,
                                                                 weights_init_scale, hidden_hidden_bias_scale, proj_size)}))

    def forward(self, x, hx=None):
        """x [T, B, D]; hx = (h [L, B, H], c [L, B, H]) or None."""
        hs, cs = [], []
        for i, l in enumerate(self.layers):
            if isinstance(l["bn"], nn.BatchNorm1d):
                x = l["bn"](x.permute(1, 2, 0).float()).permute(2, 0, 1).to(x.dtype)
            st = None if hx is None else (hx[0][i:i + 1].contiguous(), hx[1][i:i + 1].contiguous())
            x, (h, c) = l["rnn"](x, st)
            hs.append(h)
            cs.append(c)
        return x, (torch.cat(hs, 0), torch.cat(cs, 0))


class LayerNormLSTM(nn.Module):
    """LSTM whose gate pre-activations (input and recurrent parts separately) and cell state are layer-normalised
    (``common/parts/rnn.py:407`` ``ln_lstm``).  The recurrence is a Python loop over time: a training-quality variant for the
    prediction network, where sequences are short."""

    def __init__(self, input_size, hidden_size, num_layers, dropout=0.0, forget_gate_bias=1.0, t_max=None, weights_init_scale=1.0,
                 hidden_hidden_bias_scale=0.0):
        super().__init__()
        self.num_layers, self.hidden_size = num_layers, hidden_size
        self.cells = nn.ModuleList()
        for i in range(num_layers):
            d = input_size if i == 0 else hidden_size
            cell = nn.ModuleDict({"ih": nn.Linear(d, 4 * hidden_size), "hh": nn.Linear(hidden_size, 4 * hidden_size),
                                  "ln_i": nn.LayerNorm(4 * hidden_size), "ln_h": nn.LayerNorm(4 * hidden_size), "ln_c": nn.LayerNorm(hidden_size)})
            with torch.no_grad():
                if forget_gate_bias is not None:
                    cell["ih"].bias[hidden_size:2 * hidden_size].fill_(forget_gate_bias)
                    cell["hh"].bias[hidden_size:2 * hidden_size].mul_(float(hidden_hidden_bias_scale))
                for p in (cell["ih"].weight, cell["hh"].weight, cell["ih"].bias, cell["hh"].bias):
                    p.mul_(float(weights_init_scale))
            self.cells.append(cell)
        self.dropout = nn.Dropout(dropout) if dropout else None

    def forward(self, x, hx=None):
        T, B, _ = x.shape
        H = self.hidden_size
        x = x.float()
        hs, cs = [], []
        for i, cell in enumerate(self.cells):
            h = x.new_zeros(B, H) if hx is None else hx[0][i].float()
            c = x.new_zeros(B, H) if hx is None else hx[1][i].float()
            gi_all = cell["ln_i"](cell["ih"](x))
            outs = []
            for t in range(T):
                g = gi_all[t] + cell["ln_h"](cell["hh"](h))
                i_g, f_g, g_g, o_g = g.chunk(4, dim=-1)
                c = cell["ln_c"](torch.sigmoid(f_g) * c + torch.sigmoid(i_g) * torch.tanh(g_g))
                h = torch.sigmoid(o_g) * torch.tanh(c)
                outs.append(h)
            x = torch.stack(outs)
            if self.dropout is not None and i + 1 < self.num_layers:
                x = self.dropout(x)
            hs.append(h)
            cs.append(c)
        if self.dropout is not None:
            x = self.dropout(x)
        return x, (torch.stack(hs), torch.stack(cs))


def label_collate(labels, device=None):
    if isinstance(labels, torch.Tensor):
        return labels.to(torch.int64)
    if not isinstance(labels, (list, tuple)):
        raise ValueError(f"`labels` should be a list or tensor not {type(labels)}")
    bs, mx = len(labels), max(len(l) for l in labels)
    out = torch.zeros(bs, mx, dtype=torch.int64, device=device)
    for i, l in enumerate(labels):
        out[i, : len(l)] = torch.as_tensor(l, dtype=torch.int64)
    return out


class AbstractRNNTDecoder(NeuralModule):
    def __init__(self, vocab_size, blank_idx, blank_as_pad):
        super().__init__()
        self.vocab_size, self.blank_idx, self.blank_as_pad = vocab_size, blank_idx, blank_as_pad
        if blank_idx not in (0, vocab_size):
            raise ValueError("`blank_idx` must be either 0 or the final token of the vocabulary")


class RNNTDecoder(AbstractRNNTDecoder, AdapterModuleMixin):
    def __init__(self, prednet: Dict[str, Any], vocab_size: int, normalization_mode: Optional[str] = None,
                 random_state_sampling: bool = False, blank_as_pad: bool = True):
        self.pred_hidden = prednet["pred_hidden"]
        self.pred_rnn_layers = prednet["pred_rnn_layers"]
        self.blank_idx = vocab_size
        super().__init__(vocab_size=vocab_size, blank_idx=self.blank_idx, blank_as_pad=blank_as_pad)
        self.random_state_sampling = random_state_sampling
        if blank_as_pad:
            embed = nn.Embedding(vocab_size + 1, self.pred_hidden, padding_idx=self.blank_idx)
        else:
            embed = nn.Embedding(vocab_size, self.pred_hidden)
        self.prediction = nn.ModuleDict({
            "embed": embed,
            "dec_rnn": rnn(input_size=self.pred_hidden, hidden_size=prednet.get("rnn_hidden_size", -1) if
                           prednet.get("rnn_hidden_size", -1) > 0 else self.pred_hidden,
                           num_layers=self.pred_rnn_layers, norm=normalization_mode,
                           forget_gate_bias=prednet.get("forget_gate_bias", 1.0), t_max=prednet.get("t_max", None),
                           dropout=prednet.get("dropout", 0.0), weights_init_scale=prednet.get("weights_init_scale", 1.0),
                           hidden_hidden_bias_scale=prednet.get("hidden_hidden_bias_scale", 0.0),
                           proj_size=self.pred_hidden if 0 < prednet.get("rnn_hidden_size", -1) != self.pred_hidden else 0),
        })
        self._rnnt_export = False

    @property
    def input_types(self):
        return {"targets": NeuralType(("B", "T"), LabelsType()), "target_length": NeuralType(("B",), LengthsType()),
                "states": NeuralType(("D", "B", "D"), ElementType(), optional=True)}

    @property
    def output_types(self):
        return {"outputs": NeuralType(("B", "D", "T"), EmbeddedTextType()),
                "prednet_lengths": NeuralType(("B",), LengthsType()),
                "states": NeuralType(("D", "B", "D"), ElementType(), optional=True)}

    @typecheck()
    def forward(self, targets, target_length, states=None):
        y = label_collate(targets)
        g, states = self.predict(y, state=states, add_sos=not self._rnnt_export)
        return g.transpose(1, 2), target_length, states

    def predict(self, y: Optional[torch.Tensor] = None, state=None, add_sos: bool = True,
                batch_size: Optional[int] = None):
        p = next(self.parameters())
        device, dtype = p.device, p.dtype
        if y is not None:
            y = self.prediction["embed"](y.to(device))
        else:
            B = batch_size if batch_size is not None else (1 if state is None else state[0].size(1))
            y = torch.zeros((B, 1, self.pred_hidden), device=device, dtype=dtype)
        if add_sos:
            B, U, H = y.shape
            y = torch.cat([torch.zeros((B, 1, H), device=y.device, dtype=y.dtype), y], dim=1).contiguous()
        if state is None and self.random_state_sampling and self.training:
            state = self.initialize_state(y)
        if state is not None:
            state = tuple(state)
        g, hid = self.prediction["dec_rnn"](y.transpose(0, 1), state)
        g = g.transpose(0, 1)
        if self.is_adapter_available():
            g = self.forward_enabled_adapters(g)
        return g, hid

    def initialize_state(self, y: torch.Tensor):
        batch = y.size(0)
        if self.random_state_sampling and self.training:
            return (torch.randn(self.pred_rnn_layers, batch, self.pred_hidden, dtype=y.dtype, device=y.device),
                    torch.randn(self.pred_rnn_layers, batch, self.pred_hidden, dtype=y.dtype, device=y.device))
        return (torch.zeros(self.pred_rnn_layers, batch, self.pred_hidden, dtype=y.dtype, device=y.device),
                torch.zeros(self.pred_rnn_layers, batch, self.pred_hidden, dtype=y.dtype, device=y.device))

    # -- decoding helpers --------------------------------------------------------------------------
    def score_hypothesis(self, hypothesis, cache: Dict[Tuple[int], Any]):
        if hypothesis.dec_state is not None:
            device = hypothesis.dec_state[0].device
        else:
            device = next(self.parameters()).device
        blank_state = len(hypothesis.y_sequence) > 0 and hypothesis.y_sequence[-1] == self.blank_idx
        target = torch.full([1, 1], fill_value=hypothesis.y_sequence[-1], device=device, dtype=torch.long)
        lm_token = target[:, -1]
        sequence = tuple(hypothesis.y_sequence)
        if sequence in cache:
            y, new_state = cache[sequence]
        else:
            if blank_state:
                y, new_state = self.predict(None, state=None, add_sos=False, batch_size=1)
            else:
                y, new_state = self.predict(target, state=hypothesis.dec_state, add_sos=False, batch_size=1)
            y = y[:, -1:, :]
            cache[sequence] = (y, new_state)
        return y, new_state, lm_token

    def batch_select_state(self, batch_states, idx: int):
        if batch_states is None:
            return None
        return [s[:, idx] for s in batch_states]

    def batch_replace_states_mask(self, src_states, dst_states, mask, other_src_states=None):
        other = other_src_states if other_src_states is not None else dst_states
        for s, d, o in zip(src_states, dst_states, other):
            torch.where(mask.unsqueeze(0).unsqueeze(-1), s.to(d.dtype), o.to(d.dtype), out=d)

    def batch_replace_states_all(self, src_states, dst_states, batch_size=None):
        for s, d in zip(src_states, dst_states):
            if batch_size is None:
                d.copy_(s)
            else:
                d[:, :batch_size].copy_(s[:, :batch_size])

    def batch_split_states(self, batch_states):
        n = batch_states[0].shape[1]
        return [(batch_states[0][:, i], batch_states[1][:, i]) for i in range(n)]

    @classmethod
    def batch_unsplit_states(cls, batch_states, device=None, dtype=None):
        return (torch.stack([s[0] for s in batch_states], dim=1).to(device=device, dtype=dtype),
                torch.stack([s[1] for s in batch_states], dim=1).to(device=device, dtype=dtype))

    def batch_concat_states(self, batch_states):
        return [torch.stack([s[l] for s in batch_states]) for l in range(len(batch_states[0]))]

    def mask_select_states(self, states, mask):
        return states[0][:, mask], states[1][:, mask]


class StatelessNet(nn.Module):
    """Concatenated embeddings of the last ``context_size`` labels (reference: ``submodules/stateless_net.py``)."""

    def __init__(self, context_size, vocab_size, emb_dim, blank_idx, normalization_mode, dropout):
        super().__init__()
        assert context_size > 0
        self.context_size, self.vocab_size, self.emb_dim, self.blank_idx = context_size, vocab_size, emb_dim, blank_idx
        self.dropout = nn.Dropout(dropout)
        self.norm = nn.LayerNorm(emb_dim, elementwise_affine=False) if normalization_mode == "layer" else nn.Identity()
        embeds = []
        for i in range(context_size):
            embed_size = emb_dim // 2 // context_size if i != 0 else emb_dim - (emb_dim // 2 // context_size) * (context_size - 1)
            embeds.append(nn.Embedding(vocab_size + 1, embed_size, padding_idx=blank_idx))
        self.embeds = nn.ModuleList(embeds)

    def forward(self, y: Optional[torch.Tensor] = None, state: Optional[List[torch.Tensor]] = None):
        outs = []
        B, U = y.shape
        appended = y
        if state is not None:
            appended = torch.cat([state[0], y], dim=1)
            ctx_len = appended.shape[1]
            if ctx_len > self.context_size:
                appended = appended[:, -(self.context_size + U - 1):]
            state = [appended[:, -self.context_size:] if appended.shape[1] >= self.context_size else appended]
        else:
            state = [y[:, -self.context_size:]] if U >= self.context_size else [
                torch.cat([torch.full((B, self.context_size - U), self.blank_idx, dtype=y.dtype, device=y.device), y], dim=1)]
        L = appended.shape[1]
        for i in range(self.context_size):
            # label at distance i behind each of the U output positions
            shifted = torch.full((B, U), self.blank_idx, dtype=y.dtype, device=y.device)
            src_end = L - i
            src_start = src_end - U
            if src_end > 0:
                take = appended[:, max(0, src_start):src_end]
                shifted[:, U - take.shape[1]:] = take
            outs.append(self.embeds[i](shifted))
        out = self.dropout(torch.cat(outs, dim=-1))
        return self.norm(out), state


class StatelessTransducerDecoder(AbstractRNNTDecoder):
    def __init__(self, prednet: Dict[str, Any], vocab_size: int, context_size: int = 1,
                 normalization_mode: Optional[str] = None):
        self.pred_hidden = prednet["pred_hidden"]
        self.blank_idx = vocab_size
        self.context_size = context_size
        super().__init__(vocab_size=vocab_size, blank_idx=self.blank_idx, blank_as_pad=True)
        self.prediction = nn.ModuleDict({"embed": StatelessNet(context_size, vocab_size, self.pred_hidden, self.blank_idx,
                                                               normalization_mode, prednet.get("dropout", 0.0))})
        self._rnnt_export = False

    def forward(self, targets, target_length, states=None):
        y = label_collate(targets)
        g, states = self.predict(y, state=states, add_sos=not self._rnnt_export)
        return g.transpose(1, 2), target_length, states

    def predict(self, y=None, state=None, add_sos=True, batch_size=None):
        device = next(self.parameters()).device
        if y is not None:
            y = y.to(device)
            if add_sos:
                y = torch.cat([torch.full((y.shape[0], 1), self.blank_idx, dtype=y.dtype, device=device), y], dim=1)
            return self.prediction["embed"](y, state)
        B = batch_size if batch_size is not None else (1 if state is None else state[0].size(0))
        y = torch.full((B, 1), self.blank_idx, dtype=torch.long, device=device)
        return self.prediction["embed"](y, state)

    def initialize_state(self, y):
        return [torch.full([y.size(0), self.context_size], fill_value=self.vocab_size, dtype=torch.long, device=y.device)]

    def batch_replace_states_mask(self, src_states, dst_states, mask, other_src_states=None):
        other = other_src_states if other_src_states is not None else dst_states
        torch.where(mask.unsqueeze(-1), src_states[0], other[0], out=dst_states[0])


class RNNTJoint(NeuralModule, AdapterModuleMixin):
    def __init__(self, jointnet: Dict[str, Any], num_classes: int, num_extra_outputs: int = 0,
                 vocabulary: Optional[List] = None, log_softmax: Optional[bool] = None, preserve_memory: bool = False,
                 fuse_loss_wer: bool = False, fused_batch_size: Optional[int] = None, experimental_fuse_loss_wer: Any = None,
                 masking_prob: float = -1.0):
        super().__init__()
        self.vocabulary = vocabulary
        self._vocab_size = num_classes
        self._num_extra_outputs = num_extra_outputs
        self._num_classes = num_classes + 1 + num_extra_outputs
        self.masking_prob = masking_prob
        if experimental_fuse_loss_wer is not None:
            fuse_loss_wer = experimental_fuse_loss_wer
        self._fuse_loss_wer = fuse_loss_wer
        self._fused_batch_size = fused_batch_size
        if fuse_loss_wer and fused_batch_size is None:
            raise ValueError("If `fuse_loss_wer` is set, then `fused_batch_size` cannot be None!")
        self._loss = None
        self._wer = None
        self.log_softmax = log_softmax
        self.preserve_memory = preserve_memory
        self.encoder_hidden = jointnet["encoder_hidden"]
        self.pred_hidden = jointnet["pred_hidden"]
        self.joint_hidden = jointnet["joint_hidden"]
        self.activation = jointnet["activation"]
        dropout = jointnet.get("dropout", 0.0)
        self.pred = nn.Linear(self.pred_hidden, self.joint_hidden)
        self.enc = nn.Linear(self.encoder_hidden, self.joint_hidden)
        act = self.activation.lower()
        if act not in ("relu", "sigmoid", "tanh"):
            raise ValueError("Unsupported activation for joint step - please pass one of [relu, sigmoid, tanh]")
        layers: List[nn.Module] = [{"relu": nn.ReLU(inplace=True), "sigmoid": nn.Sigmoid(), "tanh": nn.Tanh()}[act]]
        if dropout:
            layers.append(nn.Dropout(p=dropout))
        layers.append(nn.Linear(self.joint_hidden, self._num_classes))
        self.joint_net = nn.Sequential(*layers)
        self._joint_dropout = dropout
        self.temperature = 1.0

    # -- properties ----------------------------------------------------------------------------------
    @property
    def num_classes_with_blank(self):
        return self._num_classes

    @property
    def num_extra_outputs(self):
        return self._num_extra_outputs

    @property
    def loss(self):
        return self._loss

    def set_loss(self, loss):
        if not self._fuse_loss_wer:
            raise ValueError("Attempting to set loss module even though `fuse_loss_wer` is not set!")
        self._loss = loss

    @property
    def wer(self):
        return self._wer

    def set_wer(self, wer):
        if not self._fuse_loss_wer:
            raise ValueError("Attempting to set WER module even though `fuse_loss_wer` is not set!")
        self._wer = wer

    @property
    def fuse_loss_wer(self):
        return self._fuse_loss_wer

    def set_fuse_loss_wer(self, fuse_loss_wer, loss=None, metric=None):
        self._fuse_loss_wer = fuse_loss_wer
        self._loss, self._wer = loss, metric

    @property
    def fused_batch_size(self):
        return self._fused_batch_size

    def set_fused_batch_size(self, fused_batch_size):
        self._fused_batch_size = fused_batch_size

    # -- compute -------------------------------------------------------------------------------------
    def project_encoder(self, encoder_output: torch.Tensor) -> torch.Tensor:
        """[B, T, D_enc] -> [B, T, H]."""
        return ops.linear(encoder_output, self.enc.weight, self.enc.bias)

    def project_prednet(self, prednet_output: torch.Tensor) -> torch.Tensor:
        """[B, U, D_pred] -> [B, U, H]."""
        return ops.linear(prednet_output, self.pred.weight, self.pred.bias)

    def joint_after_projection(self, f: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        """f: [B,T,H], g: [B,U,H] -> [B,T,U,V+1+extra] (log-softmaxed on the CPU unless ``log_softmax=False``)."""
        inp = f.unsqueeze(2) + g.unsqueeze(1)
        if self.is_adapter_available():
            inp = self.forward_enabled_adapters(inp)
        res = self.joint_net(inp.float() if inp.dtype != self.joint_net[-1].weight.dtype and not inp.is_cuda else inp)
        if self.temperature != 1.0:
            res = res / self.temperature
        if self.log_softmax is None:
            if not res.is_cuda:
                res = res.log_softmax(dim=-1)
        elif self.log_softmax:
            res = res.log_softmax(dim=-1)
        return res

    def joint(self, f: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        return self.joint_after_projection(self.project_encoder(f), self.project_prednet(g))

    def forward(self, encoder_outputs, decoder_outputs=None, encoder_lengths=None, transcripts=None,
                transcript_lengths=None, compute_wer: bool = False, keep_hypotheses: bool = False):
        """encoder_outputs: [B, D, T]; decoder_outputs: [B, D, U+1].

        Non-fused: returns joint logits [B,T,U+1,V+1+extra].  Fused: returns ``(loss, wer, wer_num, wer_denom)``.
        """
        encoder_outputs = encoder_outputs.transpose(1, 2)
        if decoder_outputs is not None:
            decoder_outputs = decoder_outputs.transpose(1, 2)
        if not self._fuse_loss_wer:
            if decoder_outputs is None:
                raise ValueError("decoder_outputs passed is None, and `fuse_loss_wer` is not set.")
            return self.joint(encoder_outputs, decoder_outputs)
        if self._loss is None or self._wer is None:
            raise ValueError("`fuse_loss_wer` flag is set, but `loss` and `wer` modules were not provided! ")
        if encoder_lengths is None or transcript_lengths is None:
            raise ValueError("`fuse_loss_wer` is set, therefore encoder and target lengths must be provided as well!")
        loss_value = None
        if decoder_outputs is not None:
            f = self.project_encoder(encoder_outputs)
            g = self.project_prednet(decoder_outputs)
            drop = float(self._joint_dropout or 0.0) if self.training else 0.0
            if drop > 0.0 and (not f.is_cuda or self.activation.lower() != "relu" or getattr(self._loss, "kind", "") == "multiblank"):
                # dropout sits between the activation and the output GEMM; the fused kernels apply it for the ReLU joint on GPUs,
                # everything else takes the generic joint
                per_utt = self._loss.forward_from_joint_fn(self, f, g, transcripts, encoder_lengths, transcript_lengths,
                                                           self._fused_batch_size)
            else:
                lin = self.joint_net[-1]
                per_utt = self._loss.forward_fused(f, g, lin.weight, lin.bias, transcripts, encoder_lengths,
                                                   transcript_lengths, self.activation.lower(), self._fused_batch_size,
                                                   dropout_p=drop)
            loss_value = self._loss.reduce(per_utt, transcript_lengths)
        wer = wer_num = wer_denom = None
        if compute_wer:
            with torch.no_grad():
                self._wer.update(predictions=encoder_outputs.transpose(1, 2).detach(),
                                 predictions_lengths=encoder_lengths, targets=transcripts,
                                 targets_lengths=transcript_lengths)
                wer, wer_num, wer_denom = self._wer.compute()
                self._wer.reset()
        return loss_value, wer, wer_num, wer_denom


class HATJoint(RNNTJoint):
    """Hybrid autoregressive transducer joint: blank probability from a separate sigmoid, label
    distribution renormalised over non-blank symbols; optional internal-LM subtraction."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.blank_pred = nn.Sequential(nn.Tanh(), nn.Dropout(p=kwargs.get("jointnet", args[0] if args else {}).get("dropout", 0.0)),
                                        nn.Linear(self.joint_hidden, 1), nn.LogSigmoid())
        self.return_hat_ilm = False

    def joint_after_projection(self, f, g):
        inp = (f.unsqueeze(2) + g.unsqueeze(1)).float()
        blank_logprob = self.blank_pred(inp)
        label_logit = self.joint_net(inp)[..., : self._vocab_size] if self.joint_net[-1].out_features > self._vocab_size \
            else self.joint_net(inp)
        scale = torch.clamp(1 - torch.exp(blank_logprob), min=torch.finfo(label_logit.dtype).eps)
        label_logprob = label_logit.log_softmax(dim=-1) + torch.log(scale)
        res = torch.cat((label_logprob, blank_logprob), dim=-1)
        if self.return_hat_ilm:
            ilm = self.joint_net(g.unsqueeze(1).float())[..., : self._vocab_size].log_softmax(dim=-1)
            return res, ilm
        return res


class SampledRNNTJoint(RNNTJoint):
    """Sampled-softmax joint for very large vocabularies: the loss is computed over the transcript tokens,
    blank and ``n_samples`` uniformly drawn negatives."""

    def __init__(self, jointnet, num_classes, n_samples, **kwargs):
        super().__init__(jointnet=jointnet, num_classes=num_classes, **kwargs)
        self.n_samples = n_samples
        self.register_buffer("blank_id", torch.tensor([self.num_classes_with_blank - 1]), persistent=False)

    def sampled_joint(self, f, g, transcript, transcript_lengths):
        f = self.project_encoder(f).unsqueeze(2)
        g = self.project_prednet(g).unsqueeze(1)
        inp = self.joint_net[:-1](f + g)
        if not self.training:
            return self.joint_net[-1](inp), transcript
        lin = self.joint_net[-1]
        with torch.no_grad():
            vocab = torch.unique(transcript)
            pool = torch.ones(self.num_classes_with_blank - 1, device=transcript.device)
            pool[vocab] = 0
            n = min(self.n_samples, int(pool.sum().item()))
            neg = torch.multinomial(pool, n) if n > 0 else vocab[:0]
            ids = torch.cat([vocab, neg, self.blank_id.to(vocab.device)])
            remap = torch.full((self.num_classes_with_blank,), -1, dtype=torch.long, device=ids.device)
            remap[ids] = torch.arange(len(ids), device=ids.device)
        logits = torch.nn.functional.linear(inp, lin.weight[ids], lin.bias[ids])
        return logits, remap[transcript]

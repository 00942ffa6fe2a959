"""CTC head: ``Conv1d(d -> V+1, k=1)`` then ``log_softmax`` over the vocabulary.

Parameter name ``decoder_layers.0.{weight,bias}`` and the [B, D, T] -> [B, T, V+1] convention follow
``nemo/collections/asr/modules/conv_asr.py:407-470``.  The 1x1 convolution is a GEMM and goes through
``ops.linear``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..core.module import AdapterModuleMixin, NeuralModule
from ..core.neural_types import AcousticEncodedRepresentation, LogprobsType, NeuralType, typecheck


class ConvASRDecoder(NeuralModule, AdapterModuleMixin):
    def __init__(self, feat_in: int, num_classes: int, init_mode: Optional[str] = "xavier_uniform",
                 vocabulary: Optional[List[str]] = None, add_blank: bool = True):
        super().__init__()
        if vocabulary is None and num_classes < 0:
            raise ValueError("Neither of the vocabulary and num_classes are set! At least one of them need to be set.")
        if num_classes <= 0:
            num_classes = len(vocabulary)
        if vocabulary is not None and num_classes != len(vocabulary):
            raise ValueError(f"If vocabulary is specified, it's length should be equal to the num_classes. "
                             f"Instead got: num_classes={num_classes} and len(vocabulary)={len(vocabulary)}")
        self.__vocabulary = list(vocabulary) if vocabulary is not None else None
        self._feat_in = feat_in
        self._num_classes = num_classes + 1 if add_blank else num_classes
        self.decoder_layers = nn.Sequential(nn.Conv1d(feat_in, self._num_classes, kernel_size=1, bias=True))
        if init_mode == "xavier_uniform":
            nn.init.xavier_uniform_(self.decoder_layers[0].weight, gain=1.0)
        self.temperature = 1.0

    @property
    def input_types(self):
        return {"encoder_output": NeuralType(("B", "D", "T"), AcousticEncodedRepresentation())}

    @property
    def output_types(self):
        return {"logprobs": NeuralType(("B", "T", "D"), LogprobsType())}

    @typecheck()
    def forward(self, encoder_output):
        x = encoder_output.transpose(1, 2)
        if self.is_adapter_available():
            x = self.forward_enabled_adapters(x)
        conv = self.decoder_layers[0]
        logits = ops.linear(x, conv.weight.squeeze(-1), conv.bias).float()
        if self.temperature != 1.0:
            logits = logits / self.temperature
        return torch.log_softmax(logits, dim=-1)

    @property
    def vocabulary(self):
        return self.__vocabulary

    @property
    def num_classes_with_blank(self):
        return self._num_classes

"""SpecAugment / SpecCutout on [B, F, T] spectrograms.

Frequency masks and (adaptive) time masks are drawn per utterance and applied in place, fully on
the device without a host synchronisation: mask start / width tensors are sampled with
``torch.rand`` for the whole batch; on a GPU one kernel then writes just the masked elements
(``ops/csrc/decode_aux.cu``), on the CPU they are applied as a broadcast comparison.  Reference behaviour:
``nemo/collections/asr/parts/submodules/spectr_augment.py:25,218`` and the Numba kernel
``parts/numba/spec_augment/spec_aug_numba.py:27-95`` (time-mask width is ``time_width`` frames, or
a fraction of the utterance length when ``time_width`` is a float — "adaptive").
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .. import ops
from ..core.module import NeuralModule
from ..core.neural_types import LengthsType, NeuralType, SpectrogramType, typecheck


class SpecAugment(torch.nn.Module):
    def __init__(self, freq_masks=0, time_masks=0, freq_width=10, time_width: Union[int, float] = 10, rng=None,
                 mask_value=0.0, use_vectorized_code: bool = True):
        super().__init__()
        self.freq_masks, self.time_masks = freq_masks, time_masks
        self.freq_width, self.time_width = freq_width, time_width
        self.mask_value = mask_value
        if isinstance(time_width, float) and not (0.0 <= time_width <= 1.0):
            raise ValueError("If `time_width` is a float value, must be in range [0, 1]")
        self.adaptive_temporal_width = isinstance(time_width, float)

    @torch.no_grad()
    def forward(self, input_spec, length):
        B, F, T = input_spec.shape
        dev = input_spec.device
        if length is None:
            length = torch.full((B,), T, device=dev, dtype=torch.long)
        f_start = f_w = t_start = t_w = None
        if self.freq_masks > 0:
            f_w = torch.randint(0, self.freq_width + 1, (B, self.freq_masks), device=dev)
            f_start = (torch.rand(B, self.freq_masks, device=dev) * (F - f_w + 1).clamp(min=1)).long()
        if self.time_masks > 0:
            if self.adaptive_temporal_width:
                tw = (length.float() * self.time_width).long().clamp(min=1)[:, None]
            else:
                tw = torch.full((B, 1), int(self.time_width), device=dev)
            t_w = (torch.rand(B, self.time_masks, device=dev) * (tw + 1).float()).long()
            hi = (length[:, None] - t_w).clamp(min=1)
            t_start = (torch.rand(B, self.time_masks, device=dev) * hi.float()).long()
        return ops.specaugment(input_spec, f_start, f_w, t_start, t_w, self.mask_value)


class SpecCutout(torch.nn.Module):
    def __init__(self, rect_masks=0, rect_time=5, rect_freq=20, rng=None):
        super().__init__()
        self.rect_masks, self.rect_time, self.rect_freq = rect_masks, rect_time, rect_freq

    @torch.no_grad()
    def forward(self, input_spec):
        B, F, T = input_spec.shape
        dev = input_spec.device
        if self.rect_masks <= 0:
            return input_spec
        fs = (torch.rand(B, self.rect_masks, device=dev) * max(1, F - self.rect_freq)).long()
        ts = (torch.rand(B, self.rect_masks, device=dev) * max(1, T - self.rect_time)).long()
        fw = torch.randint(0, self.rect_freq + 1, (B, self.rect_masks), device=dev)
        tw = torch.randint(0, self.rect_time + 1, (B, self.rect_masks), device=dev)
        f = torch.arange(F, device=dev)[None, None, :, None]
        t = torch.arange(T, device=dev)[None, None, None, :]
        m = ((f >= fs[..., None, None]) & (f < (fs + fw)[..., None, None]) &
             (t >= ts[..., None, None]) & (t < (ts + tw)[..., None, None])).any(dim=1)
        return input_spec.masked_fill(m, 0.0)


class SpectrogramAugmentation(NeuralModule):
    def __init__(self, freq_masks=0, time_masks=0, freq_width=10, time_width=10, rect_masks=0, rect_time=5,
                 rect_freq=20, rng=None, mask_value=0.0, use_vectorized_spec_augment: bool = True,
                 use_numba_spec_augment: bool = False):
        super().__init__()
        self.spec_cutout = SpecCutout(rect_masks, rect_time, rect_freq) if rect_masks > 0 else None
        self.spec_augment = SpecAugment(freq_masks, time_masks, freq_width, time_width, mask_value=mask_value) \
            if freq_masks + time_masks > 0 else None

    @property
    def input_types(self):
        return {"input_spec": NeuralType(("B", "D", "T"), SpectrogramType()),
                "length": NeuralType(("B",), LengthsType(), optional=True)}

    @property
    def output_types(self):
        return {"augmented_spec": NeuralType(("B", "D", "T"), SpectrogramType())}

    @typecheck()
    def forward(self, input_spec, length=None):
        x = input_spec
        if self.spec_cutout is not None:
            x = self.spec_cutout(x)
        if self.spec_augment is not None:
            x = self.spec_augment(x, length)
        return x


class MaskedPatchAugmentation(NeuralModule):
    """Zeroes whole time patches of ``patch_size`` frames.  ``mask_patches >= 1`` is a patch count, ``< 1`` the fraction of the shortest
    utterance's frames to cover (rounded up to whole patches); every utterance of the batch loses the same number of patches, drawn
    without replacement among the patches that lie inside its own length.  The choice is made for the whole batch at once (random scores
    per patch, the lowest-scoring valid ones are masked), so no host loop runs over the batch.  Optional frequency masks follow.
    Reference: ``asr/modules/audio_preprocessing.py`` ``MaskedPatchAugmentation``."""

    def __init__(self, patch_size: int = 48, mask_patches: float = 10.0, freq_masks: int = 0, freq_width: int = 0):
        super().__init__()
        if mask_patches < 0:
            raise ValueError("mask_patches cannot be negative")
        self.patch_size = int(patch_size)
        self.mask_patches = int(mask_patches) if mask_patches >= 1 else None
        self._mask_fraction = float(mask_patches) if mask_patches < 1 else None
        self.spec_augment = SpecAugment(freq_masks, 0, freq_width, 0) if freq_masks > 0 else None

    @property
    def input_types(self):
        return {"input_spec": NeuralType(("B", "D", "T"), SpectrogramType()), "length": NeuralType(("B",), LengthsType())}

    @property
    def output_types(self):
        return {"augmented_spec": NeuralType(("B", "D", "T"), SpectrogramType())}

    @typecheck()
    def forward(self, input_spec, length):
        B, _, T = input_spec.shape
        P = self.patch_size
        min_len = int(length.min())
        if self.mask_patches is None:
            cover = int(min_len * self._mask_fraction)
            n = -(-cover // P)
        else:
            n = self.mask_patches
        n = min(n, min_len // P)
        x = input_spec
        if n > 0:
            n_patches = -(-T // P)
            valid = torch.arange(n_patches, device=x.device)[None, :] < (length // P)[:, None]          # patches fully inside the utterance
            score = torch.rand(B, n_patches, device=x.device).masked_fill(~valid, 2.0)
            chosen = torch.zeros(B, n_patches, dtype=torch.bool, device=x.device).scatter_(1, score.topk(n, dim=1, largest=False)[1], True) & valid
            x = x.masked_fill(chosen.repeat_interleave(P, dim=1)[:, None, :T], 0.0)
        if self.spec_augment is not None:
            x = self.spec_augment(x, length)
        return x


class CropOrPadSpectrogramAugmentation(NeuralModule):
    """Every spectrogram of the batch gets exactly ``audio_length`` frames: longer inputs are cropped at a random offset per utterance,
    shorter ones zero-padded on both sides (the extra frame of an odd difference goes to the right).  All returned lengths equal
    ``audio_length``.  Reference: ``asr/modules/audio_preprocessing.py`` ``CropOrPadSpectrogramAugmentation``."""

    def __init__(self, audio_length: int):
        super().__init__()
        if audio_length < 0:
            raise ValueError("audio_length must be non-negative")
        self.audio_length = int(audio_length)

    @property
    def input_types(self):
        return {"input_signal": NeuralType(("B", "D", "T"), SpectrogramType()), "length": NeuralType(("B",), LengthsType())}

    @property
    def output_types(self):
        return {"processed_signal": NeuralType(("B", "D", "T"), SpectrogramType()), "processed_length": NeuralType(("B",), LengthsType())}

    @typecheck()
    @torch.no_grad()
    def forward(self, input_signal, length):
        B, _, T = input_signal.shape
        L = self.audio_length
        if T > L:
            off = torch.randint(0, T - L + 1, (B,), device=input_signal.device)
            idx = off[:, None] + torch.arange(L, device=input_signal.device)[None, :]
            out = torch.gather(input_signal, 2, idx[:, None, :].expand(-1, input_signal.shape[1], -1))
        else:
            left = (L - T) // 2
            out = torch.nn.functional.pad(input_signal, (left, L - T - left))
        return out, torch.full_like(length, L)

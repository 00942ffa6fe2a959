"""Log-mel front end on the kernels of csrc/logmel.cu."""
from __future__ import annotations

import ctypes

import torch

from . import native as N

_range_cache = {}
_seed = [0x9E3779B9]


def _fb_range(fb: torch.Tensor) -> torch.Tensor:
    key = (fb.data_ptr(), fb.device, tuple(fb.shape))
    r = _range_cache.get(key)
    if r is None:
        nz = fb.detach().cpu() != 0
        lo = nz.float().argmax(dim=1)
        hi = fb.shape[1] - nz.flip(1).float().argmax(dim=1)
        hi = torch.where(nz.any(dim=1), hi, lo)
        r = torch.stack([lo, hi], dim=1).to(torch.int32).contiguous().to(fb.device)
        _range_cache[key] = r
    return r


@torch.no_grad()
def logmel(x, seq_len, window, fb, n_fft, hop, win_length, preemph, log_zero_guard, normalize, pad_to, pad_value, dither):
    B, L = x.shape
    dev = x.device
    x = x.float().contiguous()
    seq_len = seq_len.long().contiguous()
    out_len = torch.div(seq_len + 2 * (n_fft // 2) - n_fft, hop, rounding_mode="floor")
    t_frames = 1 + L // hop
    T = t_frames
    if pad_to and pad_to > 0 and T % pad_to:
        T += pad_to - T % pad_to
    nfilt = fb.shape[0]
    out = torch.empty((B, nfilt, T), dtype=torch.float32, device=dev)
    fbc = fb.float().contiguous()
    rng = _fb_range(fbc)
    _seed[0] = (_seed[0] * 6364136223846793005 + 1442695040888963407) & ((1 << 63) - 1)
    N._check(N.lib().sb_logmel(N._ptr(x), ctypes.c_longlong(L), N._ptr(seq_len), N._ptr(out_len), N._ptr(window.float().contiguous()),
                               ctypes.c_int(win_length), N._ptr(fbc), N._ptr(rng), ctypes.c_int(nfilt), ctypes.c_int(n_fft),
                               ctypes.c_int(hop), ctypes.c_float(preemph or 0.0), ctypes.c_float(log_zero_guard),
                               ctypes.c_float(dither or 0.0), ctypes.c_ulonglong(_seed[0]),
                               ctypes.c_int(1 if normalize == "per_feature" else 0), ctypes.c_float(pad_value), N._ptr(out),
                               ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(t_frames), N._stream()), "sb_logmel")
    return out, out_len

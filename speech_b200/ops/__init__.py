"""Hot-op entry points used by the model code.

Every function here has two implementations: the hand-written sm_100a kernels in
``speech_b200/ops/csrc`` (bound through ``speech_b200.ops.native``), used for CUDA tensors, and
the plain-PyTorch statement in ``speech_b200.ops.reference``, used on the CPU and as the test
oracle.  On a machine with a GPU the kernels are mandatory: if the extension library is missing,
the first CUDA call raises instead of silently falling back to library kernels
(set ``SPEECH_B200_ALLOW_EAGER=1`` to run the eager reference math on a GPU on purpose, which is
what the ``--impl eager`` arm of the benchmark does).
"""
from __future__ import annotations

import contextlib
import os
import threading
from typing import Optional

import torch

from . import reference

_state = threading.local()


def get_compute_dtype() -> Optional[torch.dtype]:
    return getattr(_state, "dtype", None)


@contextlib.contextmanager
def compute_dtype(dtype: Optional[torch.dtype]):
    """Activations inside the block run in ``dtype`` (bf16 on GPUs); master weights stay fp32."""
    prev = getattr(_state, "dtype", None)
    _state.dtype = dtype
    try:
        yield
    finally:
        _state.dtype = prev


_env_eager = [os.environ.get("SPEECH_B200_ALLOW_EAGER", "0") == "1", 0]


def eager_allowed() -> bool:
    # the environment is re-read only every 4096 calls: this predicate runs once per op
    _env_eager[1] += 1
    if _env_eager[1] & 4095 == 1:
        _env_eager[0] = os.environ.get("SPEECH_B200_ALLOW_EAGER", "0") == "1"
    return _env_eager[0] or getattr(_state, "eager", False)


@contextlib.contextmanager
def eager_mode(enabled: bool = True):
    """Force the plain-PyTorch math even for CUDA tensors (baseline arm / debugging)."""
    prev = getattr(_state, "eager", False)
    _state.eager = enabled
    try:
        yield
    finally:
        _state.eager = prev


_native = None
_native_err: Optional[BaseException] = None


def _nat():
    """The ctypes binding module, loaded on first use."""
    global _native, _native_err
    if _native is None and _native_err is None:
        try:
            from . import native as _n  # noqa: F811

            _n.load()
            _native = _n
        except BaseException as e:  # noqa: BLE001
            _native_err = e
    if _native is None:
        raise RuntimeError(
            "speech_b200 native kernels are not available "
            f"({_native_err!r}). Build them with `python -m speech_b200.ops.build` "
            "or set SPEECH_B200_ALLOW_EAGER=1 to run the eager reference math."
        )
    return _native


def native_available() -> bool:
    try:
        _nat()
        return True
    except RuntimeError:
        return False


def _use_native(t: torch.Tensor) -> bool:
    if not t.is_cuda or eager_allowed():
        return False
    _nat()  # raises loudly when the library is missing on a GPU machine
    return True


def lowp(param: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Working copy of a master weight in the compute dtype (the optimizer arena keeps one up to date)."""
    dtype = dtype or get_compute_dtype()
    if dtype is None or param.dtype == dtype:
        return param
    lp = getattr(param, "_lowp", None)
    if lp is not None and lp.dtype == dtype and lp.device == param.device:
        return lp
    cache = getattr(param, "_lowp_cache", None)
    if cache is not None and cache[0] == param._version and cache[1].dtype == dtype and cache[1].device == param.device:
        return cache[1]
    t = param.detach().to(dtype)
    try:
        param._lowp_cache = (param._version, t)
    except Exception:
        pass
    return t


# ----------------------------------------------------------------------------- augmentation / LM fusion
def specaugment(x, f_start, f_width, t_start, t_width, mask_value: float = 0.0):
    """Copy of ``x`` [B, F, T] with the frequency rows ``[f_start, f_start + f_width)`` and the time ranges
    ``[t_start, t_start + t_width)`` of every utterance set to ``mask_value`` (start / width: integer [B, n] or None)."""
    if _use_native(x) and x.dtype in (torch.float32, torch.bfloat16) and (t_start is None or t_start.shape[1] <= 32):
        i32 = lambda t: None if t is None else t.to(torch.int32).contiguous()  # noqa: E731
        return _nat().specaugment_(x.clone(memory_format=torch.contiguous_format), i32(f_start), i32(f_width), i32(t_start),
                                   i32(t_width), mask_value)
    return reference.specaugment(x, f_start, f_width, t_start, t_width, mask_value)


def ngram_advance(states, arc_keys, arc_w, arc_to, backoff_w, backoff_to, V: int, depth: int, default_score: float, start_state: int):
    if _use_native(states) and depth <= 16:
        return _nat().ngram_advance(states.contiguous(), arc_keys, arc_w, arc_to, backoff_w, backoff_to, V, depth, default_score,
                                    start_state)
    return reference.ngram_advance(states, arc_keys, arc_w, arc_to, backoff_w, backoff_to, V, depth, default_score, start_state)


# ----------------------------------------------------------------------------- dense layers
def linear(x, weight, bias=None, act: Optional[str] = None, residual=None, alpha: float = 1.0, dropout_p: float = 0.0):
    """``residual + alpha * dropout(act(x W^T + b))``; ``dropout_p`` > 0 means "apply dropout now" (callers pass 0 in eval)."""
    if _use_native(x) and x.dtype == torch.bfloat16:
        return _nat().linear(x, weight, bias, act, residual, alpha, dropout_p)
    return reference.linear(x, weight, bias, act, residual, alpha, dropout_p)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if _use_native(x) and x.dtype == torch.bfloat16:
        return _nat().layer_norm(x, weight, bias, eps)
    return reference.layer_norm(x, weight, bias, eps)


def relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask=None, dropout_p: float = 0.0, training: bool = False,
                     qkv=None):
    if _use_native(q) and q.dtype == torch.bfloat16:
        return _nat().relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask, dropout_p, training, qkv=qkv)
    return reference.relpos_attention(q, k, v, p, pos_bias_u, pos_bias_v, mask, dropout_p, training)


def mha_attention(q, k, v, mask=None, dropout_p: float = 0.0, training: bool = False, scale=None):
    if _use_native(q) and q.dtype == torch.bfloat16:
        return _nat().mha_attention(q, k, v, mask, scale, dropout_p, training)
    return reference.mha_attention(q, k, v, mask, dropout_p, training, scale)


def conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean, running_var,
                     pad_mask=None, training=False, momentum=0.1, eps=1e-5, left_pad=4, right_pad=4, cache=None,
                     cache_drop_size=0, bn_stats_reduce=None):
    if _use_native(g) and g.dtype == torch.bfloat16 and cache is None and norm_type in ("batch_norm", "layer_norm"):
        return _nat().conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean,
                                         running_var, pad_mask, training, momentum, eps, left_pad, right_pad,
                                         bn_stats_reduce)
    return reference.conv_module_core(g, dw_weight, dw_bias, norm_type, norm_weight, norm_bias, running_mean,
                                      running_var, pad_mask, training, momentum, eps, left_pad, right_pad, cache,
                                      cache_drop_size, bn_stats_reduce)


def conformer_layer(layer, x, att_mask=None, pos_emb=None, pad_mask=None):
    """Whole Conformer layer (forward and backward each issued by one native call); ``None`` when the layer's configuration
    or this call is outside the executor's envelope and the caller should run the per-op path."""
    if not _use_native(x) or x.dtype != torch.bfloat16:
        return None
    from . import native_layer

    return native_layer.conformer_layer(layer, x, att_mask, pos_emb, pad_mask)


def lstm(x, weights, h0=None, c0=None, num_layers=1, dropout=0.0, training=False):
    if _use_native(x) and x.dtype == torch.bfloat16 and not (dropout > 0 and training) and hasattr(_nat(), "lstm"):
        return _nat().lstm(x, weights, h0, c0, num_layers)
    return reference.lstm(x, weights, h0, c0, num_layers, dropout, training)


# ----------------------------------------------------------------------------- losses
def transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank, durations, sigma, act="relu",
                          fastemit_lambda=0.0, sub_batch=0, dropout_p: float = 0.0):
    if _use_native(f) and f.dtype == torch.bfloat16 and act == "relu":
        return _nat().transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank, durations, sigma,
                                              fastemit_lambda, dropout_p)
    return reference.transducer_joint_loss(f, g, w, b, targets, f_len, y_len, blank, durations, sigma, act,
                                           fastemit_lambda, sub_batch, dropout_p=dropout_p)


def transducer_loss_from_logits(logits, targets, f_len, y_len, blank, durations, sigma=0.0):
    if _use_native(logits):
        return _nat().transducer_loss_from_logits(logits, targets, f_len, y_len, blank, durations, sigma)
    return reference.tdt_loss_from_logits(logits, targets, f_len, y_len, blank, durations, sigma)


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank, zero_infinity=True):
    if _use_native(log_probs) and hasattr(_nat(), "ctc_loss"):
        return _nat().ctc_loss(log_probs, targets, input_lengths, target_lengths, blank)
    return reference.ctc_loss(log_probs, targets, input_lengths, target_lengths, blank, zero_infinity)


# ----------------------------------------------------------------------------- front-end
def logmel(x, seq_len, window, fb, n_fft, hop, win_length, preemph=0.97, mag_power=2.0, log_zero_guard=2 ** -24,
           normalize="per_feature", pad_to=0, pad_value=0.0, dither=0.0, log=True):
    if _use_native(x) and normalize in ("per_feature", None) and mag_power == 2.0 and log and n_fft == 512 and hasattr(_nat(), "logmel"):
        return _nat().logmel(x, seq_len, window, fb, n_fft, hop, win_length, preemph, log_zero_guard,
                               normalize, pad_to, pad_value, dither)
    return reference.logmel(x, seq_len, window, fb, n_fft, hop, win_length, preemph, mag_power, log_zero_guard,
                            normalize, pad_to, pad_value, dither, log=log)


# ----------------------------------------------------------------------------- optimizer
def adamw_flat(master, grad, exp_avg, exp_avg_sq, lowp, lr, beta1, beta2, eps, weight_decay, step, scalars):
    """One fused AdamW pass; ``scalars[1]`` (device memory) holds the gradient multiplier (clip x scale)."""
    if _use_native(master):
        return _nat().adamw_flat(master, grad, exp_avg, exp_avg_sq, lowp, lr, beta1, beta2, eps, weight_decay, step,
                                   scalars)
    return reference.adamw_flat(master, grad, exp_avg, exp_avg_sq, lowp, lr, beta1, beta2, eps, weight_decay, step,
                                clip_coef=scalars[1])


def grad_norm_clip_coef(flat_grad, scalars, max_norm: float, grad_scale: float = 1.0):
    """scalars[0] <- ||grad * grad_scale||_2, scalars[1] <- grad_scale * min(1, max_norm / (norm + 1e-6))."""
    if _use_native(flat_grad):
        return _nat().grad_norm_clip_coef(flat_grad, scalars, max_norm, grad_scale)
    norm = flat_grad.float().norm() * grad_scale
    scalars[0] = norm
    scalars[1] = grad_scale * torch.clamp(max_norm / (norm + 1e-6), max=1.0)


from . import native  # noqa: E402,F401  (binding module; the shared library itself is loaded on first use)

"""Whole-layer execution of a Conformer layer: one native call per layer for the forward pass and one for the backward pass.

``csrc/conformer_layer.cu`` sequences every kernel of the layer on the current stream; this module marshals the layer's
parameters into its argument block once (weights live in the optimizer arena, so their addresses are stable), manages the
activation buffer that the backward pass reads, and exposes the pair as a ``torch.autograd.Function``.  Parameter gradients
are accumulated by the kernels straight into the arena's flat gradient buffer; the data-parallel engine is told when a
layer's gradients are final.

The per-op path (``ops.linear`` / ``ops.layer_norm`` / ``ops.relpos_attention`` / ``ops.conv_module_core``) computes the same
function and stays the fallback for every configuration outside the executor's envelope (streaming caches, adapters, local
attention, non-BatchNorm convolution norms, synchronised BatchNorm, frozen parameters).
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Dict, List, Optional, Tuple

import torch

from . import native as N
from . import native_blocks as NB

_vp, _f, _i, _ll, _u64 = ctypes.c_void_p, ctypes.c_float, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong


class SbLinearParams(ctypes.Structure):
    _fields_ = [("w", _vp), ("b", _vp), ("gw", _vp), ("gb", _vp)]


class SbNormParams(ctypes.Structure):
    _fields_ = [("w", _vp), ("b", _vp), ("gw", _vp), ("gb", _vp), ("eps", _f), ("pad_", _i)]


class SbConformerLayerArgs(ctypes.Structure):
    _fields_ = [
        ("B", _i), ("T", _i), ("P", _i), ("d", _i), ("dff", _i), ("H", _i), ("conv_k", _i), ("conv_left", _i),
        ("training", _i), ("fc_factor", _f), ("drop_ff", _f), ("drop_att", _f), ("drop_out", _f), ("bn_eps", _f), ("bn_momentum", _f),
        ("seeds", _u64 * 7),
        ("x", _vp), ("pos_emb", _vp), ("att_mask", _vp), ("att_mask_bstride", _i), ("launches", _i), ("pad_mask", _vp),
        ("ln_ff1", SbNormParams), ("ln_att", SbNormParams), ("ln_conv", SbNormParams), ("ln_ff2", SbNormParams), ("ln_out", SbNormParams),
        ("ff1a", SbLinearParams), ("ff1b", SbLinearParams), ("qkv", SbLinearParams), ("pos", SbLinearParams),
        ("out_proj", SbLinearParams), ("pw1", SbLinearParams), ("pw2", SbLinearParams), ("ff2a", SbLinearParams), ("ff2b", SbLinearParams),
        ("pos_u", _vp), ("pos_v", _vp), ("g_pos_u", _vp), ("g_pos_v", _vp),
        ("dw_w", _vp), ("dw_b", _vp), ("g_dw_w", _vp), ("g_dw_b", _vp),
        ("bn_w", _vp), ("bn_b", _vp), ("g_bn_w", _vp), ("g_bn_b", _vp), ("bn_mean", _vp), ("bn_var", _vp),
        ("out", _vp), ("saved", _vp), ("saved_bytes", _ll), ("scratch", _vp), ("scratch_bytes", _ll),
        ("dout", _vp), ("dx", _vp),
        ("sync_buffers", _vp), ("sync_base_off", _ll), ("sync_rank", _i), ("sync_world", _i), ("sync_epoch", ctypes.c_uint), ("pad2_", _i),
        ("prof_ms", ctypes.POINTER(_f)), ("prof_cap", _i), ("pad_", _i),
    ]


_checked_abi = [False]


def _lib():
    lib = N.lib()
    if not _checked_abi[0]:
        n = int(lib.sb_conformer_layer_args_size())
        if n != ctypes.sizeof(SbConformerLayerArgs):
            raise RuntimeError(f"conformer layer argument block: library has {n} bytes, bindings {ctypes.sizeof(SbConformerLayerArgs)}")
        _checked_abi[0] = True
    return lib


def enabled() -> bool:
    return os.environ.get("SPEECH_B200_LAYER_EXECUTOR", "1") != "0"


# ------------------------------------------------------------------------------------------------ small caches
class _ConvertCache:
    """Last few conversions of step-constant tensors (masks, positional table) keyed by tensor identity and version."""

    def __init__(self, n: int = 4):
        self.items: List[Tuple[weakref.ref, int, torch.Tensor]] = []
        self.n = n

    def get(self, t: torch.Tensor, fn):
        for ref, ver, out in self.items:
            if ref() is t and ver == t._version:
                return out
        out = fn(t)
        self.items.append((weakref.ref(t), t._version, out))
        if len(self.items) > self.n:
            self.items.pop(0)
        return out


profile_sink: Optional[list] = None   # set to a list to collect (phase, [(label, ms), ...]) for every executor call
_PROF_CAP = 160


def _prof_begin(a):
    if profile_sink is None:
        a.prof_ms, a.prof_cap = None, 0
        return None
    buf = (_f * _PROF_CAP)()
    a.prof_ms, a.prof_cap = ctypes.cast(buf, ctypes.POINTER(_f)), _PROF_CAP
    return buf


def _prof_end(phase: str, a, buf):
    if buf is None:
        return
    name = _lib().sb_conformer_layer_prof_name
    name.restype = ctypes.c_char_p
    profile_sink.append((phase, [(name(i).decode(), float(buf[i])) for i in range(min(a.launches, _PROF_CAP))]))


_masks = _ConvertCache()
_packs: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()   # layer -> _Pack (kept off the module so it deep-copies / pickles)
_scratch: Dict[torch.device, torch.Tensor] = {}
_sizes: Dict[Tuple, Tuple[int, int, int]] = {}


def _scratch_for(dev: torch.device, nbytes: int) -> torch.Tensor:
    buf = _scratch.get(dev)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes * 1.25) + 4096, dtype=torch.uint8, device=dev)
        _scratch[dev] = buf
    return buf


# ------------------------------------------------------------------------------------------------ parameter block
def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _grad_ptr(p: Optional[torch.Tensor], need: bool) -> Optional[int]:
    if p is None or not need:
        return None
    return p._grad_view.data_ptr()


def _linear(weight, bias, need: bool, keep: list) -> SbLinearParams:
    wl = N._lowp_weight(weight)
    keep.append(wl)
    return SbLinearParams(wl.data_ptr(), _ptr(bias), _grad_ptr(weight, need), _grad_ptr(bias, need))


def _norm(ln, need: bool) -> SbNormParams:
    return SbNormParams(ln.weight.data_ptr(), _ptr(ln.bias), _grad_ptr(ln.weight, need), _grad_ptr(ln.bias, need), float(ln.eps), 0)


def _static_ok(layer) -> bool:
    """Configuration checks that do not depend on the batch."""
    from ..modules.attention import RelPositionMultiHeadAttention, RelPositionMultiHeadAttentionLongformer
    from ..modules.attention import fused_qkv_weight  # noqa: F401

    att, conv = layer.self_attn, layer.conv
    if layer.self_attention_model != "rel_pos" or not isinstance(att, RelPositionMultiHeadAttention) \
            or isinstance(att, RelPositionMultiHeadAttentionLongformer):
        return False
    if conv.norm_type != "batch_norm" or conv.pointwise_activation != "glu_" or conv.kernel_size not in (5, 9, 15):
        return False
    dw = conv.depthwise_conv
    if dw._left_padding + dw._right_padding != conv.kernel_size - 1:
        return False
    d = layer.norm_out.weight.shape[0]
    if d % 8 or (d // att.h) % 8 or layer.feed_forward1.d_ff % 8 or d > 5632:
        return False
    for ln in (layer.norm_feed_forward1, layer.norm_self_att, layer.norm_conv, layer.norm_feed_forward2, layer.norm_out):
        if ln.weight is None or ln.bias is None or ln.weight.dtype != torch.float32:
            return False
    if not isinstance(layer.feed_forward1.activation, torch.nn.SiLU) or not isinstance(layer.feed_forward2.activation, torch.nn.SiLU):
        return False
    bn = conv.batch_norm
    if bn.weight is None or bn.running_mean is None or bn.momentum is None:
        return False
    return True


class _Pack:
    """Argument block of one layer with every parameter address filled in, plus what keeps those addresses alive."""

    def __init__(self, layer, need_grad: bool):
        from ..modules.attention import fused_qkv_weight

        att, conv, keep = layer.self_attn, layer.conv, []
        fused = fused_qkv_weight(att)
        if fused is None:
            raise _Unsupported("q/k/v weights are not adjacent in the optimizer arena")
        wqkv, bqkv = fused
        a = SbConformerLayerArgs()
        a.d, a.dff, a.H = layer.norm_out.weight.shape[0], layer.feed_forward1.d_ff, att.h
        a.conv_k, a.conv_left = conv.kernel_size, conv.depthwise_conv._left_padding
        a.fc_factor = float(layer.fc_factor)
        a.ln_ff1, a.ln_att = _norm(layer.norm_feed_forward1, need_grad), _norm(layer.norm_self_att, need_grad)
        a.ln_conv, a.ln_ff2 = _norm(layer.norm_conv, need_grad), _norm(layer.norm_feed_forward2, need_grad)
        a.ln_out = _norm(layer.norm_out, need_grad)
        f1, f2 = layer.feed_forward1, layer.feed_forward2
        a.ff1a, a.ff1b = _linear(f1.linear1.weight, f1.linear1.bias, need_grad, keep), _linear(f1.linear2.weight, f1.linear2.bias, need_grad, keep)
        a.ff2a, a.ff2b = _linear(f2.linear1.weight, f2.linear1.bias, need_grad, keep), _linear(f2.linear2.weight, f2.linear2.bias, need_grad, keep)
        a.qkv = _linear(wqkv, bqkv, need_grad, keep)
        a.pos = _linear(att.linear_pos.weight, None, need_grad, keep)
        a.out_proj = _linear(att.linear_out.weight, att.linear_out.bias, need_grad, keep)
        a.pw1 = _linear(conv.pointwise_conv1.weight, conv.pointwise_conv1.bias, need_grad, keep)
        a.pw2 = _linear(conv.pointwise_conv2.weight, conv.pointwise_conv2.bias, need_grad, keep)
        a.pos_u, a.pos_v = att.pos_bias_u.data_ptr(), att.pos_bias_v.data_ptr()
        a.g_pos_u, a.g_pos_v = _grad_ptr(att.pos_bias_u, need_grad), _grad_ptr(att.pos_bias_v, need_grad)
        dw, bn = conv.depthwise_conv, conv.batch_norm
        if not dw.weight.is_contiguous():
            raise _Unsupported("depthwise weight is not contiguous")
        a.dw_w, a.dw_b = dw.weight.data_ptr(), _ptr(dw.bias)
        a.g_dw_w, a.g_dw_b = _grad_ptr(dw.weight, need_grad), _grad_ptr(dw.bias, need_grad)
        a.bn_w, a.bn_b = bn.weight.data_ptr(), bn.bias.data_ptr()
        a.g_bn_w, a.g_bn_b = _grad_ptr(bn.weight, need_grad), _grad_ptr(bn.bias, need_grad)
        a.bn_mean, a.bn_var = bn.running_mean.data_ptr(), bn.running_var.data_ptr()
        a.bn_eps, a.bn_momentum = float(bn.eps), float(bn.momentum)
        self.args, self.keep = a, keep
        self.params = [p for p in layer.parameters()]
        self.fused = (wqkv, bqkv)
        self.key = _pack_key(layer, need_grad)


class _Unsupported(Exception):
    pass


def _pack_key(layer, need_grad: bool):
    w = layer.norm_out.weight
    arena = getattr(w, "_arena", None)
    lp = getattr(layer.feed_forward1.linear1.weight, "_lowp", None)
    return (id(arena), w.data_ptr(), None if lp is None else lp.data_ptr(), need_grad, layer.conv.batch_norm.running_mean.data_ptr())


def _get_pack(layer, need_grad: bool) -> Optional[_Pack]:
    pack = _packs.get(layer)
    if pack is not None and pack.key == _pack_key(layer, need_grad):
        return pack
    if need_grad:
        for p in layer.parameters():
            gv = getattr(p, "_grad_view", None)
            if not p.requires_grad or gv is None or not gv.is_cuda:
                return None
    if getattr(layer.feed_forward1.linear1.weight, "_lowp", None) is None:
        return None       # weights outside an arena: their bf16 copies are version-cached tensors whose addresses may change
    try:
        pack = _Pack(layer, need_grad)
    except _Unsupported:
        return None
    _packs[layer] = pack
    return pack


# ------------------------------------------------------------------------------------------------ autograd function
def _sizes_for(a: SbConformerLayerArgs) -> Tuple[int, int, int]:
    key = (a.B, a.T, a.d, a.dff, a.H, a.training, a.drop_att > 0.0)
    s = _sizes.get(key)
    if s is None:
        sv, fs, bs = _ll(0), _ll(0), _ll(0)
        rc = _lib().sb_conformer_layer_sizes(ctypes.byref(a), ctypes.byref(sv), ctypes.byref(fs), ctypes.byref(bs))
        if rc != 0:
            raise RuntimeError(f"sb_conformer_layer_sizes failed with code {rc}")
        s = (sv.value, fs.value, bs.value)
        _sizes[key] = s
    return s


def _set_sync(a, sync) -> None:
    """Synchronised BatchNorm: hand the executor the peer buffers and this call's epoch (one per call, same on all ranks)."""
    if sync is None or not a.training:
        a.sync_buffers, a.sync_world, a.sync_epoch = None, 0, 0
        return
    a.sync_buffers, a.sync_base_off = sync.ptrs_dev, 0
    a.sync_rank, a.sync_world, a.sync_epoch = sync.rank, sync.world, sync.next_epoch()


class _ConformerLayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, pack, dyn):
        a: SbConformerLayerArgs = pack.args
        B, T, d = x.shape
        pos, m8, mbs, pad8, training, drops, seeds, sync = dyn
        a.B, a.T, a.P = B, T, pos.shape[0]
        a.training = int(training)
        a.drop_ff, a.drop_att, a.drop_out = drops
        for i, s in enumerate(seeds):
            a.seeds[i] = s
        a.x, a.pos_emb = x.data_ptr(), pos.data_ptr()
        a.att_mask, a.att_mask_bstride, a.pad_mask = _ptr(m8), mbs, _ptr(pad8)
        _set_sync(a, sync)
        sv, fs, bs = _sizes_for(a)
        saved = torch.empty(sv, dtype=torch.uint8, device=x.device)
        scratch = _scratch_for(x.device, max(fs, bs))
        out = torch.empty((B, T, d), dtype=torch.bfloat16, device=x.device)
        a.out, a.saved, a.saved_bytes = out.data_ptr(), saved.data_ptr(), sv
        a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
        a.dout = a.dx = None
        prof = _prof_begin(a)
        rc = _lib().sb_conformer_layer_fwd(ctypes.byref(a), N._stream())
        _prof_end("forward", a, prof)
        N.launch_count += a.launches
        if rc != 0:
            raise RuntimeError(f"sb_conformer_layer_fwd failed with code {rc} (step {(-rc) // 1000}, code {(-rc) % 1000})")
        ctx.pack, ctx.saved_buf, ctx.dyn = pack, saved, dyn
        ctx.save_for_backward(x)
        ctx.dims = (B, T, d)
        return out

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        pack = ctx.pack
        a: SbConformerLayerArgs = pack.args
        B, T, d = ctx.dims
        pos, m8, mbs, pad8, training, drops, seeds, sync = ctx.dyn
        a.B, a.T, a.P = B, T, pos.shape[0]
        a.training = int(training)
        a.drop_ff, a.drop_att, a.drop_out = drops
        for i, s in enumerate(seeds):
            a.seeds[i] = s
        a.x, a.pos_emb = x.data_ptr(), pos.data_ptr()
        a.att_mask, a.att_mask_bstride, a.pad_mask = _ptr(m8), mbs, _ptr(pad8)
        _set_sync(a, sync)
        sv, fs, bs = _sizes_for(a)
        scratch = _scratch_for(x.device, max(fs, bs))
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dx = torch.empty((B, T, d), dtype=torch.bfloat16, device=x.device) if ctx.needs_input_grad[0] else None
        a.saved, a.saved_bytes = ctx.saved_buf.data_ptr(), sv
        a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
        a.dout, a.dx, a.out = dout.data_ptr(), _ptr(dx), None
        prof = _prof_begin(a)
        rc = _lib().sb_conformer_layer_bwd(ctypes.byref(a), N._stream())
        _prof_end("backward", a, prof)
        N.launch_count += a.launches
        if rc != 0:
            raise RuntimeError(f"sb_conformer_layer_bwd failed with code {rc} (step {(-rc) // 1000}, code {(-rc) % 1000})")
        arena = getattr(pack.params[0], "_arena", None)
        cb = getattr(arena, "grad_ready", None) if arena is not None else None
        if cb is not None:
            for p in pack.params:
                cb(p)
        return dx, None, None, None


def conformer_layer(layer, x: torch.Tensor, att_mask, pos_emb, pad_mask) -> Optional[torch.Tensor]:
    """Run ``layer`` through the native executor; ``None`` when this call is outside its envelope (the caller then uses the
    per-op path)."""
    if not enabled() or not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 3:
        return None
    ok = getattr(layer, "_exec_static_ok", None)
    if ok is None:
        ok = layer._exec_static_ok = _static_ok(layer)
    if not ok or pos_emb is None or pos_emb.shape[0] != 1:
        return None
    sync = None
    if layer.conv.bn_stats_reduce is not None:
        # synchronised BatchNorm: only with the peer-memory reducer, which the executor can call between its kernels
        sync = getattr(layer.conv, "bn_peer_sync", None)
        if sync is None or 2 * x.shape[2] + 1 > sync.max_elems:
            return None
    B, T, d = x.shape
    if pos_emb.shape[1] != 2 * T - 1 or B * T == 0:
        return None
    training = layer.training
    cached = _packs.get(layer)
    params = cached.params if cached is not None else list(layer.parameters())   # walking the module tree costs ~50 us
    trainable = sum(1 for p in params if p.requires_grad)
    need_grad = torch.is_grad_enabled() and (x.requires_grad or trainable > 0)
    if need_grad and trainable != len(params):
        return None
    pack = _get_pack(layer, need_grad)
    if pack is None:
        return None
    if att_mask is not None:
        m = att_mask[:, 0] if att_mask.dim() == 4 else att_mask
        if m.shape[-2:] != (T, T) or m.shape[0] not in (1, B):
            return None
        m8 = _masks.get(att_mask, lambda t: (t[:, 0] if t.dim() == 4 else t).to(torch.uint8).contiguous())
        mbs = T if m8.shape[0] > 1 else 0
    else:
        m8, mbs = None, 0
    pad8 = _masks.get(pad_mask, lambda t: t.to(torch.uint8).contiguous()) if pad_mask is not None else None
    pos = _masks.get(pos_emb, lambda t: t[0].to(torch.bfloat16).contiguous())
    p_ff = float(layer.feed_forward1.dropout.p) if training else 0.0
    p_att = float(layer.self_attn.dropout_rate) if training else 0.0
    p_out = float(layer.dropout.p) if training else 0.0
    nd, ns = N._next_dropout_seed, NB._next_seed
    seeds = (nd() if p_ff > 0 else 0, nd() if p_ff > 0 else 0, ns() if p_att > 0 else 0, nd() if p_out > 0 else 0,
             nd() if p_out > 0 else 0, nd() if p_ff > 0 else 0, nd() if p_ff > 0 else 0)
    xc = x if x.is_contiguous() else x.contiguous()
    dyn = (pos, m8, mbs, pad8, training, (p_ff, p_att, p_out), seeds, sync)
    if need_grad:
        out = _ConformerLayerFn.apply(xc, layer.norm_out.weight, pack, dyn)
    else:
        with torch.no_grad():
            out = _ConformerLayerFn.apply(xc, layer.norm_out.weight, pack, dyn)
    bn = layer.conv.batch_norm
    if training and bn.num_batches_tracked is not None:
        bn.num_batches_tracked += 1
    return out

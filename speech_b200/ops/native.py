"""ctypes bindings and autograd wrappers for the sm_100a kernel library.

The library (``libspeech_b200.so``, built by ``python -m speech_b200.ops.build``) exposes plain C entry points
that take raw device pointers, sizes and a CUDA stream.  This module turns tensors into those arguments, launches
on the current PyTorch stream and wraps each op in a ``torch.autograd.Function`` whose backward is again made
of the library's kernels.

Parameter gradients are written by the weight-gradient GEMM *directly into the optimizer arena's flat gradient
buffer* (``param._grad_view``) — no autograd accumulation pass — and the data-parallel engine is told the
gradient is final (``param._arena.grad_ready``).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Any, List, Optional, Sequence, Tuple

import torch

_LIB = None
_LIB_PATH = os.environ.get("SPEECH_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libspeech_b200.so")
launch_count = 0  # number of kernel-launching library calls (benchmarks report it)
_SMALL_M_SPLITK = os.environ.get("SPEECH_B200_SMALL_M_SPLITK", "1") != "0"


class SbGemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("a_mn_major", ctypes.c_int), ("b_mn_major", ctypes.c_int), ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong),
        ("batch0", ctypes.c_int), ("batch1", ctypes.c_int),
        ("a_bs0", ctypes.c_longlong), ("a_bs1", ctypes.c_longlong), ("b_bs0", ctypes.c_longlong), ("b_bs1", ctypes.c_longlong),
        ("D", ctypes.c_void_p), ("d_is_f32", ctypes.c_int), ("ldd", ctypes.c_longlong), ("d_bs0", ctypes.c_longlong),
        ("d_bs1", ctypes.c_longlong),
        ("bias", ctypes.c_void_p), ("bias_is_f32", ctypes.c_int),
        ("residual", ctypes.c_void_p), ("ldr", ctypes.c_longlong), ("r_bs0", ctypes.c_longlong), ("r_bs1", ctypes.c_longlong),
        ("aux", ctypes.c_void_p), ("ldx", ctypes.c_longlong), ("x_bs0", ctypes.c_longlong), ("x_bs1", ctypes.c_longlong),
        ("D_pre", ctypes.c_void_p), ("ldp", ctypes.c_longlong), ("p_bs0", ctypes.c_longlong), ("p_bs1", ctypes.c_longlong),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("act", ctypes.c_int), ("dact", ctypes.c_int),
        ("max_ctas", ctypes.c_int), ("fold_batch1", ctypes.c_int), ("tile_n", ctypes.c_int),
        ("drop_p", ctypes.c_float), ("drop_seed", ctypes.c_ulonglong), ("ksplit", ctypes.c_int), ("pad_", ctypes.c_int), ("peer_D", ctypes.c_void_p), ("peer_rows", ctypes.c_int), ("pad2_", ctypes.c_int), ("peer_A", ctypes.c_void_p), ("peer_a_rows", ctypes.c_int), ("peer_world", ctypes.c_int), ("pair", ctypes.c_int),
        ("sig_flags", ctypes.c_void_p), ("sig_counter", ctypes.c_void_p), ("sig_world", ctypes.c_int), ("sig_rank", ctypes.c_int),
        ("sig_epoch", ctypes.c_uint), ("sig_head", ctypes.c_int), ("sig_tail", ctypes.c_int), ("pad3_", ctypes.c_int),
        ("stage_src", ctypes.c_void_p), ("stage_dst", ctypes.c_void_p), ("stage_bytes", ctypes.c_longlong), ("stage_counter", ctypes.c_void_p),
        ("splitk_ws", ctypes.c_void_p), ("splitk_ws_bytes", ctypes.c_longlong),
    ]


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        raise FileNotFoundError(f"{_LIB_PATH} not found; run `python -m speech_b200.ops.build`")
    lib = ctypes.CDLL(_LIB_PATH)
    for name in dir(lib):
        pass
    lib.sb_status_string.restype = ctypes.c_char_p
    lib.sb_status_ptr.restype = ctypes.c_void_p
    _LIB = lib
    return lib


def lib():
    return _LIB if _LIB is not None else load()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_cur_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream(t: Optional[torch.Tensor] = None) -> ctypes.c_void_p:
    """Handle of the current CUDA stream of the current device (one C call; this runs once per kernel launch)."""
    if _raw_stream is not None and _cur_device is not None:
        return ctypes.c_void_p(_raw_stream(_cur_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"speech_b200 native call {what} failed with code {rc}")


def check_status(clear: bool = True) -> None:
    """Read the device status word (synchronises the current stream); raise if a kernel reported a failure."""
    out = (ctypes.c_int * 4)()
    rc = lib().sb_read_status(out, ctypes.c_int(1 if clear else 0), _stream())
    if rc != 0:
        raise RuntimeError(f"could not read the kernel status word (cuda error {rc})")
    if out[0] != 0:
        msg = lib().sb_status_string(out[0]).decode()
        raise RuntimeError(f"a speech_b200 kernel reported status {out[0]} ({msg}) in block {out[1]}, detail {out[2]}")


def status_message(code: int) -> str:
    return lib().sb_status_string(int(code)).decode()


def set_wait_seconds(seconds: float, clock_hz: float = 2.0e9) -> None:
    """Limit of every bounded in-kernel wait on the current device (0 restores the default of about a second)."""
    lib().sb_set_wait_cycles.argtypes = [ctypes.c_longlong]
    rc = lib().sb_set_wait_cycles(ctypes.c_longlong(int(max(0.0, seconds) * clock_hz)))
    if rc != 0:
        raise RuntimeError(f"sb_set_wait_cycles failed with code {rc}")


class StatusProbe:
    """Non-blocking view of the device status word: ``record()`` enqueues a copy of the word into pinned memory on the current
    stream, ``poll()`` returns the code of the last completed copy (0 = ok) without waiting for the device."""

    def __init__(self, device: torch.device):
        self.host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None
        self.device = device

    def record(self) -> None:
        rc = lib().sb_status_copy_async(ctypes.c_void_p(self.host.data_ptr()), _stream())
        if rc != 0:
            raise RuntimeError(f"sb_status_copy_async failed with code {rc}")
        self.event = torch.cuda.Event()
        self.event.record()

    def poll(self, wait: bool = False) -> int:
        if self.event is None:
            return 0
        if wait:
            self.event.synchronize()
        elif not self.event.query():
            return 0
        return int(self.host[0])


ACT = {None: 0, "none": 0, "relu": 1, "swish": 2, "silu": 2, "gelu": 3}


# ------------------------------------------------------------------------------------------------ raw GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, M: int, N: int, K: int, a_mn: bool = False, b_mn: bool = False,
         lda: Optional[int] = None, ldb: Optional[int] = None, ldd: Optional[int] = None, batch: Tuple[int, int] = (1, 1),
         a_bs: Tuple[int, int] = (0, 0), b_bs: Tuple[int, int] = (0, 0), d_bs: Tuple[int, int] = (0, 0),
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
         ldr: Optional[int] = None, r_bs: Tuple[int, int] = (0, 0), aux: Optional[torch.Tensor] = None, dact: Optional[str] = None,
         ldx: Optional[int] = None, x_bs: Tuple[int, int] = (0, 0), out_pre: Optional[torch.Tensor] = None,
         ldp: Optional[int] = None, p_bs: Tuple[int, int] = (0, 0), alpha: float = 1.0, beta: float = 0.0,
         max_ctas: int = 0, fold_batch1: bool = False, tile_n: int = 0, drop_p: float = 0.0, drop_seed: int = 0,
         ksplit: int = 0, pair: int = 0, peer_out: int = 0, peer_rows: int = 0, peer_a=None, peer_a_rows: int = 0,
         sig: Optional[Tuple[int, int, int, int, int, int, int]] = None,
         stage: Optional[Tuple[int, int, int, int]] = None) -> torch.Tensor:
    """``out = epilogue(alpha * A @ B^T)`` on raw strided bf16 operands (see csrc/gemm_tcgen05.cu).

    ``sig`` = (flag table pointer, counter pointer, world, rank, epoch, head, tail): rank synchronisation inside the kernel for
    the fused collectives (``parallel/fused.py``); ``stage`` = (device table of the ranks' shard addresses, local staging area,
    bytes per shard, counter words): remote shards are copied once into local memory by the kernel's own blocks.

    ``a_mn`` / ``b_mn``: the operand is stored transposed (A as [K, M], B as [K, N]).  ``lda`` / ``ldb`` are the row
    strides of the *stored* matrices, in elements (multiples of 8).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "GEMM operands must be bf16"
    assert out.dtype in (torch.float32, torch.bfloat16)
    # few output tiles and a long K (inference on a few hundred tokens): hand the kernel an fp32 scratch so that it can split K
    ws = None
    if (M <= 1024 and K >= 768 and ksplit == 0 and out.dtype == torch.bfloat16 and batch == (1, 1) and aux is None and drop_p <= 0.0
            and beta == 0.0 and peer_a is None and not peer_out and M * N <= (4 << 20) and _SMALL_M_SPLITK):
        ws = torch.empty(M * N, dtype=torch.float32, device=out.device)
    # one positional constructor call: field-by-field assignment through ctypes descriptors costs several microseconds
    g = SbGemmArgs(
        a.data_ptr(), b.data_ptr(), M, N, K, int(a_mn), int(b_mn),
        lda if lda is not None else (M if a_mn else K), ldb if ldb is not None else (N if b_mn else K),
        batch[0], batch[1], a_bs[0], a_bs[1], b_bs[0], b_bs[1],
        out.data_ptr(), int(out.dtype == torch.float32), ldd if ldd is not None else N, d_bs[0], d_bs[1],
        bias.data_ptr() if bias is not None else None, int(bias is not None and bias.dtype == torch.float32),
        residual.data_ptr() if residual is not None else None, (ldr if ldr is not None else N) if residual is not None else 0,
        r_bs[0], r_bs[1],
        aux.data_ptr() if aux is not None else None, (ldx if ldx is not None else N) if aux is not None else 0, x_bs[0], x_bs[1],
        out_pre.data_ptr() if out_pre is not None else None, (ldp if ldp is not None else N) if out_pre is not None else 0,
        p_bs[0], p_bs[1],
        alpha, beta, ACT[act], ACT[dact] if aux is not None else 0, max_ctas, int(fold_batch1), int(tile_n),
        float(drop_p), int(drop_seed) if drop_p > 0.0 else 0, int(ksplit), 0, int(peer_out) or None, int(peer_rows), 0,
        ctypes.cast(peer_a, ctypes.c_void_p) if peer_a is not None else None, int(peer_a_rows), len(peer_a) if peer_a is not None else 0, int(pair),
        *((int(sig[0]) or None, int(sig[1]) or None, int(sig[2]), int(sig[3]), int(sig[4]) & 0xFFFFFFFF, int(sig[5]), int(sig[6]), 0)
          if sig is not None else (None, None, 0, 0, 0, 0, 0, 0)),
        *((int(stage[0]) or None, int(stage[1]) or None, int(stage[2]), int(stage[3]) or None) if stage is not None else (None, None, 0, None)),
        ws.data_ptr() if ws is not None else None, ws.numel() * 4 if ws is not None else 0)
    _check(lib().sb_gemm_bf16(ctypes.byref(g), _stream()), "sb_gemm_bf16")
    return out


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0 or (x2.data_ptr() % 16) != 0:
        x2 = x2.contiguous()
    return x2


def _lowp_weight(w: torch.Tensor) -> torch.Tensor:
    from . import lowp

    wl = lowp(w, torch.bfloat16)
    if wl.dim() != 2:
        wl = wl.reshape(wl.shape[0], -1)
    return wl if wl.is_contiguous() else wl.contiguous()


def _write_param_grad(param: torch.Tensor, compute, shape) -> Optional[torch.Tensor]:
    """Run ``compute(out_fp32, beta)`` so that the gradient lands in the arena's flat buffer when there is one.

    Returns ``None`` when the gradient was written in place (autograd then has nothing to accumulate) or the fresh
    gradient tensor otherwise."""
    gv = getattr(param, "_grad_view", None)
    if gv is not None and gv.is_cuda:
        compute(gv.view(shape), 1.0)
        arena = getattr(param, "_arena", None)
        cb = getattr(arena, "grad_ready", None) if arena is not None else None
        if cb is not None:
            for m in getattr(param, "_members", None) or [param]:
                cb(m)
        return None
    out = torch.empty(shape, dtype=torch.float32, device=param.device)
    compute(out, 0.0)
    return out.view(param.shape)


# ------------------------------------------------------------------------------------------------ linear
class _LinearFn(torch.autograd.Function):
    """y = residual + alpha * dropout(act(x W^T + b)); saves x and (when needed) the pre-activation for backward.  The
    dropout mask is a hash of (seed, element index): the backward pass rebuilds it instead of storing it."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, act, alpha, drop_p=0.0):
        x2 = _as_2d(x)
        M, K = x2.shape
        wl = _lowp_weight(weight)
        N = wl.shape[0]
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        need_pre = act is not None and ctx.needs_input_grad[0] | ctx.needs_input_grad[1]
        pre = torch.empty_like(y) if need_pre else None
        r2 = _as_2d(residual) if residual is not None else None
        seed = _next_dropout_seed() if drop_p > 0.0 else 0
        gemm(x2, wl, y, M=M, N=N, K=K, lda=x2.stride(0), bias=bias, act=act, residual=r2,
             ldr=(r2.stride(0) if r2 is not None else None), out_pre=pre, alpha=alpha, drop_p=drop_p, drop_seed=seed)
        ctx.drop_p, ctx.drop_seed = drop_p, seed
        ctx.save_for_backward(x2, pre)
        ctx.weight, ctx.bias = weight, bias
        ctx.act, ctx.alpha = act, alpha
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, pre = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        M, K = x2.shape
        dy2 = _as_2d(dy)
        N = dy2.shape[1]
        wl = _lowp_weight(weight)
        # gradient w.r.t. the pre-activation z: dz = alpha * dy * act'(z)
        if ctx.act is not None or ctx.drop_p > 0.0:
            dz = torch.empty((M, N), dtype=torch.bfloat16, device=dy.device)
            lib_call_scale_dact(dy2, pre if ctx.act is not None else None, dz, ctx.act, ctx.alpha, ctx.drop_p, ctx.drop_seed)
        elif ctx.alpha != 1.0:
            dz = dy2 * ctx.alpha
        else:
            dz = dy2
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
            gemm(dz, wl, dx, M=M, N=K, K=N, lda=dz.stride(0), b_mn=True, ldb=K)
            dx = dx.view(ctx.x_shape)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _write_param_grad(weight, lambda out, beta: gemm(dz, x2, out, M=N, N=K, K=M, a_mn=True, lda=dz.stride(0),
                                                                  b_mn=True, ldb=x2.stride(0), beta=beta), (N, K))
        db = None
        if bias is not None and ctx.needs_input_grad[2]:
            db = _write_param_grad(bias, lambda out, beta: colsum(dz, out, accumulate=beta != 0.0), (N,))
        dres = dy if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None, None, None


_dropout_counter = [0x5EED5EED]


def _next_dropout_seed() -> int:
    """A fresh 64-bit seed per dropout site and step (host counter mixed with torch's seed, so runs are reproducible)."""
    _dropout_counter[0] = (_dropout_counter[0] * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
    return (_dropout_counter[0] ^ (torch.initial_seed() & 0xFFFFFFFFFFFFFFFF)) & 0xFFFFFFFFFFFFFFFF


def lib_call_scale_dact(dy2, pre, dz, act, alpha, drop_p: float = 0.0, drop_seed: int = 0):
    _check(lib().sb_scale_dact_dropout(_ptr(dy2), ctypes.c_longlong(dy2.stride(0)), _ptr(pre), _ptr(dz), ctypes.c_int(dy2.shape[0]),
                                       ctypes.c_int(dy2.shape[1]), ctypes.c_int(ACT[act]), ctypes.c_float(alpha),
                                       ctypes.c_float(drop_p), ctypes.c_ulonglong(drop_seed), _stream()),
           "sb_scale_dact_dropout")


def colsum(x2: torch.Tensor, out: torch.Tensor, accumulate: bool = False):
    if not accumulate:
        out.zero_()
    _check(lib().sb_colsum_bf16(_ptr(x2), ctypes.c_longlong(x2.stride(0)), ctypes.c_int(x2.shape[0]), ctypes.c_int(x2.shape[1]),
                                _ptr(out), _stream()), "sb_colsum_bf16")
    return out


def linear(x, weight, bias=None, act=None, residual=None, alpha: float = 1.0, dropout_p: float = 0.0):
    K = x.shape[-1]
    # the backward pass feeds dy [M, N] to the tensor core as a K-major operand: N must keep rows 16-byte aligned as well
    if K % 8 != 0 or x.numel() == 0 or weight.shape[0] % 8 != 0:
        from . import reference

        return reference.linear(x, weight, bias, act, residual, alpha, dropout_p)
    return _LinearFn.apply(x, weight, bias, residual, act, alpha, float(dropout_p))


# ------------------------------------------------------------------------------------------------ layer norm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows, D = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().sb_layernorm_fwd(_ptr(x2), _ptr(weight), _ptr(bias), _ptr(y), _ptr(mean), _ptr(rstd), ctypes.c_int(rows),
                                      ctypes.c_int(D), ctypes.c_float(eps), _stream()), "sb_layernorm_fwd")
        ctx.save_for_backward(x2, mean, rstd)
        ctx.weight, ctx.bias = weight, bias
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        gw = getattr(weight, "_grad_view", None)
        gb = getattr(bias, "_grad_view", None) if bias is not None else None
        direct = gw is not None and gw.is_cuda and (bias is None or gb is not None)
        if direct:
            dg, db = gw, gb
        else:
            dg = torch.zeros(D, dtype=torch.float32, device=dy.device)
            db = torch.zeros(D, dtype=torch.float32, device=dy.device) if bias is not None else None
        _check(lib().sb_layernorm_bwd(_ptr(dy2), _ptr(x2), _ptr(weight), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(dg), _ptr(db),
                                      ctypes.c_int(rows), ctypes.c_int(D), _stream()), "sb_layernorm_bwd")
        if direct:
            arena = getattr(weight, "_arena", None)
            cb = getattr(arena, "grad_ready", None) if arena is not None else None
            if cb is not None:
                cb(weight)
                if bias is not None:
                    cb(bias)
            return dx.view(ctx.shape), None, None, None
        return dx.view(ctx.shape), dg, db, None


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if x.shape[-1] % 8 != 0 or x.shape[-1] > 5632 or weight.dtype != torch.float32:
        from . import reference

        return reference.layer_norm(x, weight, bias, eps)
    return _LayerNormFn.apply(x, weight, bias, eps)


# ------------------------------------------------------------------------------------------------ optimizer
_partials = {}


def grad_norm_clip_coef(flat_grad, scalars, max_norm: float, grad_scale: float = 1.0):
    dev = flat_grad.device
    buf = _partials.get(dev)
    if buf is None:
        buf = torch.empty(int(lib().sb_grad_norm_partials()), dtype=torch.float32, device=dev)
        _partials[dev] = buf
    _check(lib().sb_grad_norm_clip(_ptr(flat_grad), ctypes.c_longlong(flat_grad.numel()), _ptr(buf), _ptr(scalars),
                                   ctypes.c_float(max_norm), ctypes.c_float(grad_scale), _stream()), "sb_grad_norm_clip")


def adamw_flat(master, grad, exp_avg, exp_avg_sq, lowp, lr, beta1, beta2, eps, weight_decay, step, scalars):
    assert master.dtype == torch.float32 and grad.dtype == torch.float32
    _check(lib().sb_adamw(_ptr(master), _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq), _ptr(lowp), ctypes.c_longlong(master.numel()),
                          ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                          ctypes.c_float(weight_decay), ctypes.c_int(step), _ptr(scalars), _stream()), "sb_adamw")


from .native_blocks import conv_module_core, mha_attention, relpos_attention  # noqa: E402,F401
def specaugment_(x: torch.Tensor, f_start, f_width, t_start, t_width, mask_value: float = 0.0) -> torch.Tensor:
    """Mask ``x`` [B, F, T] (fp32 / bf16, contiguous) in place; start / width tensors are int32 [B, n] or None."""
    B, F, T = x.shape
    nf = 0 if f_start is None else f_start.shape[1]
    nt = 0 if t_start is None else t_start.shape[1]
    _check(lib().sb_specaugment(_ptr(x), ctypes.c_int(int(x.dtype == torch.bfloat16)), ctypes.c_int(B), ctypes.c_int(F), ctypes.c_int(T),
                                _ptr(f_start), _ptr(f_width), ctypes.c_int(nf), _ptr(t_start), _ptr(t_width), ctypes.c_int(nt),
                                ctypes.c_void_p(0), ctypes.c_float(mask_value), _stream()), "sb_specaugment")
    return x


def ngram_advance(states, arc_keys, arc_w, arc_to, backoff_w, backoff_to, V: int, depth: int, default_score: float, start_state: int):
    """One back-off automaton step for every (hypothesis, token): returns ``scores [B, V]`` fp32 and ``next_states [B, V]`` int64."""
    B = states.shape[0]
    scores = torch.empty((B, V), dtype=torch.float32, device=states.device)
    nxt = torch.empty((B, V), dtype=torch.long, device=states.device)
    _check(lib().sb_ngram_advance(_ptr(states), _ptr(arc_keys), _ptr(arc_w), _ptr(arc_to), _ptr(backoff_w), _ptr(backoff_to),
                                  ctypes.c_int(arc_keys.shape[0]), ctypes.c_int(backoff_to.shape[0]), ctypes.c_int(B), ctypes.c_int(V),
                                  ctypes.c_int(depth), ctypes.c_float(default_score), ctypes.c_longlong(start_state), _ptr(scores),
                                  _ptr(nxt), _stream()), "sb_ngram_advance")
    return scores, nxt


from .native_transducer import transducer_joint_loss, transducer_loss_from_logits  # noqa: E402,F401
from .native_lstm import lstm  # noqa: E402,F401
from .native_ctc import ctc_loss  # noqa: E402,F401
from .native_logmel import logmel  # noqa: E402,F401


def __getattr__(name):
    # decode graph builder lives with the decoders; exposed here because callers look it up next to the kernels
    if name == "LabelLoopingGraph":
        from ..decoding.label_looping_graph import LabelLoopingGraph

        return LabelLoopingGraph
    raise AttributeError(name)

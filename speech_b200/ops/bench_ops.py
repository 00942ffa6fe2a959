"""Micro-benchmarks of the native kernels: ``python -m speech_b200.ops.bench_ops --op gemm --m 3750 --n 4096 --k 1024``.

Times one op with CUDA events after warm-up, rotating over enough distinct inputs that every timed launch reads
operands that are not in L2, and prints one JSON line with the achieved rate next to the library op (cuBLAS / ATen) on the
same shape.  Small ``--iters`` values make the command suitable for a profiler capture of a single kernel.
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, n_variants: int, iters: int, warmup: int) -> float:
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(iters):
        fn(i % n_variants)
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def bench_gemm(a):
    from . import native

    dev = torch.device("cuda")
    M, N, K = a.m, a.n, a.k
    per = (M * K + N * K + M * N) * 2
    nv = max(2, min(64, int(256e6 // per) + 1))  # rotate through > 2x L2 of operands
    A = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(nv)]
    B = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) for _ in range(nv)]
    D = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(nv)]
    bias = torch.randn(N, device=dev, dtype=torch.float32) if a.epilogue != "none" else None
    act = "swish" if a.epilogue == "bias_swish" else None
    ms = _time(lambda i: native.gemm(A[i], B[i], D[i], M=M, N=N, K=K, bias=bias, act=act, tile_n=a.tile_n, pair=a.pair), nv, a.iters, a.warmup)
    ms_lib = _time(lambda i: torch.matmul(A[i], B[i].t(), out=D[i]), nv, a.iters, a.warmup)
    native.check_status()
    fl = 2.0 * M * N * K
    return {"op": "gemm", "shape": [M, N, K], "epilogue": a.epilogue, "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
            "library_ms": round(ms_lib, 4), "library_tflops": round(fl / ms_lib / 1e9, 1), "variants": nv}


def bench_layernorm(a):
    from .. import ops

    dev = torch.device("cuda")
    rows, D = a.m, a.n
    nv = max(2, int(300e6 // (rows * D * 2)) + 1)
    xs = [torch.randn(rows, D, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(nv)]
    w = torch.ones(D, device=dev, requires_grad=True)
    b = torch.zeros(D, device=dev, requires_grad=True)

    def fwd_bwd(i):
        y = ops.layer_norm(xs[i], w, b, 1e-5)
        y.backward(xs[i].detach())

    def lib(i):
        y = torch.nn.functional.layer_norm(xs[i], (D,), w.to(xs[i].dtype), b.to(xs[i].dtype), 1e-5)
        y.backward(xs[i].detach())

    ms = _time(fwd_bwd, nv, a.iters, a.warmup)
    ms_lib = _time(lib, nv, a.iters, a.warmup)
    by = rows * D * 2 * 5  # x, y | dy, x, dx
    return {"op": "layernorm_fwd_bwd", "shape": [rows, D], "ms": round(ms, 4), "gbs": round(by / ms / 1e6, 1),
            "library_ms": round(ms_lib, 4)}


def bench_adamw(a):
    from . import native  # noqa: F401
    from ..core.optim.fused_adamw import FusedAdamW

    dev = torch.device("cuda")
    n = a.m * a.n
    p = torch.nn.Parameter(torch.randn(n, device=dev))
    opt = FusedAdamW([p], lr=1e-3)
    opt.arena.grad.normal_()

    def step(_):
        opt.step()

    ms = _time(step, 1, a.iters, a.warmup)
    by = n * (4 * 4 + 3 * 4 + 2)  # read p, g, m, v; write p, m, v, bf16 copy
    return {"op": "adamw", "numel": n, "ms": round(ms, 4), "gbs": round(by / ms / 1e6, 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "layernorm", "adamw"])
    ap.add_argument("--m", type=int, default=3750)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "bias_swish"])
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--pair", type=int, default=0, help="1: CTA-pair (cta_group::2) variant, -1: never, 0: default policy")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    out = {"gemm": bench_gemm, "layernorm": bench_layernorm, "adamw": bench_adamw}[a.op](a)
    print(json.dumps(out))


if __name__ == "__main__":
    main()

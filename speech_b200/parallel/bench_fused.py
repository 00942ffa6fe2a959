"""Fused GEMM + collective kernels against cuBLAS + NCCL, with roofline fractions.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m speech_b200.parallel.bench_fused

For every shape: device time (CUDA events around 20 launches after 3 warm-up launches, max over ranks) of ``GemmReduceScatter``
/ ``AllGatherGemm`` and of the library pair; the roofline time is the slower of (FLOPs per rank / measured GEMM peak) and (bytes
that must cross NVLink per rank / measured peer bandwidth).  Rank 0 prints one JSON line per shape.  Operands rotate over
several buffers so that the timed launches do not find their weights in L2.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, n=20, warm=3):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(n):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / n], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gemm-tflops", type=float, default=1634.6, help="measured bf16 GEMM peak")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from ..ops import native
    from .fused import AllGatherGemm, GemmReduceScatter

    NV = 6
    # (tokens per rank, hidden, ffn shard per rank): attention-output / down projections and QKV / up projections of a
    # tensor-parallel decoder block at hidden 2048 / ffn 6144 and at hidden 4096 / ffn 14336
    shapes = [(1024, 1024, 2048), (4096, 2048, 6144 // world), (8192, 4096, 14336 // world)]
    rs = GemmReduceScatter(max(s[0] for s in shapes), max(s[1] for s in shapes), dev)
    ag = AllGatherGemm(max(s[0] for s in shapes), max(s[1] for s in shapes), dev)
    for rows, hidden, shard in shapes:
        M = rows * world
        x = [torch.randn(M, shard, device=dev).to(torch.bfloat16) for _ in range(NV)]
        w = [torch.randn(hidden, shard, device=dev).to(torch.bfloat16) for _ in range(NV)]
        out = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)

        def lib_rs(i):
            dist.reduce_scatter_tensor(out, x[i % NV] @ w[i % NV].t())

        t_f, t_l = _timed(lambda i: rs(x[i % NV], w[i % NV])), _timed(lib_rs)
        flops = 2.0 * M * hidden * shard
        link = (world - 1) / world * M * hidden * 4          # fp32 partial sums sent to the owners
        roof = max(flops / (args.gemm_tflops * 1e12), link / (args.link_gbs * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"op": "gemm+reduce_scatter", "world": world, "M": M, "N": hidden, "K_local": shard, "fused_ms": round(t_f, 4),
                              "cublas_nccl_ms": round(t_l, 4), "roofline_ms": round(roof, 4), "fused_frac_of_roofline": round(roof / t_f, 3),
                              "library_frac_of_roofline": round(roof / t_l, 3)}), flush=True)
        xl = [torch.randn(rows, hidden, device=dev).to(torch.bfloat16) for _ in range(NV)]
        w2 = [torch.randn(shard, hidden, device=dev).to(torch.bfloat16) for _ in range(NV)]
        gathered = torch.empty(M, hidden, device=dev, dtype=torch.bfloat16)

        def lib_ag(i):
            dist.all_gather_into_tensor(gathered, xl[i % NV])
            return gathered @ w2[i % NV].t()

        t_f, t_l = _timed(lambda i: ag(xl[i % NV], w2[i % NV])), _timed(lib_ag)
        flops = 2.0 * M * shard * hidden
        link = (world - 1) * rows * hidden * 2               # the other ranks' bf16 shards read over NVLink
        roof = max(flops / (args.gemm_tflops * 1e12), link / (args.link_gbs * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"op": "all_gather+gemm", "world": world, "M": M, "N_local": shard, "K": hidden, "fused_ms": round(t_f, 4),
                              "cublas_nccl_ms": round(t_l, 4), "roofline_ms": round(roof, 4), "fused_frac_of_roofline": round(roof / t_f, 3),
                              "library_frac_of_roofline": round(roof / t_l, 3)}), flush=True)
    native.check_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Fused compute + collective operators over NVLink peer memory.

``GemmReduceScatter`` — the row-parallel linear layer of tensor parallelism (attention output / MLP down projection followed by
a reduce-scatter onto sequence-parallel shards) as ONE GEMM launch: every rank multiplies its K-shard, and the GEMM's epilogue
adds each output tile straight into the buffer of the rank that owns those rows, with fp32 vector reductions issued from the
tensor-core kernel to peer memory (``csrc/gemm_tcgen05.cu``, ``peer_D``).  No partial-result tensor is written locally and no
separate collective kernel runs; the transfer of tile i overlaps the MMAs of tile i+1 because the kernel is persistent with two
accumulators.  A flag barrier (the small-vector peer all-reduce kernel) before and after the launch orders the zeroing, the
remote reductions and the consumer's read.

The reference reaches the same result with a cuBLAS GEMM followed by an NCCL reduce-scatter
(``speechlm2/parts/parallel.py`` tensor-parallel plans over ``torch.distributed.tensor``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .symm import PeerSmallAllReduce, SymmetricBuffer


class GemmReduceScatter:
    def __init__(self, max_rows_per_rank: int, max_cols: int, device: torch.device, group=None):
        from ..ops import native

        self.native = native
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.capacity = int(max_rows_per_rank) * int(max_cols)
        self.buf = SymmetricBuffer(self.capacity * 4, device, self.group)
        self.barrier = PeerSmallAllReduce(device, self.group)
        self._token = torch.zeros(8, dtype=torch.float32, device=device)
        self.device = device

    def _sync(self) -> None:
        """All ranks' earlier work on this stream (zeroing, remote reductions) is complete and visible before anyone goes on."""
        self.barrier(self._token)

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """x [M, K_local], w [N, K_local] (bf16, this rank's K shard) -> rows [rank*M/W, (rank+1)*M/W) of sum_r x_r w_r^T."""
        M, K = x.shape
        N = w.shape[0]
        if M % self.world or (M // self.world) * N > self.capacity or N % 4 or K % 8:
            raise ValueError(f"GemmReduceScatter: M={M} must split evenly over {self.world} ranks within the buffer; N % 4 == 0, K % 8 == 0")
        rows = M // self.world
        acc = self.buf.tensor[: rows * N * 4].view(torch.float32).view(rows, N)
        acc.zero_()
        self._sync()                                        # every rank's accumulator is zero before reductions may arrive
        self.native.gemm(x, w, acc, M=M, N=N, K=K, lda=x.stride(0), ldb=w.stride(0), ldd=N, beta=1.0, peer_out=self.buf.ptrs_dev,
                         peer_rows=rows, ksplit=-1)
        self._sync()                                        # all ranks' contributions have landed
        return acc.to(out_dtype) if out_dtype != torch.float32 else acc.clone()

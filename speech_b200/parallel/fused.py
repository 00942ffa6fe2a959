"""Fused compute + collective operators over NVLink peer memory.

``GemmReduceScatter`` — the row-parallel linear layer of tensor parallelism (attention output / MLP down projection followed by
a reduce-scatter onto sequence-parallel shards) as ONE GEMM launch: every rank multiplies its K-shard, and the GEMM's epilogue
adds each output tile straight into the buffer of the rank that owns those rows, with fp32 vector reductions issued from the
tensor-core kernel to peer memory (``csrc/gemm_tcgen05.cu``, ``peer_D``).  No partial-result tensor is written locally and no
separate collective kernel runs; the transfer of tile i overlaps the MMAs of tile i+1 because the kernel is persistent with two
accumulators.  A flag barrier (the small-vector peer all-reduce kernel) before and after the launch orders the zeroing, the
remote reductions and the consumer's read.

``AllGatherGemm`` — the column-parallel linear layer fed by sequence-parallel activations (all-gather, then QKV / up projection)
as ONE GEMM launch: every rank keeps its row shard of the activations in a symmetric buffer, and the GEMM's TMA producer loads
each A tile straight from the memory of the rank that owns those rows (one tensor map per rank, plain tiled loads, no multicast).
The gathered activation matrix never exists in memory.

The reference reaches the same results with a cuBLAS GEMM preceded by an NCCL all-gather / followed by an NCCL reduce-scatter
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


class AllGatherGemm:
    def __init__(self, max_rows_per_rank: int, max_k: int, device: torch.device, group=None):
        import ctypes

        from ..ops import native

        self.native, self.ctypes = native, ctypes
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("AllGatherGemm supports up to 8 ranks")
        self.capacity = int(max_rows_per_rank) * int(max_k)
        self.buf = SymmetricBuffer(self.capacity * 2, device, self.group)
        self.peer_ptrs = [int(p) for p in self.buf.handle.buffer_ptrs]
        self.barrier = PeerSmallAllReduce(device, self.group)
        self._token = torch.zeros(8, dtype=torch.float32, device=device)

    def _sync(self) -> None:
        self.barrier(self._token)

    def __call__(self, x_local: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
        """x_local [M/W, K] (bf16, this rank's rows), w [N_local, K] -> act(concat_r(x_r) @ w^T + bias) of shape [M, N_local]."""
        rows, K = x_local.shape
        if rows % 128 or rows * K > self.capacity or K % 8:
            raise ValueError("AllGatherGemm: rows per rank must be a multiple of 128 and fit the buffer; K % 8 == 0")
        mine = self.buf.tensor[: rows * K * 2].view(torch.bfloat16).view(rows, K)
        mine.copy_(x_local)
        self._sync()                                        # every rank's shard is in place before anyone loads it
        M, N = rows * self.world, w.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
        arr = (self.ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self.native.gemm(mine, w, out, M=M, N=N, K=K, lda=K, ldb=w.stride(0), ldd=N, bias=bias, act=act, peer_a=arr, peer_a_rows=rows, pair=-1)
        self._sync()                                        # nobody overwrites its shard while a peer may still be reading it
        return out

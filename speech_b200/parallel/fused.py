"""Fused compute + collective operators over NVLink peer memory.

``GemmReduceScatter`` — the row-parallel linear layer of tensor parallelism (attention output / MLP down projection followed by
a reduce-scatter onto sequence-parallel shards) as ONE GEMM launch: every rank multiplies its K-shard, and the GEMM's epilogue
adds each output tile straight into the buffer of the rank that owns those rows, with fp32 vector reductions issued from the
tensor-core kernel to peer memory (``csrc/gemm_tcgen05.cu``, ``peer_D``).  No partial-result tensor is written locally and no
separate collective kernel runs; the transfer of tile i overlaps the MMAs of tile i+1 because the kernel is persistent with two
accumulators.  The ranks synchronise inside the kernels: the GEMM's last block publishes a "landed" flag to every rank after
system-scope fences, and the consumer kernel that converts (and clears) the accumulator waits for all ranks' flags.

``AllGatherGemm`` — the column-parallel linear layer fed by sequence-parallel activations (all-gather, then QKV / up projection)
as ONE GEMM launch: every rank keeps its row shard of the activations in a symmetric buffer.  By default the kernel's own
blocks copy each remote shard once into local memory (the epilogue warps, with plain peer loads, while the tensor pipe multiplies
this rank's own rows, which the tile order puts first); the TMA producer then reads remote rows from the local copy.  Without
staging the producer loads each A tile straight from the memory of the rank that owns those rows (one tensor map per rank, plain
tiled loads, no multicast), which sends a shard over NVLink once per column tile: only worthwhile for narrow outputs.

The reference reaches the same results with a cuBLAS GEMM preceded by an NCCL all-gather / followed by an NCCL reduce-scatter
(``speechlm2/parts/parallel.py`` tensor-parallel plans over ``torch.distributed.tensor``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .symm import SymmetricBuffer


class _RankFlags:
    """Per-operator flag arrays in symmetric memory (16 x u32 per rank: "in place" slots 0..7, "landed" slots 8..15), the device
    table of all ranks' arrays, a block counter, and the call epoch."""

    def __init__(self, device: torch.device, group):
        self.buf = SymmetricBuffer(256, device, group)
        self.table = self.buf.ptrs_dev                       # device array of the ranks' flag-array pointers
        self.mine = self.buf.tensor.data_ptr()
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.epoch = 0
        self.rank, self.world = self.buf.rank, self.buf.world

    def next(self) -> int:
        self.epoch += 1
        return self.epoch


class GemmReduceScatter:
    def __init__(self, max_rows_per_rank: int, max_cols: int, device: torch.device, group=None):
        import ctypes

        from ..ops import native

        self.native, self.ctypes = native, ctypes
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("GemmReduceScatter supports up to 8 ranks")
        self.capacity = int(max_rows_per_rank) * int(max_cols)
        self.half = -(-self.capacity * 4 // 256) * 256        # bytes of one accumulator; two alternate between calls
        self.buf = SymmetricBuffer(2 * self.half, device, self.group)
        ptrs = [int(p) for p in self.buf.handle.buffer_ptrs]
        # device tables of every rank's accumulator address, one per parity
        self.tables = [torch.tensor([p + h * self.half for p in ptrs], dtype=torch.int64, device=device) for h in range(2)]
        self.flags = _RankFlags(device, self.group)
        self.device = device
        lib = native.lib()
        lib.sb_peer_wait_reduce_out.restype = ctypes.c_int
        self.lib = lib

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """x [M, K_local], w [N, K_local] (bf16, this rank's K shard) -> rows [rank*M/W, (rank+1)*M/W) of sum_r x_r w_r^T.

        Two launches: the GEMM, whose epilogue adds every tile into its owner's accumulator and whose last block publishes
        "this rank's contributions have landed"; and the consumer, which waits for all ranks' flags, converts the accumulator
        and clears it.  Two accumulators alternate, so a rank that runs ahead adds into the one the slower rank is not reading:
        a rank can start call n only after passing call n-1's wait, i.e. after every rank has finished its GEMM n-1, which that
        rank issued after clearing the accumulator of call n-2 (the one call n uses)."""
        M, K = x.shape
        N = w.shape[0]
        if M % self.world or (M // self.world) * N > self.capacity or N % 4 or K % 8:
            raise ValueError(f"GemmReduceScatter: M={M} must split evenly over {self.world} ranks within the buffer; N % 4 == 0, K % 8 == 0")
        rows = M // self.world
        epoch = self.flags.next()
        h = epoch & 1
        acc = self.buf.tensor[h * self.half: h * self.half + rows * N * 4].view(torch.float32).view(rows, N)
        c = self.ctypes
        self.native.gemm(x, w, acc, M=M, N=N, K=K, lda=x.stride(0), ldb=w.stride(0), ldd=N, beta=1.0, peer_out=self.tables[h].data_ptr(),
                         peer_rows=rows, ksplit=-1, sig=(self.flags.table, self.flags.counter.data_ptr(), self.world, self.rank, epoch, 0, 1))
        out = torch.empty((rows, N), dtype=out_dtype, device=x.device)
        rc = self.lib.sb_peer_wait_reduce_out(c.c_void_p(acc.data_ptr()), c.c_void_p(out.data_ptr()), c.c_int(int(out_dtype == torch.bfloat16)),
                                              c.c_longlong(rows * N), c.c_void_p(self.flags.mine), c.c_int(self.world), c.c_uint(epoch),
                                              self.native._stream())
        if rc != 0:
            raise RuntimeError(f"sb_peer_wait_reduce_out failed with code {rc}")
        return out


class AllGatherGemm:
    def __init__(self, max_rows_per_rank: int, max_k: int, device: torch.device, group=None, staged: bool = True):
        """``staged``: the kernel's blocks first copy each remote shard once into local memory (plain peer loads) and the TMA
        producer reads remote rows from there; without it every A tile is loaded from the owner's memory by every column tile
        that needs it, which multiplies the NVLink traffic by the number of column tiles."""
        import ctypes

        from ..ops import native

        self.native, self.ctypes = native, ctypes
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("AllGatherGemm supports up to 8 ranks")
        self.capacity = int(max_rows_per_rank) * int(max_k)
        self.half = -(-self.capacity * 2 // 256) * 256        # bytes of one shard buffer; two alternate between calls
        self.buf = SymmetricBuffer(2 * self.half, device, self.group)
        self.peer_ptrs = [int(p) for p in self.buf.handle.buffer_ptrs]
        self.flags = _RankFlags(device, self.group)
        self.staged = bool(staged) and self.world > 1
        if self.staged:
            self.staging = torch.empty(self.world * self.half, dtype=torch.uint8, device=device)
            self.src_tables = [torch.tensor([p + h * self.half for p in self.peer_ptrs], dtype=torch.int64, device=device) for h in range(2)]
            self.stage_counter = torch.zeros(4, dtype=torch.int32, device=device)

    def input_buffer(self, rows: int, K: int) -> torch.Tensor:
        """The shard buffer of the NEXT call as a [rows, K] bf16 view: a producer kernel can write its output there directly,
        and ``__call__`` then skips the staging copy when it is handed this very tensor."""
        h = (self.flags.epoch + 1) & 1
        return self.buf.tensor[h * self.half: h * self.half + rows * K * 2].view(torch.bfloat16).view(rows, K)

    def __call__(self, x_local: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
        """x_local [M/W, K] (bf16, this rank's rows), w [N_local, K] -> act(concat_r(x_r) @ w^T + bias) of shape [M, N_local].

        One GEMM launch: its first block publishes "this rank's shard is in place", its TMA producer waits for the owner's flag
        before the first load from that rank's memory.  Two shard buffers alternate: a rank overwrites a buffer two calls after
        peers read it, and it has by then passed a wait on every peer's flag of the call in between, which that peer published
        after finishing the earlier GEMM."""
        rows, K = x_local.shape
        if rows % 128 or rows * K > self.capacity or K % 8:
            raise ValueError("AllGatherGemm: rows per rank must be a multiple of 128 and fit the buffer; K % 8 == 0")
        mine = self.input_buffer(rows, K)
        if x_local.data_ptr() != mine.data_ptr():
            mine.copy_(x_local)
        epoch = self.flags.next()
        h = epoch & 1
        M, N = rows * self.world, w.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
        sig = (self.flags.table, 0, self.world, self.rank, epoch, 1, 0)
        if self.staged:
            nbytes = rows * K * 2
            base = self.staging.data_ptr()
            arr = (self.ctypes.c_void_p * self.world)(*[mine.data_ptr() if r == self.rank else base + r * nbytes for r in range(self.world)])
            self.native.gemm(mine, w, out, M=M, N=N, K=K, lda=K, ldb=w.stride(0), ldd=N, bias=bias, act=act, peer_a=arr, peer_a_rows=rows, pair=-1,
                             sig=sig, stage=(self.src_tables[h].data_ptr(), base, nbytes, self.stage_counter.data_ptr()))
            return out
        arr = (self.ctypes.c_void_p * self.world)(*[p + h * self.half for p in self.peer_ptrs])
        self.native.gemm(mine, w, out, M=M, N=N, K=K, lda=K, ldb=w.stride(0), ldd=N, bias=bias, act=act, peer_a=arr, peer_a_rows=rows, pair=-1, sig=sig)
        return out

"""Gradient exchange through NVLink peer memory with the framework's own kernel.

The reference leaves data-parallel gradient reduction to PyTorch's c10d reducer and NCCL
(``docs/source/features/parallelisms.rst:10-40``).  Here every bucket of the flat gradient arena is reduced by one launch
of ``csrc/peer_allreduce.cu``: cast + scale to bf16, reduce-scatter by peer loads, all-gather by peer stores and unpack,
all inside the kernel, synchronised by flags in a symmetric buffer.  The symmetric buffer (same size and layout on every
rank, every rank holding plain P2P pointers to all of them) comes from ``torch.distributed._symmetric_memory``; only the
allocation and the address exchange are borrowed, the data path is the kernel's ordinary loads and stores.

Layout of the symmetric buffer: ``[flags | send (bf16) | recv (bf16)]``.  Buckets run one after another on the
communication stream and share the send / recv regions; the kernel's flag protocol makes that safe across ranks.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..utils.logging import logging
from .ddp import GradSync


class SbPeerArgs(ctypes.Structure):
    _fields_ = [("grad", ctypes.c_void_p), ("buffers", ctypes.c_void_p), ("flags_off", ctypes.c_longlong),
                ("send_off", ctypes.c_longlong), ("recv_off", ctypes.c_longlong), ("n", ctypes.c_longlong),
                ("slice", ctypes.c_longlong), ("chunk", ctypes.c_longlong), ("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("ctas", ctypes.c_int), ("epoch", ctypes.c_uint), ("scale", ctypes.c_float), ("status", ctypes.c_void_p)]


def padded_elems(n: int, world: int) -> int:
    """Elements the send / recv regions need for a bucket of ``n`` (per-rank slices are multiples of 8 elements)."""
    slice_ = -(-n // world)
    slice_ = -(-slice_ // 8) * 8
    return slice_ * world


class SymmetricBuffer:
    """A byte buffer allocated identically on every rank of ``group`` with peer addresses known to all ranks."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        self.nbytes = int(-(-nbytes // 256) * 256)
        self.tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.tensor.zero_()
        torch.cuda.synchronize(device)
        self.handle.barrier()
        torch.cuda.synchronize(device)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs_dev = int(self.handle.buffer_ptrs_dev)

    def barrier(self):
        self.handle.barrier()


class PeerAllReduce:
    """Launches the peer all-reduce kernel on fp32 buffers; one instance owns one symmetric buffer."""

    def __init__(self, max_elems: int, device: torch.device, group=None, ctas: Optional[int] = None):
        from ..ops import native

        self.native = native
        self.lib = native.lib()
        self.lib.sb_peer_flags_bytes.restype = ctypes.c_longlong
        self.lib.sb_peer_allreduce.restype = ctypes.c_int
        world = dist.get_world_size(group)
        self.flags_bytes = int(self.lib.sb_peer_flags_bytes())
        self.capacity = padded_elems(max_elems, world)
        region = -(-self.capacity * 2 // 256) * 256
        self.send_off = self.flags_bytes
        self.recv_off = self.flags_bytes + region
        self.buf = SymmetricBuffer(self.flags_bytes + 2 * region, device, group)
        self.rank, self.world = self.buf.rank, self.buf.world
        self.ctas = int(ctas or os.environ.get("SPEECH_B200_PEER_CTAS", 32))
        self.epoch = 0

    def __call__(self, flat: torch.Tensor, scale: float = 1.0) -> None:
        """In-place ``flat <- bf16_round(sum_over_ranks(bf16(flat * scale)))`` on the current stream."""
        n = flat.numel()
        if flat.dtype != torch.float32 or not flat.is_contiguous():
            raise ValueError("peer all-reduce expects a contiguous fp32 buffer")
        if padded_elems(n, self.world) > self.capacity:
            raise ValueError(f"bucket of {n} elements exceeds the symmetric buffer ({self.capacity})")
        self.epoch += 1
        a = SbPeerArgs(flat.data_ptr(), self.buf.ptrs_dev, 0, self.send_off, self.recv_off, n, 0, 0, self.rank, self.world,
                       self.ctas, self.epoch, float(scale), None)
        rc = self.lib.sb_peer_allreduce(ctypes.byref(a), self.native._stream())
        self.native.launch_count += 1
        if rc != 0:
            raise RuntimeError(f"sb_peer_allreduce failed with code {rc}")


class PeerGradSync(GradSync):
    """``GradSync`` whose buckets are reduced by the peer-memory kernel instead of an NCCL all-reduce."""

    def __init__(self, model, optimizers, world_size: int, device: torch.device, sync_batchnorm: bool = False, **kw):
        if device.type != "cuda":
            raise RuntimeError("peer-memory gradient exchange needs CUDA devices")
        super().__init__(model, optimizers, world_size, device, sync_batchnorm=sync_batchnorm, **kw)
        biggest = 1
        for b in self.buckets:
            n = b["view"].numel() if b["view"] is not None else sum(p.numel() for p in b["params"])
            biggest = max(biggest, n)
        self.reducer = PeerAllReduce(biggest, device)
        logging.info(f"peer-memory gradient exchange: {len(self.buckets)} buckets, largest {biggest * 4 / 2**20:.1f} MB, "
                     f"{self.reducer.ctas} CTAs per bucket")

    def _reduce_flat(self, flat: torch.Tensor):
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            self.reducer(flat, 1.0 / self.world_size)
        flat.record_stream(self.comm_stream)

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
        self.ctas = int(ctas or os.environ.get("SPEECH_B200_PEER_CTAS", 12))
        self.epoch = 0
        # the cast into the send region and the unpack from the receive region as wide kernels of their own (default), or inside
        # the few-block peer kernel
        self.split_local = os.environ.get("SPEECH_B200_PEER_SPLIT", "1") != "0"
        self.lib.sb_peer_allreduce_split.restype = ctypes.c_int

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
        if self.split_local:
            rc = self.lib.sb_peer_allreduce_split(ctypes.byref(a), ctypes.c_void_p(self.buf.tensor.data_ptr()), self.native._stream())
            self.native.launch_count += 3
        else:
            rc = self.lib.sb_peer_allreduce(ctypes.byref(a), self.native._stream())
            self.native.launch_count += 1
        if rc != 0:
            raise RuntimeError(f"sb_peer_allreduce failed with code {rc}")


class SbPeerSmallArgs(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("buffers", ctypes.c_void_p), ("base_off", ctypes.c_longlong), ("n", ctypes.c_int),
                ("has_extra", ctypes.c_int), ("extra", ctypes.c_float), ("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("epoch", ctypes.c_uint), ("status", ctypes.c_void_p)]


class PeerSmallAllReduce:
    """Sum of a small fp32 vector over all ranks by one single-CTA kernel over peer memory (``csrc/peer_small_allreduce.cu``).

    Every use — a direct call here or one made by the Conformer layer executor with ``ptrs_dev`` / ``next_epoch()`` — consumes
    one epoch; all ranks must make the same sequence of uses."""

    def __init__(self, device: torch.device, group=None):
        from ..ops import native

        self.native = native
        self.lib = native.lib()
        self.lib.sb_peer_small_bytes.restype = ctypes.c_longlong
        self.max_elems = int(self.lib.sb_peer_small_max())
        self.buf = SymmetricBuffer(int(self.lib.sb_peer_small_bytes()), device, group)
        self.rank, self.world, self.ptrs_dev = self.buf.rank, self.buf.world, self.buf.ptrs_dev
        self.epoch = 0

    def __deepcopy__(self, memo):
        return self   # process-wide communication state: modules that point here may be deep-copied (EMA, averaging)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def __call__(self, t: torch.Tensor, extra: Optional[float] = None) -> torch.Tensor:
        """In-place sum of ``t`` (fp32, contiguous) over ranks; with ``extra`` the tensor must have one spare element at the end
        that receives the sum of the ranks' ``extra`` values."""
        n = t.numel() - (1 if extra is not None else 0)
        if t.dtype != torch.float32 or not t.is_contiguous() or n <= 0 or t.numel() > self.max_elems:
            raise ValueError(f"small peer all-reduce takes contiguous fp32 vectors of at most {self.max_elems} elements")
        a = SbPeerSmallArgs(t.data_ptr(), self.ptrs_dev, 0, n, int(extra is not None), float(extra or 0.0), self.rank, self.world,
                            self.next_epoch(), None)
        rc = self.lib.sb_peer_small_allreduce(ctypes.byref(a), self.native._stream())
        self.native.launch_count += 1
        if rc != 0:
            raise RuntimeError(f"sb_peer_small_allreduce failed with code {rc}")
        return t


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
        # persistent GEMMs size their grids to the SMs that are left while a bucket kernel is resident on the other stream
        self.reducer.lib.sb_set_reserved_sms(ctypes.c_int(self.reducer.ctas))
        # Ranks drift apart by far more than the kernels' default wait limit of about a second in ordinary training (module
        # loading in the first step, a rank that validates or logs longer, a dataloader worker restarting): waits for a peer get
        # a minute before they give up, which then means a lost rank and fails the run (Trainer._check_kernel_status).
        self.reducer.native.set_wait_seconds(float(os.environ.get("SPEECH_B200_WAIT_SECONDS", "60")))
        logging.info(f"peer-memory gradient exchange: {len(self.buckets)} buckets, largest {biggest * 4 / 2**20:.1f} MB, "
                     f"{self.reducer.ctas} CTAs per bucket")

    def enable_sync_batchnorm(self):
        """BatchNorm statistics also travel through peer memory: the layer executor issues the small all-reduce itself."""
        super().enable_sync_batchnorm()
        self.small_reducer = PeerSmallAllReduce(self.device)
        for m in self.model.modules():
            if hasattr(m, "bn_stats_reduce"):
                m.bn_peer_sync = self.small_reducer

    def _reduce_flat(self, flat: torch.Tensor):
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            self.reducer(flat, 1.0 / self.world_size)
        flat.record_stream(self.comm_stream)

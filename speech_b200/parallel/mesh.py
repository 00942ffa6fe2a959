"""Named process-group mesh: ``(pp, dp_replicate, dp_shard, cp, tp)`` plus the flattened groups the training code asks for
(``dp`` = dp_replicate × dp_shard, ``dp_shard_cp``, ``dp_cp``), as in the reference's ``AutomodelParallelStrategy``
(``speechlm2/parts/parallel.py:168-170,265-292``).  Ranks are laid out row-major with ``tp`` fastest, so tensor-parallel
peers are neighbouring GPUs of one NVSwitch domain."""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Tuple

import torch.distributed as dist

DIM_ORDER = ("pp", "dp_replicate", "dp_shard", "cp", "tp")
FLATTENED = {"dp": ("dp_replicate", "dp_shard"), "dp_shard_cp": ("dp_shard", "cp"), "dp_cp": ("dp_replicate", "dp_shard", "cp")}


class DeviceMesh:
    def __init__(self, sizes: Dict[str, int], rank: Optional[int] = None, world_size: Optional[int] = None, create_groups: bool = True):
        self.sizes = {d: int(sizes.get(d, 1)) for d in DIM_ORDER}
        self.world = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.rank_ = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        free = [d for d in DIM_ORDER if self.sizes[d] in (-1, 0)]
        known = 1
        for d in DIM_ORDER:
            if d not in free:
                known *= self.sizes[d]
        if free:
            if len(free) > 1 or self.world % known:
                raise ValueError(f"cannot infer mesh sizes {free} for world size {self.world}")
            self.sizes[free[0]] = self.world // known
            known = self.world
        if known != self.world:
            raise ValueError(f"mesh {self.sizes} does not cover world size {self.world}")
        self.shape = tuple(self.sizes[d] for d in DIM_ORDER)
        self.coords = self._coords_of(self.rank_)
        self._groups: Dict[str, object] = {}
        self._group_ranks: Dict[str, List[int]] = {}
        for name in list(DIM_ORDER) + list(FLATTENED):
            dims = FLATTENED.get(name, (name,))
            for ranks in self._all_rank_lists(dims):
                g = dist.new_group(ranks) if (create_groups and dist.is_initialized() and len(ranks) > 1) else None
                if self.rank_ in ranks:
                    self._groups[name] = g
                    self._group_ranks[name] = ranks

    def _coords_of(self, rank: int) -> Dict[str, int]:
        c = {}
        for d, n in zip(reversed(DIM_ORDER), reversed(self.shape)):
            c[d] = rank % n
            rank //= n
        return c

    def _rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for d, n in zip(DIM_ORDER, self.shape):
            r = r * n + coords[d]
        return r

    def _all_rank_lists(self, dims: Sequence[str]) -> List[List[int]]:
        others = [d for d in DIM_ORDER if d not in dims]
        out = []
        for fixed in itertools.product(*[range(self.sizes[d]) for d in others]):
            base = dict(zip(others, fixed))
            ranks = []
            for var in itertools.product(*[range(self.sizes[d]) for d in dims]):
                c = dict(base)
                c.update(dict(zip(dims, var)))
                ranks.append(self._rank_of(c))
            out.append(sorted(ranks))
        return out

    def size(self, name: str) -> int:
        dims = FLATTENED.get(name, (name,))
        n = 1
        for d in dims:
            n *= self.sizes[d]
        return n

    def group(self, name: str):
        return self._groups.get(name)

    def ranks(self, name: str) -> List[int]:
        return self._group_ranks[name]

    def rank(self, name: str) -> int:
        return self._group_ranks[name].index(self.rank_)

    def is_dp_source(self) -> bool:
        """True on the rank that loads data for its (cp, tp) sub-mesh (reference ``datamodule.py:159-192``)."""
        return self.coords["cp"] == 0 and self.coords["tp"] == 0

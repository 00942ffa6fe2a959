"""Parallel strategy object: sizes of the mesh dimensions, validation against a model configuration, model set-up and the
gradient-exchange object for the trainer (the role of ``AutomodelParallelStrategy`` in the reference,
``speechlm2/parts/parallel.py:117-292``: mesh ``(pp, dp_replicate, dp_shard, cp, tp)`` with flattened ``dp`` / ``dp_shard_cp`` /
``dp_cp``, ``setup_distributed`` for scripts, parallelism compatibility checks, data-parallel sampler arguments).

    strategy = ParallelStrategy(dp_shard_size=4, tp_size=2, sequence_parallel=True)
    trainer = Trainer(strategy=strategy, ...)          # or: mesh = strategy.setup(); strategy.setup_model(model)

One process per GPU; ``-1`` for one size means "whatever is left of the world".
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from .mesh import DeviceMesh


@dataclass
class ParallelStrategy:
    dp_replicate_size: int = 1
    dp_shard_size: int = -1
    cp_size: int = 1
    tp_size: int = 1
    pp_size: int = 1
    sequence_parallel: bool = False
    expert_parallel: bool = False
    kind: str = "mesh"                         # what the trainer's strategy dispatch sees

    def __post_init__(self):
        self.mesh: Optional[DeviceMesh] = None

    # ------------------------------------------------------------------ process group / mesh
    @staticmethod
    def setup_distributed(backend: Optional[str] = None) -> int:
        """For scripts without a trainer: join the job described by the ``torchrun`` environment; returns the local rank."""
        local = int(os.environ.get("LOCAL_RANK", 0))
        if int(os.environ.get("WORLD_SIZE", 1)) > 1 and not dist.is_initialized():
            cuda = torch.cuda.is_available()
            if cuda:
                torch.cuda.set_device(local)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend or ("nccl" if cuda else "gloo"))
        return local

    def setup(self, world_size: Optional[int] = None, rank: Optional[int] = None, create_groups: bool = True) -> DeviceMesh:
        if self.pp_size != 1:
            raise ValueError("pipeline parallelism is not available: pp_size must be 1")
        self.mesh = DeviceMesh({"pp": self.pp_size, "dp_replicate": self.dp_replicate_size, "dp_shard": self.dp_shard_size, "cp": self.cp_size,
                                "tp": self.tp_size}, rank=rank, world_size=world_size, create_groups=create_groups)
        return self.mesh

    # ------------------------------------------------------------------ checks
    def validate(self, llm_config: Any = None, max_sequence_multiple: Optional[int] = None) -> List[str]:
        """Reasons why this strategy does not fit the model (empty list: compatible).  ``llm_config``: an ``LLMConfig`` or a
        dictionary with ``num_attention_heads``, ``num_key_value_heads``, ``intermediate_size``, ``num_experts`` ..."""
        problems: List[str] = []
        get = (lambda k, d=None: llm_config.get(k, d)) if isinstance(llm_config, dict) else (lambda k, d=None: getattr(llm_config, k, d))
        m = self.mesh
        tp = m.size("tp") if m is not None else self.tp_size
        cp = m.size("cp") if m is not None else self.cp_size
        dp = m.size("dp") if m is not None else None
        if self.pp_size != 1:
            problems.append("pp_size > 1: pipeline parallelism is not available")
        if self.sequence_parallel and tp == 1:
            problems.append("sequence_parallel needs tp_size > 1")
        if llm_config is not None:
            heads, kv = get("num_attention_heads"), get("num_key_value_heads") or get("num_attention_heads")
            if heads is not None and (heads % tp or kv % tp):
                problems.append(f"attention heads ({heads} query / {kv} key-value) are not divisible by tp_size {tp}")
            inter = get("moe_intermediate_size") if get("num_experts", 0) else get("intermediate_size")
            if inter is not None and inter % tp:
                problems.append(f"feed-forward width {inter} is not divisible by tp_size {tp}")
            ne = get("num_experts", 0) or 0
            if self.expert_parallel:
                if ne == 0:
                    problems.append("expert_parallel is set but the model has no experts")
                elif dp is not None and ne % dp:
                    problems.append(f"{ne} experts cannot be split over the {dp} data-parallel ranks")
                if cp > 1:
                    problems.append("expert_parallel with cp_size > 1: the expert group would differ from the gradient-averaging group")
        if max_sequence_multiple is not None:
            need = cp * (tp if self.sequence_parallel else 1)
            if max_sequence_multiple % need:
                problems.append(f"sequence lengths must be multiples of {need} (cp x sequence-parallel tp); the data pipeline pads to "
                                f"{max_sequence_multiple}")
        return problems

    # ------------------------------------------------------------------ model / trainer integration
    def setup_model(self, model) -> None:
        """Build the mesh if needed, check it against the model and let the model shard itself (``configure_model(mesh)``)."""
        if self.mesh is None:
            self.setup()
        cfg = getattr(getattr(model, "llm", None), "config", None)
        problems = self.validate(cfg)
        if problems:
            raise ValueError("parallel strategy does not fit the model: " + "; ".join(problems))
        if hasattr(model, "cfg"):
            from ..core.config import open_dict

            with open_dict(model.cfg):
                model.cfg.sequence_parallel = bool(self.sequence_parallel)
                model.cfg.expert_parallel = bool(self.expert_parallel)
        if not hasattr(model, "configure_model"):
            raise TypeError(f"{type(model).__name__} has no configure_model(mesh): it cannot be placed on a device mesh")
        model.configure_model(self.mesh)

    @property
    def distributed_sampler_kwargs(self) -> Dict[str, int]:
        """Ranks that must see different data: ``num_replicas`` / ``rank`` over the data-parallel group (tensor- and
        context-parallel peers of a rank read the same samples)."""
        m = self.mesh
        if m is None:
            return {"num_replicas": 1, "rank": 0}
        return {"num_replicas": m.size("dp"), "rank": m.rank("dp") if m.size("dp") > 1 else 0}

    def build_grad_sync(self, model, optimizers, device: torch.device, sync_batchnorm: bool = False):
        """The trainer's gradient-exchange object.  A fully-sharded optimizer brings its own reduce-scatter path; otherwise
        gradients are averaged over the ranks that see different tokens (``dp_cp``); with one such rank nothing is exchanged
        (tensor-parallel gradients are complete on their owner)."""
        from .ddp import GradSync

        m = self.mesh
        if any(type(o).__name__ == "FullyShardedAdamW" for o in optimizers):
            from .fsdp2 import FSDP2GradSync

            return FSDP2GradSync(model, optimizers, m.size("dp_shard_cp") if m is not None else 1, device, sync_batchnorm=sync_batchnorm)
        if m is None or m.size("dp_cp") == 1:
            return None
        return GradSync(model, optimizers, m.size("dp_cp"), device, sync_batchnorm=sync_batchnorm, group=m.group("dp_cp"))

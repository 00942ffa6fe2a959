"""Checkpoints in PyTorch's distributed-checkpoint (DCP) directory format: every rank writes the pieces it holds, a ``.metadata``
file describes the global tensors, and a checkpoint can be loaded on a different number of ranks or converted to a single file.

Three uses:
* ``DCPCheckpointIO.save_checkpoint / load_checkpoint`` — trainer-level save and restore; tensors are de-duplicated across
  ranks by the DCP planner (a replicated tensor is written once), row-sharded tensors are declared through ``sharded`` and written
  as ``ShardedTensor``-free plain chunks with global offsets, so they re-assemble (or re-shard) on load.
* ``load_dcp_into_model`` — pretrained weights published as a DCP directory into a module (``strict`` or partial).
* ``dcp_to_single_file`` / ``single_file_to_dcp`` — conversion to and from a ``torch.save`` state dict.

Reference: the reference reaches DCP through its training strategy's checkpoint IO and ``speechlm2/parts/pretrained.py`` (DCP
directories of HF models); the DCP library itself is PyTorch's.
"""
from __future__ import annotations

import json
import os
import threading
import warnings
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

__all__ = ["DCPCheckpointIO", "dcp_to_single_file", "is_dcp_checkpoint", "load_dcp_into_model", "single_file_to_dcp"]


def is_dcp_checkpoint(path: str) -> bool:
    return os.path.isdir(path) and os.path.exists(os.path.join(path, ".metadata"))


def _quiet(fn, *a, **k):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")                      # single-process use prints an "assuming single process" warning per call
        return fn(*a, **k)


class _RowShard:
    """A rank's rows ``[offset, offset + local.shape[0])`` of a tensor with ``global_rows`` rows, presented to DCP as a chunk of the
    global tensor (what a DTensor sharded on dim 0 would declare) without needing a device mesh."""

    def __init__(self, local: torch.Tensor, offset: int, global_rows: int):
        self.local, self.offset, self.global_rows = local, offset, global_rows


class DCPCheckpointIO:
    """``save_checkpoint(state, path, sharded={name: (row offset, global rows)})``: ``state`` is a (nested) dict of tensors and plain
    values; names in ``sharded`` hold only this rank's rows.  ``async_save`` stages to CPU and writes on a background thread
    (``finalize()`` joins)."""

    def __init__(self, async_save: bool = False, process_group=None):
        self.async_save, self.pg = async_save, process_group
        self._pending: List[threading.Thread] = []

    @staticmethod
    def _world() -> Tuple[int, int]:
        return (dist.get_rank(), dist.get_world_size()) if dist.is_available() and dist.is_initialized() else (0, 1)

    def save_checkpoint(self, state: Dict[str, Any], path: str, sharded: Optional[Dict[str, Tuple[int, int]]] = None, extra: Optional[dict] = None) -> None:
        rank, world = self._world()
        sharded = sharded or {}
        os.makedirs(path, exist_ok=True)
        plain, pieces = {}, {}
        for k, v in state.items():
            if k in sharded:
                off, rows = sharded[k]
                pieces[k] = {"offset": int(off), "rows": int(rows), "shape": list(v.shape[1:]), "dtype": str(v.dtype).replace("torch.", "")}
                plain[f"__rows__/{k}/{rank}"] = v.detach()
            else:
                plain[k] = v.detach() if torch.is_tensor(v) else v
        if self.async_save:
            plain = {k: (v.to("cpu", copy=True) if torch.is_tensor(v) else v) for k, v in plain.items()}

        def write():
            _quiet(dcp.save, plain, checkpoint_id=path, process_group=self.pg)
            # which rows each rank wrote: small JSON beside the DCP files, one per rank, merged by the loader
            with open(os.path.join(path, f"rows_{rank:05d}.json"), "w") as f:
                json.dump({"world_size": world, "pieces": pieces, "extra": extra or {}}, f)

        if self.async_save and world == 1:
            t = threading.Thread(target=write, daemon=True)
            t.start()
            self._pending.append(t)
        else:
            write()                                          # the collective inside dcp.save must run on the calling thread

    def finalize(self) -> None:
        for t in self._pending:
            t.join()
        self._pending.clear()

    @staticmethod
    def _row_index(path: str) -> Tuple[Dict[str, List[Tuple[int, int, int]]], dict]:
        """``{name: [(rank, offset, rows)]}`` merged over the per-rank files, and the ``extra`` of rank 0."""
        table: Dict[str, List[Tuple[int, int, int]]] = {}
        extra: dict = {}
        for f in sorted(os.listdir(path)):
            if f.startswith("rows_") and f.endswith(".json"):
                r = int(f[5:10])
                d = json.load(open(os.path.join(path, f)))
                if r == 0:
                    extra = d.get("extra", {})
                for k, p in d["pieces"].items():
                    table.setdefault(k, []).append((r, p["offset"], p["rows"]))
        return table, extra

    def load_checkpoint(self, path: str, template: Optional[Dict[str, Any]] = None, sharded: Optional[Dict[str, Tuple[int, int]]] = None,
                        map_location="cpu") -> Tuple[Dict[str, Any], dict]:
        """Without ``template``: everything in the checkpoint, row-sharded tensors assembled in full.  With ``template`` (a state dict
        of the right shapes, e.g. ``model.state_dict()``): loads in place into it; names in ``sharded`` get the rows
        ``[offset, offset + local rows)`` of the assembled tensor — any world size, not only the one that saved."""
        if not is_dcp_checkpoint(path):
            raise FileNotFoundError(f"{path} is not a DCP checkpoint directory")
        table, extra = self._row_index(path)
        meta = _quiet(dcp.FileSystemReader(path).read_metadata)
        full: Dict[str, Any] = {}
        for k, md in meta.state_dict_metadata.items():
            if hasattr(md, "size"):
                full[k] = torch.empty(tuple(md.size), dtype=md.properties.dtype, device=map_location)
        if full:
            _quiet(dcp.load, full, checkpoint_id=path, process_group=self.pg)
        # non-tensor entries are stored as bytes
        rest = {k: None for k, md in meta.state_dict_metadata.items() if not hasattr(md, "size")}
        if rest:
            _quiet(dcp.load, rest, checkpoint_id=path, process_group=self.pg)
            full.update(rest)
        out: Dict[str, Any] = {}
        for k, v in full.items():
            if not k.startswith("__rows__/"):
                out[k] = v
        for name, pieces in table.items():
            pieces = sorted(set(pieces), key=lambda p: p[1])
            out[name] = torch.cat([full[f"__rows__/{name}/{r}"] for r, _, _ in pieces], dim=0)
        if template is None:
            return out, extra
        sharded = sharded or {}
        for k, dst in template.items():
            if k not in out:
                raise KeyError(f"{k} is not in the checkpoint")
            src = out[k]
            if k in sharded and torch.is_tensor(dst):
                off = int(sharded[k][0])
                src = src[off: off + dst.shape[0]]
            if torch.is_tensor(dst):
                if tuple(dst.shape) != tuple(src.shape):
                    raise ValueError(f"{k}: checkpoint has {tuple(src.shape)}, the model wants {tuple(dst.shape)}")
                dst.copy_(src)
            else:
                template[k] = src
        return template, extra


def load_dcp_into_model(model: torch.nn.Module, path: str, strict: bool = True, prefix: str = "") -> Tuple[List[str], List[str]]:
    """Returns ``(missing, unexpected)`` like ``load_state_dict``; ``prefix`` is stripped from the checkpoint's names
    (e.g. ``"model."`` for checkpoints written by a wrapper)."""
    state, _ = DCPCheckpointIO().load_checkpoint(path)
    if prefix:
        state = {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}
    own = model.state_dict()
    missing = [k for k in own if k not in state]
    unexpected = [k for k in state if k not in own]
    if strict and (missing or unexpected):
        raise RuntimeError(f"DCP checkpoint does not match the model: missing {missing[:5]}, unexpected {unexpected[:5]}")
    model.load_state_dict({k: v for k, v in state.items() if k in own}, strict=False)
    return missing, unexpected


def dcp_to_single_file(path: str, out_file: str) -> None:
    state, extra = DCPCheckpointIO().load_checkpoint(path)
    torch.save({"state_dict": state, "extra": extra}, out_file)


def single_file_to_dcp(in_file: str, path: str) -> None:
    obj = torch.load(in_file, map_location="cpu", weights_only=False)
    state = obj["state_dict"] if isinstance(obj, dict) and "state_dict" in obj else obj
    DCPCheckpointIO().save_checkpoint(dict(state), path, extra=obj.get("extra") if isinstance(obj, dict) else None)

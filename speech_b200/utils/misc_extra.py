"""Further framework utilities.

* Sequence packing: ``first_fit`` / ``first_fit_decreasing`` / ``first_fit_shuffle`` bin packing of sequence lengths, the length
  histogram, ``create_packing_strategy`` (which lengths share a pack) and ``fill_packing_strategy`` (the packed examples with
  ``seq_start_id`` boundaries).
* Data-store paths: ``is_datastore_path`` (``ais://``, ``s3://``, ``gs://`` ...), ``bucket_and_object_from_uri``,
  ``datastore_path_to_local_path``, ``DataStoreObject`` (a remote object with a local cached copy fetched on first use through the
  registered fetcher), ``open_best``.
* ``str_to_dtype``, ``CastToFloat`` / ``CastToFloatAll`` / ``cast_tensor`` / ``avoid_bfloat16_autocast_context`` / ``monkeypatched`` /
  ``maybe_cast_to_type``.
* ``update_model_config`` (dataclass defaults + user overrides with sub-config handling), ``assert_dataclass_signature_match``.
* ``robust_copy`` (retries with back-off), ``add_optimizer_args`` / ``add_scheduler_args`` / ``add_asr_args`` argparse groups,
  ``is_tarred_path``.

References: ``nemo/utils/{sequence_packing_utils,data_utils,dtype,cast_utils,config_utils,file_utils,arguments}.py``.
"""
from __future__ import annotations

import contextlib
import dataclasses
import inspect
import os
import pathlib
import shutil
import time
from argparse import ArgumentParser
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

__all__ = ["CastToFloat", "CastToFloatAll", "DataStoreObject", "add_asr_args", "add_optimizer_args", "add_scheduler_args", "assert_dataclass_signature_match",
           "avoid_bfloat16_autocast_context", "bucket_and_object_from_uri", "cast_tensor", "create_hist", "create_packing_strategy", "datastore_path_to_local_path",
           "fill_packing_strategy", "first_fit", "first_fit_decreasing", "first_fit_shuffle", "is_datastore_path", "is_tarred_path", "maybe_cast_to_type",
           "monkeypatched", "open_best", "resolve_cache_dir", "robust_copy", "str_to_dtype", "update_model_config"]


# ------------------------------------------------------------------------------------------------ sequence packing
def first_fit(seqlens: Sequence[int], pack_size: int) -> List[List[int]]:
    """Each length goes into the first pack that still has room; a new pack is opened when none has."""
    bins: List[List[int]] = []
    room: List[int] = []
    for s in seqlens:
        for i, r in enumerate(room):
            if s <= r:
                bins[i].append(s)
                room[i] -= s
                break
        else:
            bins.append([s])
            room.append(pack_size - s)
    return bins


def first_fit_decreasing(seqlens: Sequence[int], pack_size: int) -> List[List[int]]:
    return first_fit(sorted(seqlens, reverse=True), pack_size)


def first_fit_shuffle(seqlens: Sequence[int], pack_size: int, seed: int = 0) -> List[List[int]]:
    s = list(seqlens)
    np.random.default_rng(seed).shuffle(s)
    return first_fit(s, pack_size)


def create_hist(dataset: Sequence[Dict[str, Any]], truncate_seq_len: int) -> Tuple[Dict[int, List[Dict[str, Any]]], List[int]]:
    """``{length: [examples of that length]}`` and the count per length 0..truncate_seq_len (longer examples are cut)."""
    by_len: Dict[int, List[Dict[str, Any]]] = {}
    for ex in dataset:
        n = min(len(ex["input_ids"]) - 1, truncate_seq_len)                 # the last token has no next-token target
        by_len.setdefault(n, []).append(ex)
    return by_len, [len(by_len.get(n, [])) for n in range(truncate_seq_len + 1)]


def create_packing_strategy(histogram: Sequence[int], pack_size: int, packing_algorithm: str = "first_fit_shuffle", seed: int = 0) -> Tuple[List[List[int]], Dict[str, float]]:
    seqlens = [n for n, c in enumerate(histogram) for _ in range(c)]
    fn = {"first_fit": first_fit, "first_fit_decreasing": first_fit_decreasing, "first_fit_shuffle": lambda s, p: first_fit_shuffle(s, p, seed)}[packing_algorithm]
    packs = fn(seqlens, pack_size)
    used = sum(sum(p) for p in packs)
    meta = {"dataset_max_seqlen": max(seqlens) if seqlens else 0, "num_packs": len(packs), "packing_factor": len(seqlens) / max(1, len(packs)),
            "packing_efficiency": used / max(1, len(packs) * pack_size)}
    return packs, meta


def fill_packing_strategy(assignments: Sequence[Sequence[int]], sequences: Dict[int, List[Dict[str, Any]]], pack_size: int, pad_id: int = 0, seed: int = 0
                          ) -> List[Dict[str, Any]]:
    """Draws, for every length in every pack, one example of that length (without replacement) and concatenates them:
    ``input_ids``, ``loss_mask`` and ``seq_start_id`` (where each example starts inside the pack)."""
    rng = np.random.default_rng(seed)
    pools = {n: list(rng.permutation(len(v))) for n, v in sequences.items()}
    out = []
    for pack in assignments:
        ids: List[int] = []
        mask: List[int] = []
        starts: List[int] = []
        for n in pack:
            ex = sequences[n][int(pools[n].pop())]
            toks = list(ex["input_ids"])[: n + 1]
            starts.append(len(ids))
            ids += toks
            lm = list(ex.get("loss_mask", [1] * len(toks)))[: len(toks)]
            mask += lm
        out.append({"input_ids": ids, "loss_mask": mask, "seq_start_id": starts})
    return out


# ------------------------------------------------------------------------------------------------ data stores
_STORES = ("ais://", "s3://", "gs://", "msc://", "http://", "https://")


def resolve_cache_dir() -> pathlib.Path:
    return pathlib.Path(os.environ.get("NEMO_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "speech_b200"))


def is_datastore_path(path) -> bool:
    return str(path).startswith(_STORES)


def is_tarred_path(path) -> bool:
    return str(path).endswith((".tar", ".tar.gz", ".tgz"))


def bucket_and_object_from_uri(uri: str) -> Tuple[str, str]:
    if "://" not in uri:
        raise ValueError(f"not a store URI: {uri}")
    rest = uri.split("://", 1)[1]
    bucket, _, obj = rest.partition("/")
    return bucket, obj


def datastore_path_to_local_path(store_path: str) -> str:
    """``<cache>/datastore/<scheme>/<bucket>/<object>``."""
    scheme = store_path.split("://", 1)[0]
    bucket, obj = bucket_and_object_from_uri(store_path)
    return str(resolve_cache_dir() / "datastore" / scheme / bucket / obj)


class DataStoreObject:
    """``local_path`` fetches on first use (``fetch(url, destination)`` — by default the fetcher registered for the URL's scheme
    with ``utils.misc.register_object_store_fetcher``); a plain local path is returned as is."""

    def __init__(self, store_path: str, local_path: Optional[str] = None, get: bool = False, fetch: Optional[Callable[[str, str], Any]] = None):
        self.store_path, self._local, self._fetch = store_path, local_path, fetch
        if get:
            self.get()

    def get(self, force: bool = False) -> str:
        if not is_datastore_path(self.store_path):
            self._local = self.store_path
            return self._local
        dest = self._local or datastore_path_to_local_path(self.store_path)
        if force or not os.path.exists(dest):
            os.makedirs(os.path.dirname(dest), exist_ok=True)
            fetch = self._fetch
            if fetch is None:
                from .misc import _FETCHERS

                fetch = _FETCHERS.get(self.store_path.split("://", 1)[0])
            if fetch is None:
                raise RuntimeError(f"no fetcher registered for {self.store_path.split('://', 1)[0]}:// (this machine has no network by itself)")
            tmp = dest + ".part"
            fetch(self.store_path, tmp)
            os.replace(tmp, dest)
        self._local = dest
        return dest

    @property
    def local_path(self) -> str:
        return self.get()

    def __str__(self):
        return f"{type(self).__name__}: store_path={self.store_path}, local_path={self._local}"


def open_best(path: str, mode: str = "rb", fetch: Optional[Callable[[str, str], Any]] = None):
    """Opens a local file directly and a store object through its cached copy."""
    return open(DataStoreObject(path, fetch=fetch).local_path if is_datastore_path(path) else path, mode)


# ------------------------------------------------------------------------------------------------ dtypes and casting
_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "float": torch.float32, "32": torch.float32, "32-true": torch.float32, "fp16": torch.float16,
           "float16": torch.float16, "half": torch.float16, "16": torch.float16, "16-mixed": torch.float16, "16-true": torch.float16, "bf16": torch.bfloat16,
           "bfloat16": torch.bfloat16, "bf16-mixed": torch.bfloat16, "bf16-true": torch.bfloat16, "bf16-flash": torch.bfloat16, "fp64": torch.float64,
           "float64": torch.float64, "double": torch.float64, "fp8": torch.float8_e4m3fn, "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2}


def str_to_dtype(dtype: Union[str, int, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    key = str(dtype).lower().replace("torch.", "")
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {dtype!r}; known: {sorted(_DTYPES)}")
    return _DTYPES[key]


def cast_tensor(x, from_dtype=torch.float16, to_dtype=torch.float32):
    return x.to(to_dtype) if torch.is_tensor(x) and x.dtype == from_dtype else x


def _cast_all(x, from_dtype, to_dtype):
    if torch.is_tensor(x):
        return cast_tensor(x, from_dtype, to_dtype)
    if isinstance(x, dict):
        return {k: _cast_all(v, from_dtype, to_dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cast_all(v, from_dtype, to_dtype) for v in x)
    return x


@contextlib.contextmanager
def avoid_bfloat16_autocast_context():
    """Inside a bf16 autocast region: run in fp32 instead (for ops whose bf16 kernels are missing or too coarse)."""
    if torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.bfloat16:
        with torch.autocast("cuda", dtype=torch.float32):
            yield
    else:
        yield


class CastToFloat(torch.nn.Module):
    """Runs the wrapped module in fp32 whatever the input dtype and casts the result back."""

    def __init__(self, mod: torch.nn.Module):
        super().__init__()
        self.mod = mod

    def forward(self, x):
        with torch.autocast(x.device.type, enabled=False):
            return self.mod(x.to(torch.float32)).to(x.dtype)


class CastToFloatAll(torch.nn.Module):
    def __init__(self, mod: torch.nn.Module):
        super().__init__()
        self.mod = mod

    def forward(self, *args):
        dt = next((a.dtype for a in args if torch.is_tensor(a) and a.is_floating_point()), torch.float32)
        dev = next((a.device.type for a in args if torch.is_tensor(a)), "cpu")
        with torch.autocast(dev, enabled=False):
            out = self.mod(*[a.to(torch.float32) if torch.is_tensor(a) and a.is_floating_point() else a for a in args])
        return _cast_all(out, torch.float32, dt)


@contextlib.contextmanager
def monkeypatched(obj, name: str, patch):
    old = getattr(obj, name)
    setattr(obj, name, patch)
    try:
        yield obj
    finally:
        setattr(obj, name, old)


def maybe_cast_to_type(x: Any, type_: type) -> Any:
    return None if x is None else type_(x)


# ------------------------------------------------------------------------------------------------ configs
def update_model_config(model_cls_config, update_cfg, drop_missing_subconfigs: bool = True):
    """``model_cls_config``: a dataclass instance (the schema with defaults); ``update_cfg``: a user config.  User values replace
    defaults; optional sub-configs (``train_ds``, ``validation_ds``, ``test_ds``, ``optim``) absent from the user config are dropped
    from the result when ``drop_missing_subconfigs``; keys the user adds inside those sub-configs are accepted."""
    from ..core.config import OmegaConf, open_dict

    base = OmegaConf.create(dataclasses.asdict(model_cls_config) if dataclasses.is_dataclass(model_cls_config) else dict(model_cls_config))
    upd = update_cfg if not isinstance(update_cfg, dict) else OmegaConf.create(update_cfg)
    for sub in ("train_ds", "validation_ds", "test_ds", "optim"):
        holder_b = base.get("model", base)
        holder_u = upd.get("model", upd)
        if sub in holder_b and (sub not in holder_u or holder_u.get(sub) is None) and drop_missing_subconfigs:
            with open_dict(holder_b):
                holder_b.pop(sub)
    return OmegaConf.merge(base, upd)


def assert_dataclass_signature_match(cls: type, datacls: type, ignore_args: Optional[Sequence[str]] = None, remap_args: Optional[Dict[str, str]] = None
                                     ) -> Tuple[bool, Optional[set], Optional[set]]:
    """Whether the constructor arguments of ``cls`` and the fields of ``datacls`` are the same set (after ignoring / renaming):
    ``(match, arguments only in the class, fields only in the dataclass)``."""
    cls_args = set(inspect.signature(cls.__init__).parameters) - {"self", "args", "kwargs"}
    dc_args = {f.name for f in dataclasses.fields(datacls)} - {"_target_"}
    for a in ignore_args or ():
        cls_args.discard(a)
        dc_args.discard(a)
    for old, new in (remap_args or {}).items():
        if old in cls_args:
            cls_args.discard(old)
            cls_args.add(new)
    if cls_args == dc_args:
        return True, None, None
    return False, cls_args - dc_args, dc_args - cls_args


# ------------------------------------------------------------------------------------------------ files, argparse
def robust_copy(src: Union[str, pathlib.Path], dst: Union[str, pathlib.Path], retries: int = 3, backoff: float = 0.5, copy_fn: Callable = shutil.copy2) -> str:
    """Copy with retries (network file systems fail transiently); the copy lands under a temporary name first."""
    src, dst = str(src), str(dst)
    if os.path.isdir(dst):
        dst = os.path.join(dst, os.path.basename(src))
    last: Optional[Exception] = None
    for k in range(retries):
        try:
            tmp = dst + ".part"
            copy_fn(src, tmp)
            os.replace(tmp, dst)
            return dst
        except OSError as e:
            last = e
            time.sleep(backoff * (2 ** k))
    raise OSError(f"copy {src} -> {dst} failed after {retries} attempts: {last}")


def add_optimizer_args(parent: ArgumentParser, optimizer: str = "adam", default_lr: Optional[float] = None, default_opt_args: Optional[Sequence[str]] = None) -> ArgumentParser:
    g = parent.add_argument_group("optimizer")
    g.add_argument("--optimizer", type=str, default=optimizer)
    g.add_argument("--lr", type=float, default=default_lr, required=default_lr is None)
    g.add_argument("--opt_args", default=list(default_opt_args or []), nargs="+", type=str, help="key=value pairs handed to the optimizer")
    return parent


def add_scheduler_args(parent: ArgumentParser) -> ArgumentParser:
    g = parent.add_argument_group("scheduler")
    g.add_argument("--warmup_steps", type=int, default=None)
    g.add_argument("--warmup_ratio", type=float, default=None)
    g.add_argument("--hold_steps", type=int, default=None)
    g.add_argument("--hold_ratio", type=float, default=None)
    g.add_argument("--min_lr", type=float, default=0.0)
    g.add_argument("--last_epoch", type=int, default=-1)
    return parent


def add_asr_args(parent: ArgumentParser) -> ArgumentParser:
    g = parent.add_argument_group("asr")
    g.add_argument("--asr_model", type=str, required=True, help="model file or name")
    g.add_argument("--train_dataset", type=str, required=True)
    g.add_argument("--eval_dataset", type=str, required=True)
    return parent

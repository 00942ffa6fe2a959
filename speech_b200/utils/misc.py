"""Small utilities of the framework layer (one module instead of the reference's many ``nemo/utils/*.py`` files).

* precision: ``HalfPrecisionForAudio`` (cast float batch tensors to the compute dtype except audio), ``resolve_trainer_cfg``
  (``trainer_utils.py:40,115,143``)
* profiling: NVTX range stack (``nvtx.py:35-60``), forward / backward norm dump hooks (``debug_hook.py:185``)
* distributed helpers: ``initialize_distributed``, ``gather_objects``, shared ``temporary_directory`` (``distributed.py:32,66,108``)
* model utils: artifact path helpers, ``inject_model_parallel_rank``, config version upgrade, ``check_lib_version``
* env / import / cast helpers, safe tar extraction (``tar_utils.safe_extract``), ``maybe_download_from_cloud`` (local cache only:
  there is no network in the target environment), ``SequenceLengthResolver`` of the OOMptimizer (``oomptimizer.py:34``)
* ``ShardedCheckpointIO``: per-rank shard files + index for sharded optimizer state, with an asynchronous writer thread
  (role of ``callbacks/dist_ckpt_io.py:72-202``)
* ``object_store_url``: ``s3://`` / ``msc://`` URLs are recognised and rejected with a clear error unless a fetcher is registered
"""
from __future__ import annotations

import contextlib
import importlib
import json
import os
import shutil
import tarfile
import tempfile
import threading
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .logging import logging


# ---------------------------------------------------------------------------------------------- precision
class HalfPrecisionForAudio:
    """Batch transform: float tensors go to ``dtype`` unless their key contains ``audio`` (waveforms stay fp32)."""

    def __init__(self, precision: str = "bf16-mixed"):
        self.dtype = torch.bfloat16 if "bf16" in str(precision) else (torch.float16 if "16" in str(precision) else torch.float32)

    def convert_input(self, batch: Any) -> Any:
        if isinstance(batch, dict):
            return {k: (v if "audio" in k else self._cast(v)) for k, v in batch.items()}
        return batch

    def _cast(self, v):
        if torch.is_tensor(v) and v.is_floating_point():
            return v.to(self.dtype)
        if isinstance(v, (list, tuple)):
            return type(v)(self._cast(x) for x in v)
        if isinstance(v, dict):
            return self.convert_input(v)
        return v


def resolve_trainer_cfg(trainer_cfg) -> Dict[str, Any]:
    """Instantiate ``_target_`` entries of a trainer config (strategy, callbacks, plugins); everything else passes through."""
    from ..core.config import to_container
    from ..core.instantiate import from_config_dict

    cfg = to_container(trainer_cfg, resolve=True) if not isinstance(trainer_cfg, dict) else dict(trainer_cfg)
    if isinstance(cfg.get("strategy"), dict) and "_target_" in cfg["strategy"]:
        cfg["strategy"] = from_config_dict(cfg["strategy"])
    if cfg.get("callbacks"):
        cfg["callbacks"] = [from_config_dict(c) if isinstance(c, dict) and "_target_" in c else c for c in cfg["callbacks"]]
    cfg.pop("plugins", None)
    return cfg


# ---------------------------------------------------------------------------------------------- profiling
_nvtx_stack: List[str] = []


def nvtx_range_push(msg: str, enabled: bool = True) -> None:
    if enabled and torch.cuda.is_available():
        _nvtx_stack.append(msg)
        torch.cuda.nvtx.range_push(msg)


def nvtx_range_pop(msg: Optional[str] = None, enabled: bool = True) -> None:
    if enabled and torch.cuda.is_available() and _nvtx_stack:
        top = _nvtx_stack.pop()
        if msg is not None and top != msg:
            raise RuntimeError(f"NVTX range mismatch: popping '{msg}' but '{top}' is open")
        torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def nvtx_range(msg: str, enabled: bool = True):
    nvtx_range_push(msg, enabled)
    try:
        yield
    finally:
        nvtx_range_pop(msg, enabled)


def register_debug_hooks(module: torch.nn.Module, sink: Optional[Callable[[str], None]] = None, every_n: int = 1) -> List[Any]:
    """Log the L2 norm of every sub-module's outputs (forward) and output gradients (backward)."""
    sink = sink or logging.info
    handles = []
    counter = {"n": 0}

    def norm_of(x):
        if torch.is_tensor(x) and x.is_floating_point():
            return float(x.detach().float().norm())
        if isinstance(x, (list, tuple)):
            vals = [norm_of(v) for v in x]
            vals = [v for v in vals if v is not None]
            return sum(v * v for v in vals) ** 0.5 if vals else None
        return None

    for name, m in module.named_modules():
        if not name:
            continue

        def fwd(mod, inp, out, name=name):
            counter["n"] += 1
            if counter["n"] % every_n == 0:
                v = norm_of(out)
                if v is not None:
                    sink(f"debug_info_forward/{name}: {v:.6g}")

        def bwd(mod, gin, gout, name=name):
            v = norm_of(gout)
            if v is not None:
                sink(f"debug_info_backward/{name}: {v:.6g}")

        handles.append(m.register_forward_hook(fwd))
        handles.append(m.register_full_backward_hook(bwd))
    return handles


# ---------------------------------------------------------------------------------------------- distributed helpers
def initialize_distributed(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Initialise ``torch.distributed`` from the launcher's environment; returns (local_rank, rank, world_size)."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(local)
        dist.init_process_group(backend, rank=rank, world_size=world)
    return local, rank, world


def gather_objects(partial: List[Any], main_rank: Optional[int] = None) -> Optional[List[Any]]:
    """Concatenate per-rank lists on every rank (or only on ``main_rank``)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(partial)
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, partial)
    if main_rank is not None and dist.get_rank() != main_rank:
        return None
    return [x for part in out for x in part]


@contextlib.contextmanager
def temporary_directory():
    """One temporary directory shared by all ranks (created by rank 0, removed after a barrier)."""
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    path = [tempfile.mkdtemp() if (not distributed or dist.get_rank() == 0) else None]
    if distributed:
        dist.broadcast_object_list(path, src=0)
    try:
        yield path[0]
    finally:
        if distributed:
            dist.barrier()
        if not distributed or dist.get_rank() == 0:
            shutil.rmtree(path[0], ignore_errors=True)


# ---------------------------------------------------------------------------------------------- model utils
def inject_model_parallel_rank(filepath: str, tp_rank: int = 0, tp_size: int = 1, pp_rank: int = 0, pp_size: int = 1) -> str:
    """``dir/file.ckpt`` → ``dir/mp_rank_XX[_YYY]/file.ckpt`` when model parallelism is on."""
    if tp_size <= 1 and pp_size <= 1:
        return filepath
    d, f = os.path.split(filepath)
    sub = f"mp_rank_{tp_rank:02d}" if pp_size <= 1 else f"tp_rank_{tp_rank:02d}_pp_rank_{pp_rank:03d}"
    return os.path.join(d, sub, f)


def maybe_update_config_version(cfg):
    """Old configs used ``cls`` + ``params``; rewrite them as ``_target_`` + inline parameters."""
    from ..core.config import OmegaConf, to_container

    c = to_container(cfg, resolve=False) if not isinstance(cfg, dict) else dict(cfg)

    def fix(node):
        if isinstance(node, dict):
            if "cls" in node and "params" in node and "_target_" not in node:
                new = {"_target_": node["cls"], **(node["params"] or {})}
                return {k: fix(v) for k, v in new.items()}
            return {k: fix(v) for k, v in node.items()}
        if isinstance(node, list):
            return [fix(v) for v in node]
        return node

    return OmegaConf.create(fix(c))


def check_lib_version(lib_name: str, checked_version: str, operator) -> Tuple[Optional[bool], str]:
    try:
        mod = importlib.import_module(lib_name)
    except ImportError:
        return None, f"{lib_name} is not installed"
    ver = getattr(mod, "__version__", None)
    if ver is None:
        return None, f"{lib_name} has no __version__"

    def key(v):
        return tuple(int(p) for p in "".join(ch if ch.isdigit() or ch == "." else " " for ch in v).split()[0].split(".") if p)

    ok = operator(key(ver), key(checked_version))
    return ok, f"{lib_name} {ver} {'satisfies' if ok else 'does not satisfy'} the requirement {checked_version}"


# ---------------------------------------------------------------------------------------------- env / import / cast
def get_envbool(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    if v.lower() in ("1", "true", "t", "yes", "y", "on"):
        return True
    if v.lower() in ("0", "false", "f", "no", "n", "off", ""):
        return False
    raise ValueError(f"environment variable {name}={v!r} is not a boolean")


def get_envint(name: str, default: Optional[int] = None) -> Optional[int]:
    v = os.environ.get(name)
    return default if v is None else int(v)


def safe_import(module: str, alt: Any = None) -> Tuple[Any, bool]:
    try:
        return importlib.import_module(module), True
    except Exception:  # noqa: BLE001
        return alt, False


@contextlib.contextmanager
def avoid_float16_autocast_context():
    """Inside fp16 autocast switch to bf16 (or fp32) for numerically fragile blocks."""
    if torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.float16:
        with torch.autocast("cuda", dtype=torch.bfloat16 if torch.cuda.is_bf16_supported() else torch.float32):
            yield
    else:
        yield


def cast_all(x, from_dtype=torch.float16, to_dtype=torch.float32):
    if torch.is_tensor(x):
        return x.to(to_dtype) if x.dtype == from_dtype else x
    if isinstance(x, dict):
        return {k: cast_all(v, from_dtype, to_dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(cast_all(v, from_dtype, to_dtype) for v in x)
    return x


# ---------------------------------------------------------------------------------------------- archives / downloads
def safe_extract(tar: tarfile.TarFile, path: str = ".", members: Optional[Iterable[tarfile.TarInfo]] = None) -> None:
    """Extract refusing absolute paths, ``..`` components and links that point outside ``path``."""
    root = os.path.realpath(path)
    todo = list(members) if members is not None else tar.getmembers()
    for m in todo:
        dest = os.path.realpath(os.path.join(path, m.name))
        if os.path.isabs(m.name) or not (dest == root or dest.startswith(root + os.sep)):
            raise ValueError(f"refusing to extract '{m.name}' outside of '{path}'")
        if m.issym() or m.islnk():
            target = os.path.realpath(os.path.join(os.path.dirname(dest), m.linkname))
            if not (target == root or target.startswith(root + os.sep)):
                raise ValueError(f"refusing to extract link '{m.name}' -> '{m.linkname}'")
    for m in todo:
        tar.extract(m, path)


_FETCHERS: Dict[str, Callable[[str, str], str]] = {}


def register_object_store_fetcher(scheme: str, fn: Callable[[str, str], str]) -> None:
    _FETCHERS[scheme] = fn


def object_store_url(path: str) -> Optional[str]:
    for scheme in ("s3://", "msc://", "gs://", "ais://"):
        if str(path).startswith(scheme):
            return scheme[:-3]
    return None


def maybe_download_from_cloud(url: str, filename: str, subfolder: Optional[str] = None, cache_dir: Optional[str] = None,
                              refresh_cache: bool = False) -> str:
    """Return the cached copy of ``url + filename``; without network access only an existing cache entry (or a registered
    fetcher for the URL scheme) can satisfy the request."""
    cache_dir = cache_dir or os.environ.get("NEMO_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "speech_b200")
    dest_dir = os.path.join(cache_dir, subfolder) if subfolder else cache_dir
    dest = os.path.join(dest_dir, filename)
    if os.path.exists(dest) and not refresh_cache:
        return dest
    scheme = object_store_url(url) or url.split("://", 1)[0]
    if scheme in _FETCHERS:
        os.makedirs(dest_dir, exist_ok=True)
        return _FETCHERS[scheme](url + filename, dest)
    raise FileNotFoundError(f"{filename} is not in the local cache ({dest_dir}) and no fetcher is registered for '{scheme}://' URLs")


# ---------------------------------------------------------------------------------------------- OOMptimizer helper
class SequenceLengthResolver:
    """Maps one bucket (max input length, max output length) to concrete tensor shapes for a model's input schema
    (``{"inputs": [{"name", "type", "seq_length": "input"|"output", "vocab_size"}]}``)."""

    def __init__(self, schema: dict):
        self.schema = schema

    def __call__(self, batch_size: int, input_len: int, output_len: int, device="cpu") -> Dict[str, torch.Tensor]:
        out = {}
        for item in self.schema["inputs"]:
            L = input_len if item.get("seq_length", "input") == "input" else output_len
            t = str(item.get("type", ""))
            if t == "lengths" or "Lengths" in t:
                out[item["name"]] = torch.full((batch_size,), L, dtype=torch.long, device=device)
            elif t == "labels" or "Labels" in t:
                out[item["name"]] = torch.randint(0, int(item.get("vocab_size") or 2), (batch_size, L), device=device)
            else:
                out[item["name"]] = torch.randn(batch_size, L, device=device)
        return out


# ---------------------------------------------------------------------------------------------- sharded checkpoint IO
class ShardedCheckpointIO:
    """Every rank writes ``<dir>/shard_<rank>.pt`` (its slice of sharded state) and rank 0 writes ``index.json``; ``save``
    can run on a background thread (``async_save=True``) and is finalised by ``wait()`` — before the next save and at exit."""

    def __init__(self, async_save: bool = False):
        self.async_save = async_save
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    @staticmethod
    def _rank_world() -> Tuple[int, int]:
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
        return 0, 1

    def save(self, state: Dict[str, Any], directory: str, common: Optional[Dict[str, Any]] = None) -> None:
        self.wait()
        rank, world = self._rank_world()
        os.makedirs(directory, exist_ok=True)
        cpu = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in state.items()}     # snapshot before returning

        def work():
            try:
                tmp = os.path.join(directory, f".shard_{rank}.tmp")
                torch.save(cpu, tmp)
                os.replace(tmp, os.path.join(directory, f"shard_{rank}.pt"))
                if rank == 0:
                    with open(os.path.join(directory, "index.json"), "w") as f:
                        json.dump({"world_size": world, "keys": sorted(cpu), "common": common or {}}, f)
            except BaseException as e:  # noqa: BLE001
                self._error = e

        if self.async_save:
            self._thread = threading.Thread(target=work, daemon=True)
            self._thread.start()
        else:
            work()
            self.wait()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise e

    def load(self, directory: str, rank: Optional[int] = None) -> Dict[str, Any]:
        r, world = self._rank_world()
        rank = r if rank is None else rank
        with open(os.path.join(directory, "index.json")) as f:
            idx = json.load(f)
        if idx["world_size"] != world and rank >= idx["world_size"]:
            raise ValueError(f"checkpoint was written by {idx['world_size']} ranks; rank {rank} has no shard")
        return torch.load(os.path.join(directory, f"shard_{rank}.pt"), map_location="cpu", weights_only=False)

    def load_all(self, directory: str) -> List[Dict[str, Any]]:
        with open(os.path.join(directory, "index.json")) as f:
            idx = json.load(f)
        return [torch.load(os.path.join(directory, f"shard_{r}.pt"), map_location="cpu", weights_only=False)
                for r in range(idx["world_size"])]


# ------------------------------------------------------------------------------------------------ model utilities
def wrap_training_step(fn):
    """Decorator for ``training_step``: a ``'log'`` entry in the returned dictionary (the older way of reporting step metrics)
    is taken out and sent through ``self.log_dict`` (reference ``utils/model_utils.py:470-478``)."""
    import functools

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        out = fn(self, *args, **kwargs)
        if isinstance(out, dict) and "log" in out:
            self.log_dict(out.pop("log"))
        return out
    return wrapper


def uninject_model_parallel_rank(filepath: str) -> str:
    """Inverse of :func:`inject_model_parallel_rank`: ``dir/mp_rank_01/x.ckpt`` -> ``dir/x.ckpt``."""
    filepath = str(filepath)
    parent = os.path.basename(os.path.dirname(filepath))
    if any(tag in parent for tag in ("mp_rank", "tp_rank", "fsdp_shard")):
        return os.path.join(os.path.dirname(os.path.dirname(filepath)), os.path.basename(filepath))
    return filepath


def ckpt_to_dir(filepath: str) -> str:
    """Directory that holds a sharded checkpoint named like the file: ``a/b/step=10.ckpt`` -> ``a/b/step=10``."""
    filepath = str(filepath)
    return filepath[: -len(".ckpt")] if filepath.endswith(".ckpt") else filepath


def import_class_by_path(path: str):
    """``"package.module.Class"`` -> the class object."""
    import importlib

    mod, _, name = path.rpartition(".")
    return getattr(importlib.import_module(mod), name)


def resolve_subclass_pretrained_model_info(base_class) -> List[Any]:
    """Pretrained-model records of ``base_class`` and of every subclass that has been imported, each tagged with its class,
    sorted and without duplicates."""
    seen, out = set(), []

    def walk(cls):
        for sub in cls.__subclasses__():
            walk(sub)
        lst = getattr(cls, "list_available_models", None)
        for info in (lst() or []) if lst is not None else []:
            if getattr(info, "class_", None) is None:
                info.class_ = cls
            key = (getattr(info, "pretrained_model_name", repr(info)), info.class_.__name__)
            if key not in seen:
                seen.add(key)
                out.append(info)
    walk(base_class)
    return sorted(out, key=lambda i: (getattr(i, "pretrained_model_name", ""), i.class_.__name__))


def param_is_not_shared(param) -> bool:
    return not getattr(param, "shared", False)


def unwrap_model(model, module_instances: Optional[Tuple[type, ...]] = None):
    """Strip wrapper modules (anything with a ``.module`` attribute of the given types, or any wrapper when no types are given);
    lists are unwrapped element-wise."""
    if isinstance(model, (list, tuple)):
        return type(model)(unwrap_model(m, module_instances) for m in model)
    while hasattr(model, "module") and (module_instances is None or isinstance(model, module_instances)):
        model = model.module
    return model


def parse_dataset_as_name(name: str) -> str:
    """Log prefix of a validation / test set from its manifest path: base name without extension, ``manifest`` and separators
    stripped (``/data/dev_other_manifest.json`` -> ``dev_other``)."""
    base = os.path.splitext(os.path.basename(str(name).rstrip("/")))[0] if os.path.splitext(str(name))[1] else os.path.basename(str(name).rstrip("/"))
    base = base.replace("-", "_")
    for junk in ("manifest", "dataset"):
        base = base.replace(junk, "")
    base = "_".join(p for p in base.split("_") if p)
    return base or "dataset"


def unique_names_check(name_list: Optional[List[str]]) -> None:
    """Warn when two validation / test sets would log under the same prefix (their metrics would overwrite each other)."""
    if not name_list:
        return
    seen: Dict[str, int] = {}
    for n in name_list:
        seen[n] = seen.get(n, 0) + 1
    dup = [n for n, c in seen.items() if c > 1]
    if dup:
        from .logging import logging

        logging.warning(f"dataset names are not unique, metrics will collide: {dup}")

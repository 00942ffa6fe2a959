"""YAML configuration tree with attribute access, interpolation, resolvers and CLI overrides.

This is the framework's own stand-in for the Hydra + OmegaConf pair that the reference
uses for every entry point (reference: ``nemo/core/config/hydra_runner.py:26-145``).  It
implements the subset of behaviour that model code and ``.nemo`` files rely on:

* ``DictConfig`` / ``ListConfig`` nodes with ``cfg.a.b`` and ``cfg["a"]["b"]`` access,
* ``${a.b}`` interpolation and function resolvers ``${multiply:x,y}``, ``${sum:...}``,
  ``${gpu_name:}`` (reference resolvers: ``hydra_runner.py:46-52``),
* ``key=value`` / ``+key=value`` / ``~key`` command line overrides,
* YAML load / save with ``resolve=True`` as used when a model config is written into a
  checkpoint (reference: ``nemo/core/classes/common.py:902``),
* ``open_dict`` and struct mode, ``MISSING`` (``???``) values.
"""
from __future__ import annotations

import contextlib
import copy
import functools
import io
import os
import re
import sys
from typing import Any, Callable, Dict, Iterable, List, Optional, Union

import yaml

MISSING = "???"

_RESOLVERS: Dict[str, Callable[..., Any]] = {}


class ConfigError(Exception):
    pass


class MissingMandatoryValue(ConfigError):
    pass


class ConfigKeyError(ConfigError, KeyError):
    pass


def register_resolver(name: str, fn: Callable[..., Any], replace: bool = True) -> None:
    if name in _RESOLVERS and not replace:
        return
    _RESOLVERS[name] = fn


def _gpu_name() -> str:
    try:
        import torch

        if torch.cuda.is_available():
            return torch.cuda.get_device_name(0).replace(" ", "_")
    except Exception:  # pragma: no cover
        pass
    return "cpu"


def _num(x):
    if isinstance(x, (int, float)):
        return x
    try:
        return int(x)
    except (TypeError, ValueError):
        return float(x)


register_resolver("multiply", lambda *a: functools.reduce(lambda x, y: x * y, [_num(v) for v in a]))
register_resolver("sum", lambda *a: sum(_num(v) for v in a))
register_resolver("gpu_name", lambda *a: _gpu_name())
register_resolver("oc.env", lambda k, d=None: os.environ.get(k, d))
register_resolver("now", lambda fmt="%Y-%m-%d_%H-%M-%S": __import__("datetime").datetime.now().strftime(fmt))

_INTERP = re.compile(r"\$\{([^${}]*)\}")


def _wrap(value: Any, parent: Optional["_Node"], key: Any) -> Any:
    if isinstance(value, _Node):
        if value._parent is not None and value._parent is not parent:
            value = copy.deepcopy(value)
        value._parent, value._key = parent, key
        return value
    if isinstance(value, dict):
        return DictConfig(value, _parent=parent, _key=key)
    if isinstance(value, (list, tuple)):
        return ListConfig(value, _parent=parent, _key=key)
    if hasattr(value, "__dataclass_fields__") and not isinstance(value, type):
        import dataclasses

        return DictConfig(dataclasses.asdict(value), _parent=parent, _key=key)
    return value


class _Node:
    _parent: Optional["_Node"]
    _key: Any

    def _root(self) -> "_Node":
        n = self
        while n._parent is not None:
            n = n._parent
        return n

    def _full_key(self, key: Any = None) -> str:
        parts: List[str] = []
        n: Optional[_Node] = self
        while n is not None and n._parent is not None:
            parts.append(str(n._key))
            n = n._parent
        parts.reverse()
        if key is not None:
            parts.append(str(key))
        return ".".join(parts)

    # ---- interpolation -------------------------------------------------
    def _select_from(self, path: str, origin: "_Node") -> Any:
        node: Any = self._root()
        if path.startswith("."):
            # relative interpolation: one dot = sibling of the node holding the value
            node = origin
            path = path[1:]
            while path.startswith("."):
                node = node._parent if node._parent is not None else node
                path = path[1:]
        if path == "":
            return node
        for part in _split_path(path):
            if isinstance(node, DictConfig):
                if part not in node._content:
                    raise ConfigKeyError(f"Interpolation key '{path}' not found")
                node = node._get(part, resolve=True)
            elif isinstance(node, ListConfig):
                node = node._get(int(part), resolve=True)
            else:
                raise ConfigKeyError(f"Interpolation key '{path}' not found")
        return node

    def _resolve_value(self, value: Any) -> Any:
        if not isinstance(value, str) or "${" not in value:
            return value
        origin = self

        def one(expr: str) -> Any:
            expr = expr.strip()
            if ":" in expr and not expr.startswith("."):
                name, _, argstr = expr.partition(":")
                if name in _RESOLVERS:
                    args = [_parse_scalar(a.strip()) for a in _split_args(argstr)] if argstr.strip() else []
                    return _RESOLVERS[name](*args)
                raise ConfigError(f"Unknown resolver '{name}' in '${{{expr}}}'")
            return self._select_from(expr, origin)

        # Resolve innermost expressions first so nesting works.
        for _ in range(32):
            m = _INTERP.fullmatch(value) if isinstance(value, str) else None
            if m:
                value = one(m.group(1))
                if isinstance(value, str) and "${" in value:
                    continue
                return value
            if not isinstance(value, str) or "${" not in value:
                return value
            new = _INTERP.sub(lambda mm: str(one(mm.group(1))), value, count=1)
            if new == value:
                return value
            value = new
        raise ConfigError(f"Interpolation too deep: {value}")


def _split_path(path: str) -> List[str]:
    out: List[str] = []
    for part in path.split("."):
        if "[" in part:
            head, *idx = part.replace("]", "").split("[")
            if head:
                out.append(head)
            out.extend(idx)
        elif part != "":
            out.append(part)
    return out


def _split_args(s: str) -> List[str]:
    depth, cur, out = 0, "", []
    for ch in s:
        if ch in "[{(":
            depth += 1
        elif ch in "]})":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    out.append(cur)
    return out


def _parse_scalar(text: str) -> Any:
    if not isinstance(text, str):
        return text
    if "${" in text:
        return text
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


class DictConfig(_Node):
    def __init__(self, content: Optional[dict] = None, _parent=None, _key=None, flags=None):
        object.__setattr__(self, "_content", {})
        object.__setattr__(self, "_parent", _parent)
        object.__setattr__(self, "_key", _key)
        object.__setattr__(self, "_struct", None)
        if content is not None:
            if isinstance(content, DictConfig):
                content = content._content
            for k, v in content.items():
                self._content[k] = _wrap(copy.deepcopy(v) if isinstance(v, _Node) else v, self, k)

    # struct mode ---------------------------------------------------------
    def _is_struct(self) -> bool:
        n: Optional[_Node] = self
        while n is not None:
            s = getattr(n, "_struct", None)
            if s is not None:
                return bool(s)
            n = n._parent
        return False

    def _get(self, key, resolve=True):
        v = self._content[key]
        if resolve and isinstance(v, str):
            if v == MISSING:
                raise MissingMandatoryValue(f"Missing mandatory value: {self._full_key(key)}")
            v = self._resolve_value(v)
        return v

    # mapping protocol ----------------------------------------------------
    def __getattr__(self, key):
        if key.startswith("__") and key.endswith("__"):
            raise AttributeError(key)
        try:
            return self._get(key)
        except KeyError:
            if self._is_struct():
                raise AttributeError(f"Key '{key}' is not in struct ({self._full_key(key)})")
            return None

    def __getitem__(self, key):
        try:
            return self._get(key)
        except KeyError:
            raise ConfigKeyError(f"Missing key {self._full_key(key)}")

    def __setattr__(self, key, value):
        if key in ("_content", "_parent", "_key", "_struct"):
            object.__setattr__(self, key, value)
        else:
            self.__setitem__(key, value)

    def __setitem__(self, key, value):
        if key not in self._content and self._is_struct():
            raise ConfigKeyError(f"Key '{key}' is not in struct ({self._full_key(key)})")
        self._content[key] = _wrap(value, self, key)

    def __delattr__(self, key):
        del self._content[key]

    def __delitem__(self, key):
        del self._content[key]

    def __contains__(self, key):
        return key in self._content

    def __iter__(self):
        return iter(self._content)

    def __len__(self):
        return len(self._content)

    def __eq__(self, other):
        if isinstance(other, DictConfig):
            return to_container(self) == to_container(other)
        if isinstance(other, dict):
            return to_container(self) == other
        return NotImplemented

    def __ne__(self, other):
        r = self.__eq__(other)
        return r if r is NotImplemented else not r

    __hash__ = None  # type: ignore

    def keys(self):
        return self._content.keys()

    def values(self):
        return [self._get(k) for k in self._content]

    def items(self):
        return [(k, self._get(k)) for k in self._content]

    def get(self, key, default=None):
        if key in self._content:
            v = self._content[key]
            if isinstance(v, str) and v == MISSING:
                return default
            v = self._get(key)
            return default if v is None and default is not None else v
        return default

    def pop(self, key, *default):
        if key in self._content:
            v = self._get(key, resolve=False)
            del self._content[key]
            return v
        if default:
            return default[0]
        raise ConfigKeyError(key)

    def setdefault(self, key, default=None):
        if key not in self._content:
            self[key] = default
        return self[key]

    def update(self, other=None, **kw):
        src = dict(other.items_raw() if isinstance(other, DictConfig) else (other or {}))
        src.update(kw)
        for k, v in src.items():
            self[k] = v

    def items_raw(self):
        return list(self._content.items())

    def copy(self):
        return copy.deepcopy(self)

    def __deepcopy__(self, memo):
        new = DictConfig()
        for k, v in self._content.items():
            new._content[k] = _wrap(copy.deepcopy(v, memo), new, k)
        object.__setattr__(new, "_struct", self._struct)
        return new

    def __repr__(self):
        return repr(to_container(self, resolve=False))

    def __getstate__(self):
        return {"content": to_container(self, resolve=False), "struct": self._struct}

    def __setstate__(self, state):
        DictConfig.__init__(self, state["content"])
        object.__setattr__(self, "_struct", state.get("struct"))

    def __dir__(self):
        return list(self._content.keys())


class ListConfig(_Node):
    def __init__(self, content: Optional[Iterable] = None, _parent=None, _key=None):
        self._content: List[Any] = []
        self._parent = _parent
        self._key = _key
        self._struct = None
        for i, v in enumerate(content or []):
            self._content.append(_wrap(copy.deepcopy(v) if isinstance(v, _Node) else v, self, i))

    def _get(self, idx, resolve=True):
        v = self._content[idx]
        if resolve and isinstance(v, str):
            v = self._resolve_value(v)
        return v

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return ListConfig([self._get(i) for i in range(*idx.indices(len(self._content)))])
        return self._get(idx)

    def __setitem__(self, idx, value):
        self._content[idx] = _wrap(value, self, idx)

    def __len__(self):
        return len(self._content)

    def __iter__(self):
        for i in range(len(self._content)):
            yield self._get(i)

    def __contains__(self, item):
        return any(v == item for v in self)

    def append(self, value):
        self._content.append(_wrap(value, self, len(self._content)))

    def extend(self, values):
        for v in values:
            self.append(v)

    def index(self, v):
        return list(self).index(v)

    def __eq__(self, other):
        if isinstance(other, (ListConfig, list, tuple)):
            return to_container(self) == (to_container(other) if isinstance(other, ListConfig) else list(other))
        return NotImplemented

    __hash__ = None  # type: ignore

    def __add__(self, other):
        return ListConfig(list(self) + list(other))

    def __deepcopy__(self, memo):
        new = ListConfig()
        for i, v in enumerate(self._content):
            new._content.append(_wrap(copy.deepcopy(v, memo), new, i))
        return new

    def __repr__(self):
        return repr(to_container(self, resolve=False))

    def __getstate__(self):
        return {"content": to_container(self, resolve=False)}

    def __setstate__(self, state):
        ListConfig.__init__(self, state["content"])


def to_container(cfg: Any, resolve: bool = False, throw_on_missing: bool = False) -> Any:
    if isinstance(cfg, DictConfig):
        out = {}
        for k in cfg._content:
            raw = cfg._content[k]
            if isinstance(raw, _Node):
                out[k] = to_container(raw, resolve, throw_on_missing)
            elif resolve and isinstance(raw, str) and "${" in raw:
                out[k] = to_container(cfg._get(k), resolve, throw_on_missing)
            else:
                if throw_on_missing and raw == MISSING:
                    raise MissingMandatoryValue(cfg._full_key(k))
                out[k] = raw
        return out
    if isinstance(cfg, ListConfig):
        out_l = []
        for i, raw in enumerate(cfg._content):
            if isinstance(raw, _Node):
                out_l.append(to_container(raw, resolve, throw_on_missing))
            elif resolve and isinstance(raw, str) and "${" in raw:
                out_l.append(to_container(cfg._get(i), resolve, throw_on_missing))
            else:
                out_l.append(raw)
        return out_l
    if isinstance(cfg, dict):
        return {k: to_container(v, resolve, throw_on_missing) for k, v in cfg.items()}
    if isinstance(cfg, (list, tuple)):
        return [to_container(v, resolve, throw_on_missing) for v in cfg]
    return cfg


class _Loader(yaml.SafeLoader):
    pass


# YAML 1.1 parses "1e-3" as a string; accept it as a float like OmegaConf does.
_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(
        r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
        |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
        |\.[0-9_]+(?:[eE][-+][0-9]+)?
        |[-+]?\.(?:inf|Inf|INF)
        |\.(?:nan|NaN|NAN))$""",
        re.X,
    ),
    list("-+0123456789."),
)


class _Dumper(yaml.SafeDumper):
    def ignore_aliases(self, data):
        return True


class OmegaConf:
    """Namespace with the handful of static helpers model code uses."""

    @staticmethod
    def create(obj: Any = None) -> Union[DictConfig, ListConfig]:
        if obj is None:
            return DictConfig({})
        if isinstance(obj, str):
            obj = yaml.load(obj, Loader=_Loader)
            if obj is None:
                return DictConfig({})
        if isinstance(obj, (DictConfig, ListConfig)):
            return copy.deepcopy(obj)
        out = _wrap(obj, None, None)
        if not isinstance(out, _Node):
            raise ConfigError(f"Cannot create a config from {type(obj)}")
        return out

    @staticmethod
    def structured(obj: Any) -> DictConfig:
        import dataclasses

        if isinstance(obj, type):
            obj = obj()
        return DictConfig(dataclasses.asdict(obj))

    @staticmethod
    def load(path_or_file) -> Union[DictConfig, ListConfig]:
        if hasattr(path_or_file, "read"):
            data = yaml.load(path_or_file, Loader=_Loader)
        else:
            with open(path_or_file, "r", encoding="utf-8") as f:
                data = yaml.load(f, Loader=_Loader)
        return OmegaConf.create(data if data is not None else {})

    @staticmethod
    def to_yaml(cfg: Any, resolve: bool = False, sort_keys: bool = False) -> str:
        return yaml.dump(
            to_container(cfg, resolve=resolve), Dumper=_Dumper, default_flow_style=False, sort_keys=sort_keys,
            allow_unicode=True,
        )

    @staticmethod
    def save(config: Any, f, resolve: bool = False) -> None:
        text = OmegaConf.to_yaml(config, resolve=resolve)
        if hasattr(f, "write"):
            f.write(text)
        else:
            with open(f, "w", encoding="utf-8") as fh:
                fh.write(text)

    to_container = staticmethod(to_container)

    @staticmethod
    def to_object(cfg):
        return to_container(cfg, resolve=True)

    @staticmethod
    def resolve(cfg: Union[DictConfig, ListConfig]) -> None:
        resolved = to_container(cfg, resolve=True)
        if isinstance(cfg, DictConfig):
            for k, v in resolved.items():
                cfg._content[k] = _wrap(v, cfg, k)
        else:
            cfg._content = [_wrap(v, cfg, i) for i, v in enumerate(resolved)]

    @staticmethod
    def merge(*configs: Any) -> DictConfig:
        out = OmegaConf.create({})
        for c in configs:
            if c is None:
                continue
            if not isinstance(c, _Node):
                c = OmegaConf.create(c)
            _merge_into(out, c)
        return out

    @staticmethod
    def set_struct(cfg: DictConfig, value: Optional[bool]) -> None:
        object.__setattr__(cfg, "_struct", value)

    @staticmethod
    def is_struct(cfg: DictConfig) -> bool:
        return cfg._is_struct()

    @staticmethod
    def is_config(obj) -> bool:
        return isinstance(obj, _Node)

    @staticmethod
    def is_dict(obj) -> bool:
        return isinstance(obj, DictConfig)

    @staticmethod
    def is_list(obj) -> bool:
        return isinstance(obj, ListConfig)

    @staticmethod
    def is_missing(cfg: DictConfig, key) -> bool:
        return key in cfg._content and cfg._content[key] == MISSING

    @staticmethod
    def select(cfg: _Node, key: str, default: Any = None) -> Any:
        node: Any = cfg
        try:
            for part in _split_path(key):
                if isinstance(node, DictConfig):
                    node = node[part]
                elif isinstance(node, ListConfig):
                    node = node[int(part)]
                else:
                    return default
        except (KeyError, IndexError, ConfigError):
            return default
        return node

    @staticmethod
    def update(cfg: DictConfig, key: str, value: Any, force_add: bool = True, merge: bool = False) -> None:
        parts = _split_path(key)
        node: Any = cfg
        with open_dict(cfg) if force_add else contextlib.nullcontext():
            for part in parts[:-1]:
                if isinstance(node, ListConfig):
                    node = node[int(part)]
                    continue
                if part not in node or not isinstance(node._content[part], _Node):
                    node[part] = {}
                node = node._content[part]
            last = parts[-1]
            if isinstance(node, ListConfig):
                node[int(last)] = value
            elif merge and isinstance(value, (dict, DictConfig)) and isinstance(node._content.get(last), DictConfig):
                _merge_into(node._content[last], OmegaConf.create(value))
            else:
                node[last] = value

    @staticmethod
    def register_new_resolver(name: str, fn: Callable[..., Any], replace: bool = False) -> None:
        register_resolver(name, fn, replace=True)

    @staticmethod
    def from_dotlist(dotlist: List[str]) -> DictConfig:
        cfg = OmegaConf.create({})
        apply_overrides(cfg, dotlist)
        return cfg


def _merge_into(dst: DictConfig, src: DictConfig) -> None:
    for k, v in src._content.items():
        if isinstance(v, DictConfig) and isinstance(dst._content.get(k), DictConfig):
            _merge_into(dst._content[k], v)
        else:
            dst._content[k] = _wrap(copy.deepcopy(v), dst, k)


@contextlib.contextmanager
def open_dict(cfg: DictConfig):
    prev = cfg._struct
    object.__setattr__(cfg, "_struct", False)
    try:
        yield cfg
    finally:
        object.__setattr__(cfg, "_struct", prev)


@contextlib.contextmanager
def read_write(cfg):
    yield cfg


def apply_overrides(cfg: DictConfig, overrides: Iterable[str]) -> DictConfig:
    """Apply Hydra-style ``a.b=value``, ``+a.b=value``, ``++a.b=value`` and ``~a.b`` overrides."""
    for ov in overrides:
        ov = ov.strip()
        if not ov:
            continue
        if ov.startswith("~"):
            parts = _split_path(ov[1:].split("=")[0])
            node: Any = cfg
            for p in parts[:-1]:
                node = node[p]
            node.pop(parts[-1], None)
            continue
        if "=" not in ov:
            raise ConfigError(f"Override '{ov}' is not of the form key=value")
        key, _, val = ov.partition("=")
        force = key.startswith("+")
        key = key.lstrip("+")
        value = _parse_scalar(val)
        if value == "null":
            value = None
        OmegaConf.update(cfg, key, value, force_add=True)
    return cfg


def hydra_runner(config_path: Optional[str] = ".", config_name: Optional[str] = None, schema: Any = None):
    """Decorator for ``main(cfg)`` entry points.

    Behaves like the reference's launcher decorator (``hydra_runner.py:53-143``): the YAML
    named by ``--config-path`` / ``--config-name`` (or the decorator defaults) is loaded,
    ``key=value`` overrides from ``sys.argv`` are applied, the working directory is left
    unchanged and no ``.hydra`` output directory is written.

    ``-m`` / ``--multirun`` turns comma-separated override values into a sweep (``lr=1e-3,1e-4 model.size=small,large`` is four
    jobs, Cartesian product, first key slowest).  Jobs run one after the other in this process by default; with
    ``hydra.launcher.n_jobs=N`` (or ``hydra/launcher=processes``) each job is a child process running the same script with
    its own overrides, at most N at a time, each pinned to one GPU of ``hydra.launcher.gpus=[0,1,...]`` when given
    (the reference's process launcher, ``core/utils/process_launcher/launcher.py``).  The wrapper then returns the list of
    results (task return values, or ``(overrides, return code, log path)`` for child processes).
    """

    def decorator(task_function: Callable[[DictConfig], Any]):
        @functools.wraps(task_function)
        def wrapper(cfg_passthrough: Optional[DictConfig] = None, argv: Optional[List[str]] = None):
            if cfg_passthrough is not None:
                return task_function(cfg_passthrough)
            args = list(sys.argv[1:] if argv is None else argv)
            cpath, cname, overrides = config_path, config_name, []
            multirun = False
            i = 0
            while i < len(args):
                a = args[i]
                if a in ("-m", "--multirun"):
                    multirun = True
                    i += 1
                elif a in ("--config-path", "-cp"):
                    cpath = args[i + 1]
                    i += 2
                elif a.startswith("--config-path="):
                    cpath = a.split("=", 1)[1]
                    i += 1
                elif a in ("--config-name", "-cn"):
                    cname = args[i + 1]
                    i += 2
                elif a.startswith("--config-name="):
                    cname = a.split("=", 1)[1]
                    i += 1
                else:
                    overrides.append(a)
                    i += 1
            cfg = OmegaConf.create({})
            if schema is not None:
                cfg = OmegaConf.structured(schema)
            if cname is not None:
                base = cpath or "."
                if not os.path.isabs(base):
                    mod = sys.modules.get(task_function.__module__)
                    mod_dir = os.path.dirname(os.path.abspath(getattr(mod, "__file__", "."))) if mod else "."
                    cand = os.path.join(mod_dir, base)
                    base = cand if os.path.isdir(cand) else base
                fname = cname if cname.endswith((".yaml", ".yml")) else cname + ".yaml"
                cfg = OmegaConf.merge(cfg, OmegaConf.load(os.path.join(base, fname)))
            if multirun:
                launcher = {o.split("=", 1)[0]: o.split("=", 1)[1] for o in overrides if o.startswith(("hydra.launcher.", "hydra/launcher="))}
                overrides = [o for o in overrides if not o.startswith(("hydra.launcher.", "hydra/launcher="))]
                jobs = expand_multirun_overrides(overrides)
                n_jobs = int(launcher.get("hydra.launcher.n_jobs", 0) or 0)
                if n_jobs > 0 or launcher.get("hydra/launcher") == "processes":
                    from ..utils.extras import ProcessLauncher

                    gpus = launcher.get("hydra.launcher.gpus")
                    gpu_ids = [int(g) for g in gpus.strip("[]").split(",") if g.strip()] if gpus else None
                    mod = sys.modules.get(task_function.__module__)
                    script = os.path.abspath(getattr(mod, "__file__", sys.argv[0]))
                    base_cmd = [sys.executable, script] + ([f"--config-path={cpath}"] if cpath else []) + ([f"--config-name={cname}"] if cname else [])
                    pl = ProcessLauncher(base_cmd, gpu_ids=gpu_ids, max_parallel=n_jobs or None,
                                         log_dir=launcher.get("hydra.launcher.log_dir", "multirun"))
                    return pl.launch(jobs)
                results = []
                for job in jobs:
                    c = OmegaConf.create(to_container(cfg, resolve=False))
                    apply_overrides(c, job)
                    results.append(task_function(c))
                return results
            apply_overrides(cfg, overrides)
            return task_function(cfg)

        return wrapper

    return decorator


def expand_multirun_overrides(overrides: Sequence[str]) -> List[List[str]]:
    """``["lr=1e-3,1e-4", "size=small", "aug=[a,b],[c]"]`` -> one override list per job.  Commas inside brackets, braces,
    parentheses or quotes do not split; the first swept key varies slowest."""
    def split_top(v: str) -> List[str]:
        parts, depth, cur, quote = [], 0, "", None
        for ch in v:
            if quote:
                cur += ch
                if ch == quote:
                    quote = None
                continue
            if ch in "\"'":
                quote = ch
            elif ch in "[{(":
                depth += 1
            elif ch in "]})":
                depth -= 1
            if ch == "," and depth == 0:
                parts.append(cur)
                cur = ""
            else:
                cur += ch
        return parts + [cur]

    jobs: List[List[str]] = [[]]
    for o in overrides:
        if "=" not in o:
            jobs = [j + [o] for j in jobs]
            continue
        k, v = o.split("=", 1)
        vals = split_top(v)
        jobs = [j + [f"{k}={x}"] for j in jobs for x in vals]
    return jobs


def cfg_get(cfg: Any, key: str, default: Any = None) -> Any:
    """``cfg.get`` that also works for plain dicts and ``None``."""
    if cfg is None:
        return default
    if isinstance(cfg, (dict, DictConfig)):
        v = cfg.get(key, default)
        return default if v is None else v
    return getattr(cfg, key, default)

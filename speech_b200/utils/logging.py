"""Rank-aware logger and process-wide application state.

``logging`` prints on global rank 0 by default, supports "log once" messages and extra file
handlers (reference: ``nemo/utils/nemo_logging.py``); ``AppState`` is the singleton that holds
ranks, world size, log directories and the folder of the ``.nemo`` file being restored
(reference: ``nemo/utils/app_state.py:33``).
"""
from __future__ import annotations

import enum
import logging as _pylogging
import os
import sys
import threading
from typing import Any, Dict, Optional, Set


class logging_mode(enum.IntEnum):
    EACH = 0
    ONCE = 1


def get_rank() -> int:
    for k in ("RANK", "SLURM_PROCID", "OMPI_COMM_WORLD_RANK"):
        if k in os.environ:
            try:
                return int(os.environ[k])
            except ValueError:
                pass
    return 0


def is_global_rank_zero() -> bool:
    return get_rank() == 0


class _Formatter(_pylogging.Formatter):
    COLORS = {"WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[31;1m", "DEBUG": "\033[36m"}

    def __init__(self, color: bool):
        super().__init__("[speech_b200 %(levelname).1s %(asctime)s %(module)s:%(lineno)d rank:%(rank)s] %(message)s",
                         "%Y-%m-%d %H:%M:%S")
        self.color = color

    def format(self, record):
        record.rank = get_rank()
        s = super().format(record)
        if self.color and record.levelname in self.COLORS:
            s = self.COLORS[record.levelname] + s + "\033[0m"
        return s


class Logger:
    NOTSET, DEBUG, INFO, WARNING, ERROR, CRITICAL = 0, 10, 20, 30, 40, 50

    def __init__(self):
        self._logger = _pylogging.getLogger("speech_b200")
        self._logger.propagate = False
        self._once: Set[str] = set()
        self._lock = threading.Lock()
        self._handlers: Dict[str, _pylogging.Handler] = {}
        if not self._logger.handlers:
            h = _pylogging.StreamHandler(sys.stderr)
            h.setFormatter(_Formatter(color=sys.stderr.isatty()))
            self._logger.addHandler(h)
            self._handlers["stream"] = h
        self._logger.setLevel(int(os.environ.get("SPEECH_B200_LOG_LEVEL", _pylogging.INFO)))
        self.rank0_only = os.environ.get("SPEECH_B200_LOG_ALL_RANKS", "0") != "1"

    def setLevel(self, level: int):
        self._logger.setLevel(level)

    set_verbosity = setLevel

    def getEffectiveLevel(self) -> int:
        return self._logger.getEffectiveLevel()

    get_verbosity = getEffectiveLevel

    def add_file_handler(self, path: str):
        if path in self._handlers:
            return
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        h = _pylogging.FileHandler(path)
        h.setFormatter(_Formatter(color=False))
        self._logger.addHandler(h)
        self._handlers[path] = h

    def add_err_file_handler(self, path: str):
        if path in self._handlers:
            return
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        h = _pylogging.FileHandler(path)
        h.setLevel(_pylogging.ERROR)
        h.setFormatter(_Formatter(color=False))
        self._logger.addHandler(h)
        self._handlers[path] = h

    def remove_file_handlers(self):
        for k, h in list(self._handlers.items()):
            if k != "stream":
                self._logger.removeHandler(h)
                h.close()
                del self._handlers[k]

    def _log(self, level: int, msg: Any, *args, mode=logging_mode.EACH, all_ranks: bool = False, **kw):
        if self.rank0_only and not all_ranks and not is_global_rank_zero() and level < _pylogging.ERROR:
            return
        msg = str(msg)
        if mode == logging_mode.ONCE:
            with self._lock:
                if msg in self._once:
                    return
                self._once.add(msg)
        self._logger.log(level, msg, *args, stacklevel=3, **kw)

    def debug(self, msg, *a, **k):
        self._log(_pylogging.DEBUG, msg, *a, **k)

    def info(self, msg, *a, **k):
        self._log(_pylogging.INFO, msg, *a, **k)

    def warning(self, msg, *a, **k):
        self._log(_pylogging.WARNING, msg, *a, **k)

    warn = warning

    def error(self, msg, *a, **k):
        self._log(_pylogging.ERROR, msg, *a, **k)

    def critical(self, msg, *a, **k):
        self._log(_pylogging.CRITICAL, msg, *a, **k)

    def exception(self, msg, *a, **k):
        self._log(_pylogging.ERROR, msg, *a, exc_info=True, **k)


logging = Logger()


class _Singleton(type):
    _instances: Dict[type, Any] = {}
    _lock = threading.Lock()

    def __call__(cls, *args, **kwargs):
        with cls._lock:
            if cls not in cls._instances:
                cls._instances[cls] = super().__call__(*args, **kwargs)
        return cls._instances[cls]


class AppState(metaclass=_Singleton):
    def __init__(self):
        self.reset()

    def reset(self):
        self.device_id: Optional[int] = None
        self.local_rank: Optional[int] = None
        self.global_rank: Optional[int] = None
        self.world_size: Optional[int] = None
        self.tensor_model_parallel_size: int = 1
        self.tensor_model_parallel_rank: int = 0
        self.pipeline_model_parallel_size: int = 1
        self.data_parallel_size: Optional[int] = None
        self.data_parallel_rank: Optional[int] = None
        self.model_parallel_size: Optional[int] = None
        self.log_dir: Optional[str] = None
        self.exp_dir: Optional[str] = None
        self.name: Optional[str] = None
        self.version: Optional[str] = None
        self.checkpoint_name: Optional[str] = None
        self.create_checkpoint_callback: bool = True
        self.checkpoint_callback_params: Optional[dict] = None
        self.cmd_args = None
        self.restore: bool = False
        self.model_restore_path: Optional[str] = None
        self.nemo_file_folder: Optional[str] = None
        self.is_model_being_restored: bool = False
        self._all_model_restore_paths = []
        self._model_guid_map: Dict[str, Any] = {}
        self._nvtx_ranges: bool = False
        self.random_seed: Optional[int] = None

    def register_model_guid(self, guid: str, restoration_path: Optional[str] = None):
        self._model_guid_map[guid] = {"guid": guid, "restoration_path": restoration_path}

    def get_model_metadata_from_guid(self, guid: str):
        return self._model_guid_map.get(guid)

    def reset_model_guid_registry(self):
        self._model_guid_map.clear()

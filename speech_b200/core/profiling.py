"""Step-window profiling and scheduled freezing, driven by keys of the model config.

``StepHooks`` is owned by every :class:`ModelPT` and runs in its ``on_train_batch_start`` / ``on_train_batch_end``.  Config
keys (the reference reads the same ones in ``core/classes/modelPT.py:1783-2050``):

``nsys_profile: {enabled, start_step, end_step, ranks: [0], gen_shape: false}``
    Brackets the steps ``[start_step, end_step]`` with ``cudaProfilerStart`` / ``cudaProfilerStop`` on the listed ranks, so
    that an external ``nsys profile --capture-range=cudaProfilerApi`` (or ``ncu --profile-from-start off``) records only
    that window, and pushes an NVTX range per step; ``gen_shape`` records argument shapes in the autograd NVTX ranges.
``memory_profile: {enabled, start_step, end_step, rank: 0, output_path}``
    Records the CUDA caching-allocator history over the window and dumps
    ``<output_path>/memory_profile_rank<r>.pickle`` (viewable with PyTorch's memory visualiser).
``chakra_profile: {enabled, start_step, end_step, warmup_steps, active_steps, trace_dir}``
    Execution-trace capture: an ``ExecutionTraceObserver`` writes ``<trace_dir>/<job>_chakra/rank-<r>.json`` while a Kineto
    profile of the same steps goes to ``<trace_dir>/<job>_kineto``.  Cannot be combined with ``nsys_profile``.
``freeze_updates: {enabled, modules: {name: n | [first, last]}}``
    Sub-module ``name`` is frozen while the update count (1-based) is ``<= n`` (for ever if ``-1``), or lies in
    ``[first, last]`` (``last = -1``: for ever); it is kept in train mode while frozen so that dropout and batch statistics
    behave as in normal training (``modelPT.py:1993-2013``).
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch

from ..utils.logging import logging


def _window(cfg, what: str):
    s, e = cfg.get("start_step", 0), cfg.get("end_step", 0)
    if type(s) is not int or type(e) is not int:
        raise ValueError(f"{what} start_step / end_step must be integers, found {type(s).__name__} / {type(e).__name__}")
    if e < s:
        raise ValueError(f"{what} end_step must be greater than or equal to start_step")
    return s, e


class StepHooks:
    def __init__(self, cfg, rank: int = 0, cuda_api=None):
        """``cuda_api`` (tests): an object with ``profiler_start / profiler_stop / nvtx_push / nvtx_pop / record_memory /
        dump_memory``; by default the calls go to ``torch.cuda``."""
        self.rank = rank
        self.api = cuda_api or _TorchCudaApi()
        get = (lambda k: cfg.get(k, None)) if cfg is not None and hasattr(cfg, "get") else (lambda k: None)
        self.nsys = self.mem = self.chakra = None
        self.freeze: Optional[Dict[str, Any]] = None
        n = get("nsys_profile")
        if n is not None and n is not False and n.get("enabled", False):
            s, e = _window(n, "nsys_profile")
            self.nsys = {"start": s, "end": e, "ranks": list(n.get("ranks", [0])), "gen_shape": bool(n.get("gen_shape", False)),
                         "started": False, "done": False, "ctx": None}
            logging.info(f"nsys profiling window: steps {s}..{e} on ranks {self.nsys['ranks']}")
        m = get("memory_profile")
        if m is not None and m.get("enabled", False):
            s, e = _window(m, "memory_profile")
            out = m.get("output_path", None)
            if out is None or not os.path.isdir(out):
                raise ValueError(f"memory_profile.output_path ({out}) is not set or is not a directory")
            self.mem = {"start": s, "end": e, "rank": int(m.get("rank", 0)), "out": out, "started": False, "done": False}
        c = get("chakra_profile")
        if c is not None and c.get("enabled", False):
            if self.nsys is not None:
                raise ValueError("chakra_profile and nsys_profile cannot both be enabled")
            s, e = _window(c, "chakra_profile")
            td = c.get("trace_dir", None)
            if td is None or not os.path.isdir(td):
                raise ValueError(f"chakra_profile.trace_dir ({td}) is not set or does not exist")
            job = os.environ.get("SLURM_JOB_ID", "0")
            self.chakra = {"start": s, "end": e, "warmup": int(c.get("warmup_steps", 0)), "active": int(c.get("active_steps", 1)),
                           "et_dir": os.path.join(td, f"{job}_chakra"), "kineto_dir": os.path.join(td, f"{job}_kineto"),
                           "running": False, "et": None, "prof": None}
            os.makedirs(self.chakra["et_dir"], exist_ok=True)
            os.makedirs(self.chakra["kineto_dir"], exist_ok=True)
        f = get("freeze_updates")
        if f is not None and f.get("enabled", False):
            mods = {k: (list(v) if isinstance(v, (list, tuple)) or hasattr(v, "__iter__") and not isinstance(v, (str, int)) else int(v))
                    for k, v in dict(f.get("modules", {})).items()}
            for k, v in mods.items():
                if isinstance(v, list) and len(v) != 2:
                    raise ValueError(f"freeze_updates.modules.{k}: a list must be [first_step, last_step]")
            self.freeze = {"modules": mods, "is_frozen": {k: False for k in mods}}

    @property
    def active(self) -> bool:
        return any(x is not None for x in (self.nsys, self.mem, self.chakra, self.freeze))

    # ------------------------------------------------------------------ per step
    def batch_start(self, model, batch_idx: int, global_step: int) -> None:
        c = self.chakra
        if c is not None and not c["running"] and c["start"] <= global_step <= c["end"]:
            from torch.profiler import ExecutionTraceObserver, ProfilerActivity, profile, schedule, tensorboard_trace_handler

            logging.info(f"====== Start chakra profiling from global_step {global_step} ======")
            c["et"] = ExecutionTraceObserver()
            c["et"].register_callback(os.path.join(c["et_dir"], f"rank-{self.rank}.json"))
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            c["prof"] = profile(activities=acts, schedule=schedule(wait=0, warmup=c["warmup"], active=c["active"]),
                                on_trace_ready=tensorboard_trace_handler(c["kineto_dir"]), execution_trace_observer=c["et"])
            c["prof"].start()
            c["running"] = True
        n = self.nsys
        if n is not None and not n["started"] and batch_idx >= n["start"] and self.rank in n["ranks"]:
            logging.info("====== Start nsys profiling ======")
            self.api.profiler_start()
            if n["gen_shape"]:
                n["ctx"] = torch.autograd.profiler.emit_nvtx(record_shapes=True)
                n["ctx"].__enter__()
            n["started"] = True
        if n is not None and n["started"] and not n["done"]:
            self.api.nvtx_push(f"step {global_step}")
        m = self.mem
        if m is not None and not m["started"] and batch_idx >= m["start"] and self.rank == m["rank"]:
            logging.info("====== Start CUDA memory profiling ======")
            self.api.record_memory(True)
            m["started"] = True
        self._apply_freeze(model, global_step + 1)

    def batch_end(self, model, batch_idx: int, global_step: int) -> None:
        c = self.chakra
        if c is not None and c["running"]:
            if global_step - 1 >= c["end"]:
                logging.info(f"====== End chakra profiling at global_step {global_step} ======")
                c["prof"].stop()
                c["et"].unregister_callback()
                c["running"] = False
            elif global_step - 1 >= c["start"]:
                c["prof"].step()
        n = self.nsys
        if n is not None and n["started"] and not n["done"]:
            self.api.nvtx_pop()
            if batch_idx >= n["end"] and self.rank in n["ranks"]:
                logging.info("====== End nsys profiling ======")
                if n["ctx"] is not None:
                    n["ctx"].__exit__(None, None, None)
                    n["ctx"] = None
                self.api.profiler_stop()
                n["done"] = True
        m = self.mem
        if m is not None and m["started"] and not m["done"] and batch_idx >= m["end"] and self.rank == m["rank"]:
            path = os.path.join(m["out"], f"memory_profile_rank{m['rank']}.pickle")
            logging.info(f"====== End CUDA memory profiling; snapshot -> {path} ======")
            self.api.dump_memory(path)
            self.api.record_memory(False)
            m["done"] = True

    def close(self) -> None:
        """End of the run: stop whatever window is still open (training may end inside it)."""
        c = self.chakra
        if c is not None and c["running"]:
            c["prof"].stop()
            c["et"].unregister_callback()
            c["running"] = False
        n = self.nsys
        if n is not None and n["started"] and not n["done"]:
            if n["ctx"] is not None:
                n["ctx"].__exit__(None, None, None)
            self.api.profiler_stop()
            n["done"] = True
        m = self.mem
        if m is not None and m["started"] and not m["done"]:
            self.api.dump_memory(os.path.join(m["out"], f"memory_profile_rank{m['rank']}.pickle"))
            self.api.record_memory(False)
            m["done"] = True

    # ------------------------------------------------------------------ freezing by schedule
    def _apply_freeze(self, model, num_updates: int) -> None:
        f = self.freeze
        if f is None or not model.training:
            return
        for name, steps in f["modules"].items():
            if isinstance(steps, list):
                should = num_updates >= steps[0] and (num_updates <= steps[1] or steps[1] == -1)
            else:
                should = num_updates <= steps or steps == -1
            sub = getattr(model, name)           # a wrong name raises here, at the first step
            if should and not f["is_frozen"][name]:
                _freeze(sub)
                sub.train()
                f["is_frozen"][name] = True
                logging.info(f"froze '{name}' at update {num_updates}")
            elif not should and f["is_frozen"][name]:
                _unfreeze(sub)
                f["is_frozen"][name] = False
                logging.info(f"unfroze '{name}' at update {num_updates}")


def _freeze(m: torch.nn.Module) -> None:
    if hasattr(m, "freeze"):
        m.freeze()
    else:
        for p in m.parameters():
            p.requires_grad = False


def _unfreeze(m: torch.nn.Module) -> None:
    if hasattr(m, "unfreeze"):
        m.unfreeze()
    else:
        for p in m.parameters():
            p.requires_grad = True
    m.train()


class _TorchCudaApi:
    def profiler_start(self):
        if torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStart()

    def profiler_stop(self):
        if torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()

    def nvtx_push(self, name: str):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)

    def nvtx_pop(self):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()

    def record_memory(self, on: bool):
        if torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=100000 if on else None, enabled="all" if on else None)

    def dump_memory(self, path: str):
        if torch.cuda.is_available():
            torch.cuda.memory._dump_snapshot(path)

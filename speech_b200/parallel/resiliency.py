"""Failure and straggler detection on the host.

The reference delegates to ``nvidia-resiliency-ext`` callbacks created by ``exp_manager``
(``utils/exp_manager.py:744-806``: ``StragglerDetectionCallback``, ``FaultToleranceCallback``).  Here the same roles are
implemented with host-side mechanisms only — nothing in this module makes a GPU fault, hang or trap:

* ``HeartbeatMonitor`` — every rank stamps a key in the rendezvous store (or a file) once per step; ranks whose stamp is
  older than ``timeout`` are reported.  The check runs on the host between steps, before the next launch.
* ``StragglerDetectionCallback`` — per-step wall time (and optionally CUDA-event time of the step) is all-gathered every
  ``report_time_interval`` seconds; ranks slower than ``threshold`` × median are logged and exposed as
  ``trainer.callback_metrics['straggler/...']``; can stop training when asked to.
* ``FaultToleranceCallback`` — heartbeat + "last good step" bookkeeping; on a detected dead peer or a raised exception it
  saves an emergency checkpoint (when every rank is still alive to do so) and exits with ``RESTART_EXIT_CODE`` so an outer
  launcher restarts the job, which then resumes from the newest checkpoint (``exp_manager`` resume logic).
* ``check_kernel_status`` — reads the device status word the kernels of this framework write when one of their bounded
  waits runs out, and raises a host exception instead of letting the step continue.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.logging import logging

RESTART_EXIT_CODE = 75     # EX_TEMPFAIL: "try again"


class HeartbeatMonitor:
    def __init__(self, rank: int, world_size: int, timeout: float = 600.0, store=None, directory: Optional[str] = None,
                 clock=time.time):
        self.rank, self.world, self.timeout, self.store, self.dir, self.clock = rank, world_size, timeout, store, directory, clock
        if store is None and directory is None:
            raise ValueError("HeartbeatMonitor needs a torch.distributed store or a directory")
        if directory is not None:
            os.makedirs(directory, exist_ok=True)

    def _key(self, r: int) -> str:
        return f"heartbeat/{r}"

    def beat(self, step: int) -> None:
        payload = json.dumps({"t": self.clock(), "step": int(step)})
        if self.store is not None:
            self.store.set(self._key(self.rank), payload)
        else:
            tmp = os.path.join(self.dir, f"hb_{self.rank}.tmp")
            with open(tmp, "w") as f:
                f.write(payload)
            os.replace(tmp, os.path.join(self.dir, f"hb_{self.rank}.json"))

    def read(self, r: int) -> Optional[Dict[str, Any]]:
        try:
            if self.store is not None:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    return None
                return json.loads(self.store.get(self._key(r)).decode())
            with open(os.path.join(self.dir, f"hb_{r}.json")) as f:
                return json.load(f)
        except (FileNotFoundError, RuntimeError, ValueError):
            return None

    def dead_ranks(self) -> List[int]:
        now = self.clock()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            hb = self.read(r)
            if hb is None or now - float(hb["t"]) > self.timeout:
                out.append(r)
        return out


class StragglerDetectionCallback:
    def __init__(self, report_time_interval: float = 300.0, calc_relative_gpu_perf: bool = True,
                 calc_individual_gpu_perf: bool = True, num_gpu_perf_scores_to_log: int = 5, gpu_relative_perf_threshold: float = 0.7,
                 gpu_individual_perf_threshold: float = 0.7, stop_if_detected: bool = False, clock=time.perf_counter):
        self.interval, self.rel_thr, self.ind_thr = report_time_interval, gpu_relative_perf_threshold, gpu_individual_perf_threshold
        self.stop_if_detected, self.n_log, self.clock = stop_if_detected, num_gpu_perf_scores_to_log, clock
        self.step_times: List[float] = []
        self.best_time: Optional[float] = None
        self._t0 = None
        self._last_report = None
        self.last_report: Dict[str, Any] = {}

    def on_train_batch_start(self, trainer, model, batch, batch_idx):
        self._t0 = self.clock()
        if self._last_report is None:
            self._last_report = self._t0

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if self._t0 is None:
            return
        now = self.clock()
        self.step_times.append(now - self._t0)
        if now - self._last_report >= self.interval:
            self.report(trainer)
            self._last_report = now

    def report(self, trainer=None) -> Dict[str, Any]:
        if not self.step_times:
            return {}
        mine = sorted(self.step_times)[len(self.step_times) // 2]
        self.best_time = mine if self.best_time is None else min(self.best_time, mine)
        self.step_times = []
        times = [mine]
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            objs = [None] * dist.get_world_size()
            dist.all_gather_object(objs, mine)
            times = [float(t) for t in objs]
        med = sorted(times)[len(times) // 2]
        rel = [med / t if t > 0 else 1.0 for t in times]                 # 1.0 = as fast as the median rank
        ind = self.best_time / mine if mine > 0 else 1.0                  # 1.0 = as fast as this rank's own best
        stragglers = [r for r, s in enumerate(rel) if s < self.rel_thr]
        rep = {"relative_perf": rel, "individual_perf": ind, "stragglers": stragglers, "median_step_time": med}
        self.last_report = rep
        if stragglers:
            logging.warning(f"straggler ranks (relative performance < {self.rel_thr}): "
                            + ", ".join(f"{r} ({rel[r]:.2f})" for r in stragglers[: self.n_log]))
        if ind < self.ind_thr:
            logging.warning(f"this rank runs at {ind:.2f} of its own best step time")
        if trainer is not None:
            trainer.callback_metrics["straggler/min_relative_perf"] = min(rel)
            trainer.callback_metrics["straggler/individual_perf"] = ind
            if self.stop_if_detected and stragglers:
                trainer.should_stop = True
        return rep


def check_kernel_status() -> None:
    """Raise if a kernel of this framework reported a timed-out wait (bounded waits write a status word, never trap)."""
    if torch.cuda.is_available():
        from ..ops import native

        native.check_status()


class FaultToleranceCallback:
    def __init__(self, heartbeat_timeout: float = 600.0, check_every_n_steps: int = 1, directory: Optional[str] = None,
                 exit_on_failure: bool = True, save_on_failure: bool = True, check_kernels_every_n_steps: int = 0,
                 max_restarts: Optional[int] = None):
        self.timeout, self.every, self.dir = heartbeat_timeout, check_every_n_steps, directory
        self.exit_on_failure, self.save_on_failure = exit_on_failure, save_on_failure
        self.check_kernels_every = check_kernels_every_n_steps
        self.monitor: Optional[HeartbeatMonitor] = None
        self.failures: List[str] = []

    def setup(self, trainer, model, stage):
        rank = getattr(trainer, "global_rank", 0)
        world = getattr(trainer, "world_size", 1)
        d = self.dir or os.path.join(getattr(trainer, "log_dir", None) or ".", "heartbeats")
        self.monitor = HeartbeatMonitor(rank, world, self.timeout, directory=d)

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if self.monitor is None:
            self.setup(trainer, model, "fit")
        step = getattr(trainer, "global_step", batch_idx)
        self.monitor.beat(step)
        if self.check_kernels_every and step % self.check_kernels_every == 0:
            check_kernel_status()
        if step % max(1, self.every) == 0:
            dead = self.monitor.dead_ranks()
            if dead:
                self.on_failure(trainer, f"no heartbeat from ranks {dead} for more than {self.timeout:.0f} s")

    def on_exception(self, trainer, model, exception):
        self.on_failure(trainer, f"exception on rank {getattr(trainer, 'global_rank', 0)}: {exception!r}", peers_alive=False)

    def on_failure(self, trainer, reason: str, peers_alive: bool = False) -> None:
        self.failures.append(reason)
        logging.error(f"fault tolerance: {reason}")
        if self.save_on_failure and peers_alive and hasattr(trainer, "save_checkpoint"):
            try:
                trainer.save_checkpoint(os.path.join(getattr(trainer, "log_dir", "."), "emergency-last.ckpt"))
            except Exception as e:  # noqa: BLE001
                logging.error(f"emergency checkpoint failed: {e!r}")
        if self.exit_on_failure:
            sys.exit(RESTART_EXIT_CODE)
        trainer.should_stop = True

"""Trainer callbacks: checkpointing with ``.nemo`` export, preemption, wall-clock limit, timers, EMA.

Behaviour follows the reference callbacks:

* ``NeMoModelCheckpoint`` — top-k by monitored metric, ``-last`` / ``-end`` checkpoints,
  ``-unfinished`` marker files written before and removed after each save so that an
  interrupted save is never resumed from, ``.nemo`` export on save / best / train end
  (``nemo/utils/callbacks/nemo_model_checkpoint.py:39-748``).
* ``PreemptionCallback`` — SIGTERM sets a flag on rank 0 that is broadcast once per step; all
  ranks then save ``-last`` and exit 0 (``nemo/utils/callbacks/preemption.py:24-118``).
* ``StatelessTimer`` — stop cleanly after ``max_time_per_run`` (``nemo/utils/exp_manager.py:1423-1487``).
* ``TimingCallback`` — ``train_step_timing in s`` etc. (``exp_manager.py:294-411``).
* ``EMA`` — exponential moving average of weights, swapped in for validation and saved as
  ``-EMA`` twins (``nemo/collections/common/callbacks/ema.py:27-165``).
"""
from __future__ import annotations

import datetime
import glob
import os
import re
import signal
import sys
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..core.trainer import Callback
from .logging import is_global_rank_zero, logging
from .timers import NamedTimer


class NeMoModelCheckpoint(Callback):
    UNFINISHED_CHECKPOINT_SUFFIX = "-unfinished"

    def __init__(self, dirpath: Optional[str] = None, filename: Optional[str] = None, monitor: Optional[str] = "val_loss",
                 mode: str = "min", save_top_k: int = 3, save_last: bool = True, always_save_nemo: bool = False,
                 save_nemo_on_train_end: bool = True, save_best_model: bool = False, postfix: str = ".nemo",
                 every_n_train_steps: Optional[int] = None, every_n_epochs: Optional[int] = None,
                 save_on_train_epoch_end: bool = False, save_weights_only: bool = False,
                 save_last_n_optim_states: int = -1, prefix: Optional[str] = None, verbose: bool = True, **_):
        self.dirpath, self.filename, self.monitor, self.mode = dirpath, filename, monitor, mode
        self.save_top_k, self.save_last = save_top_k, save_last
        self.always_save_nemo, self.save_nemo_on_train_end = always_save_nemo, save_nemo_on_train_end
        self.save_best_model, self.postfix = save_best_model, postfix
        self.every_n_train_steps, self.every_n_epochs = every_n_train_steps, every_n_epochs
        self.save_weights_only = save_weights_only
        self.save_last_n_optim_states = save_last_n_optim_states
        self.prefix = prefix or "model"
        self.best_k_models: Dict[str, float] = {}
        self.best_model_path = ""
        self.best_model_score: Optional[float] = None
        self.last_model_path = ""
        self.previous_best_path = ""
        self._last_saved_step = -1

    # ---------------------------------------------------------------- helpers
    def _better(self, a: float, b: float) -> bool:
        return a < b if self.mode == "min" else a > b

    def format_checkpoint_name(self, trainer, metrics: Dict[str, Any]) -> str:
        tmpl = self.filename or f"{self.prefix}--{{{self.monitor}:.4f}}-{{epoch}}"
        vals = {k: (float(v) if torch.is_tensor(v) else v) for k, v in metrics.items()}
        vals.update(epoch=trainer.current_epoch, step=trainer.global_step)

        def sub(m):
            key, fmt = m.group(1), m.group(2) or ""
            v = vals.get(key, 0.0)
            try:
                return f"{key}=" + format(v, fmt[1:] if fmt else "")
            except (ValueError, TypeError):
                return f"{key}={v}"

        return re.sub(r"\{([A-Za-z0-9_/ ]+)(:[^}]*)?\}", sub, tmpl)

    @classmethod
    def format_checkpoint_unfinished_marker_path(cls, checkpoint_path: str) -> str:
        base, _ = os.path.splitext(checkpoint_path)
        return base + cls.UNFINISHED_CHECKPOINT_SUFFIX

    @classmethod
    def is_checkpoint_unfinished(cls, checkpoint_path: str) -> bool:
        return os.path.exists(cls.format_checkpoint_unfinished_marker_path(checkpoint_path))

    def _barrier(self, trainer):
        if trainer.world_size > 1 and dist.is_initialized():
            dist.barrier()

    def _save(self, trainer, path: str, weights_only: bool = False):
        marker = self.format_checkpoint_unfinished_marker_path(path)
        if trainer.is_global_zero:
            os.makedirs(os.path.dirname(path), exist_ok=True)
            open(marker, "w").close()
        self._barrier(trainer)
        trainer.save_checkpoint(path, weights_only=weights_only or self.save_weights_only)
        if trainer.is_global_zero and os.path.exists(marker):
            os.remove(marker)
        self._barrier(trainer)
        ema = next((c for c in trainer.callbacks if isinstance(c, EMA)), None)
        if ema is not None and ema.initialized:
            with ema.swapped(trainer.model):
                trainer.save_checkpoint(path.replace(".ckpt", "-EMA.ckpt"), weights_only=True)

    def _remove(self, trainer, path: str):
        if trainer.is_global_zero:
            for p in (path, path.replace(".ckpt", "-EMA.ckpt"), self.format_checkpoint_unfinished_marker_path(path)):
                if os.path.exists(p):
                    os.remove(p)

    def _drop_optimizer_states(self, trainer):
        """Keep optimizer states only in the newest ``save_last_n_optim_states`` top-k checkpoints."""
        n = self.save_last_n_optim_states
        if n < 0 or not trainer.is_global_zero:
            return
        paths = sorted(self.best_k_models, key=lambda p: os.path.getmtime(p) if os.path.exists(p) else 0, reverse=True)
        for p in paths[n:]:
            if os.path.exists(p):
                ck = torch.load(p, map_location="cpu", weights_only=False)
                if "optimizer_states" in ck:
                    ck.pop("optimizer_states", None), ck.pop("lr_schedulers", None)
                    torch.save(ck, p)

    # ---------------------------------------------------------------- resume bookkeeping
    def setup(self, trainer, model, stage: str):
        if self.dirpath is None:
            self.dirpath = os.path.join(trainer.log_dir or trainer.default_root_dir, "checkpoints")
        self.nemo_topk_check_previous_run()
        if trainer.is_global_zero:
            self._remove_unfinished_checkpoints()
        self._barrier(trainer)

    def nemo_topk_check_previous_run(self):
        """Rebuild the top-k table from the file names left by earlier runs."""
        self.best_k_models = {}
        if not self.dirpath or not os.path.isdir(self.dirpath) or not self.monitor:
            return
        for path in glob.glob(os.path.join(self.dirpath, "*.ckpt")):
            base = os.path.basename(path)
            if base.endswith("-last.ckpt") or base.endswith("-end.ckpt") or base.endswith("-EMA.ckpt"):
                continue
            if self.is_checkpoint_unfinished(path):
                continue
            m = re.search(re.escape(self.monitor) + r"=(-?[0-9]+\.?[0-9]*(?:e[-+]?[0-9]+)?)", base)
            if m:
                self.best_k_models[path] = float(m.group(1))
        if self.best_k_models:
            best = (min if self.mode == "min" else max)(self.best_k_models, key=self.best_k_models.get)
            self.best_model_path, self.best_model_score = best, self.best_k_models[best]
        while self.save_top_k >= 0 and len(self.best_k_models) > max(self.save_top_k, 0):
            worst = (max if self.mode == "min" else min)(self.best_k_models, key=self.best_k_models.get)
            self.best_k_models.pop(worst)
            if is_global_rank_zero() and os.path.exists(worst):
                os.remove(worst)

    def _remove_unfinished_checkpoints(self):
        if not self.dirpath or not os.path.isdir(self.dirpath):
            return
        for marker in glob.glob(os.path.join(self.dirpath, "*" + self.UNFINISHED_CHECKPOINT_SUFFIX)):
            ck = marker[: -len(self.UNFINISHED_CHECKPOINT_SUFFIX)] + ".ckpt"
            for p in (ck, marker):
                if os.path.exists(p):
                    logging.warning(f"Removing unfinished checkpoint artefact {p}")
                    os.remove(p)

    # ---------------------------------------------------------------- hooks
    def _save_topk(self, trainer, model):
        if trainer.global_step == self._last_saved_step or trainer.sanity_checking:
            return
        self._last_saved_step = trainer.global_step
        metrics = dict(trainer.callback_metrics)
        if self.monitor and self.monitor in metrics and self.save_top_k != 0:
            score = float(metrics[self.monitor])
            path = os.path.join(self.dirpath, self.format_checkpoint_name(trainer, metrics) + ".ckpt")
            keep = self.save_top_k < 0 or len(self.best_k_models) < self.save_top_k or any(
                self._better(score, s) for s in self.best_k_models.values())
            if keep:
                self._save(trainer, path)
                self.best_k_models[path] = score
                if self.save_top_k > 0 and len(self.best_k_models) > self.save_top_k:
                    worst = (max if self.mode == "min" else min)(self.best_k_models, key=self.best_k_models.get)
                    self.best_k_models.pop(worst)
                    self._remove(trainer, worst)
                best = (min if self.mode == "min" else max)(self.best_k_models, key=self.best_k_models.get)
                if best != self.best_model_path:
                    self.previous_best_path, self.best_model_path = self.best_model_path, best
                    self.best_model_score = self.best_k_models[best]
                    if self.save_best_model:
                        model.save_to(os.path.join(self.dirpath, self.prefix + "_best" + self.postfix))
                self._drop_optimizer_states(trainer)
        elif not self.monitor and self.save_top_k != 0:
            path = os.path.join(self.dirpath, self.format_checkpoint_name(trainer, metrics) + ".ckpt")
            self._save(trainer, path)
        if self.save_last:
            self._save_last(trainer)
        if self.always_save_nemo:
            model.save_to(os.path.join(self.dirpath, self.prefix + self.postfix))

    def _save_last(self, trainer):
        path = os.path.join(self.dirpath, f"{self.prefix}--{self.monitor or 'step'}={_metric(trainer, self.monitor):.4f}"
                                          f"-epoch={trainer.current_epoch}-last.ckpt")
        prev = self.last_model_path
        self._save(trainer, path)
        self.last_model_path = path
        if trainer.is_global_zero:
            for old in glob.glob(os.path.join(self.dirpath, "*-last.ckpt")):
                if os.path.abspath(old) != os.path.abspath(path):
                    self._remove(trainer, old)

    def on_validation_end(self, trainer, model):
        if trainer.state_fn == "fit":
            self._save_topk(trainer, model)

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        n = self.every_n_train_steps
        if n and trainer.global_step > 0 and trainer.global_step % n == 0 and trainer.global_step != self._last_saved_step \
                and (batch_idx + 1) % trainer.accumulate_grad_batches == 0:
            self._save_topk(trainer, model)

    def on_train_end(self, trainer, model):
        if trainer.fast_dev_run:
            return
        if self.save_last and trainer.global_step != self._last_saved_step:
            self._save_last(trainer)
        if self.save_best_model and self.best_model_path and os.path.exists(self.best_model_path):
            trainer._restore_checkpoint(self.best_model_path, weights_only=True)
        if self.save_nemo_on_train_end:
            model.save_to(os.path.join(self.dirpath, self.prefix + self.postfix))
        end = os.path.join(self.dirpath, f"{self.prefix}--end.ckpt")
        if trainer._should_stop_steps() or (trainer.max_epochs and trainer.current_epoch >= trainer.max_epochs > 0):
            self._save(trainer, end.replace("--end", f"--{self.monitor or 'step'}={_metric(trainer, self.monitor):.4f}"
                                                     f"-epoch={trainer.current_epoch}-end"), weights_only=False)

    def state_dict(self):
        return {"best_k_models": dict(self.best_k_models), "best_model_path": self.best_model_path,
                "best_model_score": self.best_model_score, "last_model_path": self.last_model_path}

    def load_state_dict(self, state):
        self.best_model_path = state.get("best_model_path", "")
        self.best_model_score = state.get("best_model_score")
        self.last_model_path = state.get("last_model_path", "")


def _metric(trainer, name) -> float:
    v = trainer.callback_metrics.get(name, 0.0) if name else float(trainer.global_step)
    return float(v) if v is not None else 0.0


class PreemptionCallback(Callback):
    def __init__(self, checkpoint_callback: Optional[NeMoModelCheckpoint] = None, sig: Optional[int] = None):
        self.sig = sig if sig is not None else signal.SIGTERM
        self.checkpoint_callback = checkpoint_callback
        self.preemption_enabled = False
        self._interrupted = False
        self._old = None

    @property
    def interrupted(self) -> bool:
        return self._interrupted

    def _broadcast_flag(self, trainer) -> bool:
        if trainer.world_size > 1 and dist.is_initialized():
            t = torch.tensor([int(self._interrupted)], dtype=torch.int32,
                             device=trainer.device if dist.get_backend() == "nccl" else "cpu")
            dist.broadcast(t, 0)
            return bool(t.item())
        return self._interrupted

    def on_train_start(self, trainer, model):
        def handler(signum, frame):
            self._interrupted = True

        try:
            self._old = signal.signal(self.sig, handler)
            self.preemption_enabled = True
        except ValueError:  # not in main thread
            self.preemption_enabled = False

    def on_train_end(self, trainer, model):
        if self.preemption_enabled and self._old is not None:
            signal.signal(self.sig, self._old)

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if not self.preemption_enabled:
            return
        if self._broadcast_flag(trainer):
            logging.info("Received preemption signal: saving a -last checkpoint and exiting")
            ck = self.checkpoint_callback or trainer.checkpoint_callback
            if ck is not None:
                ck._save_last(trainer)
            trainer.interrupted = True
            sys.exit(0)


class StatelessTimer(Callback):
    """Stops training after ``duration`` of wall clock in *this* run (not accumulated over resumes)."""

    def __init__(self, duration: Any = None, interval: str = "step", verbose: bool = True):
        if isinstance(duration, str):
            d, h, m, s = (int(x) for x in duration.split(":"))
            duration = datetime.timedelta(days=d, hours=h, minutes=m, seconds=s)
        elif isinstance(duration, dict):
            duration = datetime.timedelta(**duration)
        self.duration: Optional[datetime.timedelta] = duration
        self._start = None

    def on_fit_start(self, trainer, model):
        self._start = time.monotonic()

    def time_elapsed(self) -> float:
        return 0.0 if self._start is None else time.monotonic() - self._start

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if self.duration is None:
            return
        stop = self.time_elapsed() >= self.duration.total_seconds()
        if trainer.world_size > 1 and dist.is_initialized():
            t = torch.tensor([int(stop)], device=trainer.device if dist.get_backend() == "nccl" else "cpu")
            dist.broadcast(t, 0)
            stop = bool(t.item())
        if stop:
            logging.info("Time limit reached: saving last checkpoint and signalling the trainer to stop")
            ck = trainer.checkpoint_callback
            if ck is not None:
                ck._save_last(trainer)
            trainer.should_stop = True

    def state_dict(self):
        return {}


class TimingCallback(Callback):
    def __init__(self, timer_kwargs: Optional[dict] = None, log_tokens_per_sec: bool = False, sync_cuda: bool = True):
        self.timer = NamedTimer(sync_cuda=sync_cuda, **(timer_kwargs or {}))
        self.log_tokens_per_sec = log_tokens_per_sec

    def _on_start(self, name):
        if self.timer.buffer_size <= 0:
            self.timer.reset(name)
        if self.timer.is_active(name):
            self.timer.stop(name)
        self.timer.start(name)

    def _on_end(self, name, model):
        self.timer.stop(name)
        model.log(name + " in s", torch.as_tensor(self.timer[name]))

    def on_train_batch_start(self, trainer, model, batch, batch_idx):
        self._on_start("train_step_timing")

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        self._on_end("train_step_timing", model)
        if self.log_tokens_per_sec and isinstance(batch, dict) and "num_tokens" in batch:
            dt = self.timer["train_step_timing"]
            model.log("tokens_per_sec_per_gpu", float(batch["num_tokens"]) / max(dt, 1e-9))

    def on_before_backward(self, trainer, model, loss):
        self._on_start("train_backward_timing")

    def on_after_backward(self, trainer, model):
        self._on_end("train_backward_timing", model)

    def on_validation_start(self, trainer, model):
        self._on_start("validation_step_timing")

    def on_validation_end(self, trainer, model):
        self._on_end("validation_step_timing", model)


class EMA(Callback):
    def __init__(self, decay: float = 0.999, validate_original_weights: bool = False, every_n_steps: int = 1,
                 cpu_offload: bool = False):
        if not 0.0 <= decay <= 1.0:
            raise ValueError("EMA decay value must be between 0 and 1")
        self.decay, self.validate_original_weights = decay, validate_original_weights
        self.every_n_steps, self.cpu_offload = every_n_steps, cpu_offload
        self.shadow: List[torch.Tensor] = []
        self.initialized = False
        self._swapped = False

    def _params(self, model):
        return [p for p in model.parameters() if p.requires_grad]

    def on_train_start(self, trainer, model):
        if not self.initialized:
            dev = "cpu" if self.cpu_offload else None
            self.shadow = [p.detach().clone().to(dev) if dev else p.detach().clone() for p in self._params(model)]
            self.initialized = True

    @torch.no_grad()
    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if (batch_idx + 1) % trainer.accumulate_grad_batches != 0 or trainer.global_step % self.every_n_steps != 0:
            return
        params = self._params(model)
        if self.cpu_offload:
            for s, p in zip(self.shadow, params):
                s.lerp_(p.detach().to(s.device), 1.0 - self.decay)
        else:
            torch._foreach_lerp_(self.shadow, [p.detach() for p in params], 1.0 - self.decay)

    @torch.no_grad()
    def swap_model_weights(self, model):
        for s, p in zip(self.shadow, self._params(model)):
            tmp = p.detach().clone()
            p.copy_(s.to(p.device))
            s.copy_(tmp.to(s.device))
        self._swapped = not self._swapped
        for p in model.parameters():
            ar = getattr(p, "_arena", None)
            if ar is not None:
                ar.refresh_lowp()
                break

    def swapped(self, model):
        import contextlib

        @contextlib.contextmanager
        def ctx():
            self.swap_model_weights(model)
            try:
                yield
            finally:
                self.swap_model_weights(model)

        return ctx()

    def on_validation_start(self, trainer, model):
        if self.initialized and not self.validate_original_weights:
            self.swap_model_weights(model)

    def on_validation_end(self, trainer, model):
        if self.initialized and not self.validate_original_weights and self._swapped:
            self.swap_model_weights(model)

    on_test_start = on_validation_start
    on_test_end = on_validation_end

    def state_dict(self):
        return {"shadow": [s.cpu() for s in self.shadow], "decay": self.decay}

    def load_state_dict(self, state):
        sh = state.get("shadow", [])
        if sh:
            self.shadow = list(sh)
            self.initialized = True

    def on_load_checkpoint(self, trainer, model, checkpoint):
        if self.initialized:
            params = self._params(model)
            self.shadow = [s.to("cpu" if self.cpu_offload else p.device) for s, p in zip(self.shadow, params)]


class EarlyStopping(Callback):
    def __init__(self, monitor: str = "val_loss", mode: str = "min", min_delta: float = 0.001, patience: int = 10, **_):
        self.monitor, self.mode, self.min_delta, self.patience = monitor, mode, min_delta, patience
        self.best: Optional[float] = None
        self.wait = 0

    def on_validation_end(self, trainer, model):
        if self.monitor not in trainer.callback_metrics or trainer.sanity_checking:
            return
        cur = float(trainer.callback_metrics[self.monitor])
        improved = self.best is None or (cur < self.best - self.min_delta if self.mode == "min" else cur > self.best + self.min_delta)
        if improved:
            self.best, self.wait = cur, 0
        else:
            self.wait += 1
            if self.wait >= self.patience:
                trainer.should_stop = True

    def state_dict(self):
        return {"best": self.best, "wait": self.wait}

    def load_state_dict(self, state):
        self.best, self.wait = state.get("best"), state.get("wait", 0)


class SkipResumeTrainingValidationLoop(Callback):
    """Marker: after a resume, do not re-run validation for the step that was just validated."""

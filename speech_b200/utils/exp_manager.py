"""Experiment manager: log directory, loggers, checkpoint callback, resume logic, timers.

Config keys and behaviour follow ``nemo/utils/exp_manager.py``: ``ExpManagerConfig``
(``:232-291``); log dir ``exp_dir/name/version`` (``get_log_dir`` ``:1085``); resume picks the
single ``*last.ckpt`` that has no ``-unfinished`` marker, refuses to continue past ``*end.ckpt``
unless ``resume_past_end``, and moves logs of the previous run into ``run_N/``
(``check_resume`` ``:871-1048``); writes ``cmd-args.log`` and ``git-info.log`` (``:793-801``);
adds the timing, EMA, early-stopping, preemption and wall-clock callbacks (``:726-784``).
"""
from __future__ import annotations

import csv
import dataclasses
import glob
import json
import os
import re
import shutil
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

from ..core.config import DictConfig, OmegaConf, to_container
from .callbacks import EMA, EarlyStopping, NeMoModelCheckpoint, PreemptionCallback, StatelessTimer, TimingCallback
from .logging import AppState, is_global_rank_zero, logging


class NotFoundError(Exception):
    pass


class LoggerMisconfigurationError(Exception):
    pass


class CheckpointMisconfigurationError(Exception):
    pass


@dataclass
class CallbackParams:
    filepath: Optional[str] = None
    dirpath: Optional[str] = None
    filename: Optional[str] = None
    monitor: Optional[str] = "val_loss"
    verbose: Optional[bool] = True
    save_last: Optional[bool] = True
    save_top_k: Optional[int] = 3
    save_weights_only: Optional[bool] = False
    mode: Optional[str] = "min"
    auto_insert_metric_name: bool = True
    every_n_epochs: Optional[int] = 1
    every_n_train_steps: Optional[int] = None
    train_time_interval: Optional[Any] = None
    prefix: Optional[str] = None
    postfix: str = ".nemo"
    save_best_model: bool = False
    always_save_nemo: bool = False
    save_nemo_on_train_end: Optional[bool] = True
    model_parallel_size: Optional[int] = None
    save_on_train_epoch_end: Optional[bool] = False
    async_save: Optional[bool] = False
    save_last_n_optim_states: Optional[int] = -1


@dataclass
class StepTimingParams:
    reduction: Optional[str] = "mean"
    sync_cuda: Optional[bool] = False
    buffer_size: Optional[int] = 1


@dataclass
class EMAParams:
    enable: Optional[bool] = False
    decay: Optional[float] = 0.999
    cpu_offload: Optional[bool] = False
    validate_original_weights: Optional[bool] = False
    every_n_steps: int = 1


@dataclass
class EarlyStoppingParams:
    monitor: str = "val_loss"
    mode: str = "min"
    min_delta: float = 0.001
    patience: int = 10
    verbose: bool = True
    strict: bool = True


@dataclass
class ExpManagerConfig:
    explicit_log_dir: Optional[str] = None
    exp_dir: Optional[str] = None
    name: Optional[str] = None
    version: Optional[str] = None
    use_datetime_version: Optional[bool] = True
    resume_if_exists: Optional[bool] = False
    resume_past_end: Optional[bool] = False
    resume_ignore_no_checkpoint: Optional[bool] = False
    resume_from_checkpoint: Optional[str] = None
    create_tensorboard_logger: Optional[bool] = True
    summary_writer_kwargs: Optional[Dict[Any, Any]] = None
    create_wandb_logger: Optional[bool] = False
    wandb_logger_kwargs: Optional[Dict[Any, Any]] = None
    create_mlflow_logger: Optional[bool] = False
    mlflow_logger_kwargs: Optional[Dict[Any, Any]] = None
    create_dllogger_logger: Optional[bool] = False
    dllogger_logger_kwargs: Optional[Dict[Any, Any]] = None
    create_clearml_logger: Optional[bool] = False
    clearml_logger_kwargs: Optional[Dict[Any, Any]] = None
    create_neptune_logger: Optional[bool] = False
    neptune_logger_kwargs: Optional[Dict[Any, Any]] = None
    create_checkpoint_callback: Optional[bool] = True
    checkpoint_callback_params: Optional[CallbackParams] = field(default_factory=CallbackParams)
    create_early_stopping_callback: Optional[bool] = False
    early_stopping_callback_params: Optional[EarlyStoppingParams] = field(default_factory=EarlyStoppingParams)
    create_preemption_callback: Optional[bool] = True
    files_to_copy: Optional[List[str]] = None
    log_step_timing: Optional[bool] = True
    log_delta_step_timing: Optional[bool] = False
    step_timing_kwargs: Optional[StepTimingParams] = field(default_factory=StepTimingParams)
    log_local_rank_0_only: Optional[bool] = False
    log_global_rank_0_only: Optional[bool] = False
    disable_validation_on_resume: Optional[bool] = True
    ema: Optional[EMAParams] = field(default_factory=EMAParams)
    max_time_per_run: Optional[str] = None
    seconds_to_sleep: float = 5
    create_straggler_detection_callback: Optional[bool] = False
    create_fault_tolerance_callback: Optional[bool] = False
    log_tflops_per_sec_per_gpu: Optional[bool] = True


# ---------------------------------------------------------------------- loggers
class BaseLogger:
    def __init__(self, save_dir: str, name: str = "", version: str = ""):
        self.save_dir, self.name, self.version = save_dir, name, version
        self.log_dir = save_dir

    def log_metrics(self, metrics: Dict[str, float], step: int): ...
    def log_hyperparams(self, params: Dict[str, Any]): ...
    def finalize(self, status: str = "success"): ...


class JSONLLogger(BaseLogger):
    """One JSON object per logging call in ``metrics.jsonl`` — always available, no dependencies."""

    def __init__(self, save_dir, name="", version=""):
        super().__init__(save_dir, name, version)
        os.makedirs(save_dir, exist_ok=True)
        self.path = os.path.join(save_dir, "metrics.jsonl")

    def log_metrics(self, metrics, step):
        with open(self.path, "a") as f:
            f.write(json.dumps({"step": step, "time": time.time(), **metrics}) + "\n")

    def log_hyperparams(self, params):
        with open(os.path.join(self.save_dir, "hparams.json"), "w") as f:
            json.dump(params, f, indent=1, default=str)


class TensorBoardLogger(BaseLogger):
    def __init__(self, save_dir, name="", version="", **kwargs):
        super().__init__(save_dir, name, version)
        from torch.utils.tensorboard import SummaryWriter

        self.writer = SummaryWriter(log_dir=save_dir, **(kwargs or {}))

    def log_metrics(self, metrics, step):
        for k, v in metrics.items():
            self.writer.add_scalar(k, v, step)

    def log_hyperparams(self, params):
        self.writer.add_text("hparams", "```\n" + OmegaConf.to_yaml(params) + "\n```")

    def finalize(self, status="success"):
        self.writer.flush()
        self.writer.close()


class WandbLogger(BaseLogger):
    def __init__(self, save_dir, name="", version="", **kwargs):
        super().__init__(save_dir, name, version)
        import wandb

        kwargs.setdefault("mode", os.environ.get("WANDB_MODE", "offline"))
        self.run = wandb.init(dir=save_dir, name=kwargs.pop("name", name), **kwargs)

    def log_metrics(self, metrics, step):
        self.run.log(metrics, step=step)

    def finalize(self, status="success"):
        self.run.finish()


class MLFlowLogger(BaseLogger):
    def __init__(self, save_dir, name="", version="", **kwargs):
        super().__init__(save_dir, name, version)
        import mlflow  # noqa: F401  (optional dependency)

        self.mlflow = mlflow
        mlflow.set_tracking_uri(kwargs.get("tracking_uri", "file:" + os.path.join(save_dir, "mlruns")))
        mlflow.set_experiment(kwargs.get("experiment_name", name))
        self.run = mlflow.start_run(run_name=kwargs.get("run_name", version))

    def log_metrics(self, metrics, step):
        self.mlflow.log_metrics(metrics, step=step)

    def finalize(self, status="success"):
        self.mlflow.end_run()


class ClearMLLogger(BaseLogger):
    """ClearML task logger (reference ``nemo/utils/loggers/clearml_logger.py``): scalars go to the task's logger, one series
    per metric name; the optional package is imported on construction."""

    def __init__(self, save_dir, name="", version="", **kwargs):
        super().__init__(save_dir, name, version)
        from clearml import Task

        self.task = Task.init(project_name=kwargs.get("project", name) or "speech_b200", task_name=kwargs.get("task", version) or name,
                              output_uri=kwargs.get("output_uri", None), reuse_last_task_id=False)
        self.log_cfg = bool(kwargs.get("log_cfg", False))

    def log_metrics(self, metrics, step):
        lg = self.task.get_logger()
        for k, v in metrics.items():
            lg.report_scalar(title=k, series=k, value=float(v), iteration=int(step))

    def log_hyperparams(self, params):
        self.task.connect(dict(params) if isinstance(params, dict) else {"config": str(params)})

    def finalize(self, status="success"):
        self.task.close()


class NeptuneLogger(BaseLogger):
    """Neptune run logger (the reference hands ``neptune_logger_kwargs`` to Lightning's NeptuneLogger)."""

    def __init__(self, save_dir, name="", version="", **kwargs):
        super().__init__(save_dir, name, version)
        import neptune

        kwargs.setdefault("name", name)
        self.run = neptune.init_run(**kwargs)
        self.prefix = kwargs.get("prefix", "training")

    def log_metrics(self, metrics, step):
        for k, v in metrics.items():
            self.run[f"{self.prefix}/{k}"].append(float(v), step=int(step))

    def log_hyperparams(self, params):
        self.run["hyperparams"] = dict(params) if isinstance(params, dict) else str(params)

    def finalize(self, status="success"):
        self.run.stop()


class DLLogger(JSONLLogger):
    """DLLogger-style JSON stream (``DLLL`` prefix per line)."""

    def log_metrics(self, metrics, step):
        with open(os.path.join(self.save_dir, "dllogger.json"), "a") as f:
            f.write("DLLL " + json.dumps({"timestamp": time.time(), "type": "LOG", "step": step, "data": metrics}) + "\n")


def configure_loggers(trainer, exp_dir, log_dir, name, version, cfg: DictConfig):
    loggers = [JSONLLogger(str(log_dir), name, version)]
    if cfg.create_tensorboard_logger:
        try:
            kw = to_container(cfg.summary_writer_kwargs) if cfg.summary_writer_kwargs else {}
            loggers.append(TensorBoardLogger(str(log_dir), name, version, **kw))
        except Exception as e:  # tensorboard not importable
            logging.warning(f"TensorBoard logger disabled: {e}")
    optional = [("create_wandb_logger", "wandb_logger_kwargs", WandbLogger),
                ("create_mlflow_logger", "mlflow_logger_kwargs", MLFlowLogger),
                ("create_dllogger_logger", "dllogger_logger_kwargs", DLLogger)]
    for flag, kwname, cls in optional:
        if cfg.get(flag, False):
            kw = to_container(cfg.get(kwname)) if cfg.get(kwname) else {}
            if cls is WandbLogger and not kw:
                raise ValueError("If you are trying to create wandb logger, wandb_logger_kwargs must be provided")
            try:
                loggers.append(cls(str(log_dir), name, version, **kw))
            except ImportError as e:
                raise LoggerMisconfigurationError(f"{cls.__name__} requested but its package is missing: {e}")
    for flag, kwname, cls in (("create_clearml_logger", "clearml_logger_kwargs", ClearMLLogger),
                              ("create_neptune_logger", "neptune_logger_kwargs", NeptuneLogger)):
        if cfg.get(flag, False):
            kw = to_container(cfg.get(kwname)) if cfg.get(kwname) else {}
            try:
                loggers.append(cls(str(log_dir), name, version, **kw))
            except ImportError as e:
                raise LoggerMisconfigurationError(f"{cls.__name__} requested but its package is missing: {e}")
    trainer.loggers = loggers if is_global_rank_zero() else []


# ---------------------------------------------------------------------- directories / resume
def get_log_dir(trainer, exp_dir=None, name=None, version=None, explicit_log_dir=None, use_datetime_version=True,
                resume_if_exists=False):
    if explicit_log_dir:
        if exp_dir or version:
            logging.error(f"explicit_log_dir={explicit_log_dir} overrides exp_dir={exp_dir} and version={version}")
        return Path(explicit_log_dir), str(explicit_log_dir), "", ""
    exp_dir = exp_dir or str(Path.cwd() / "nemo_experiments")
    name = name or "default"
    version = version or os.environ.get("NEMO_EXPM_VERSION", None)
    if resume_if_exists:
        if version is None:
            version = ""  # resumed runs share one directory
    elif version is None:
        if use_datetime_version:
            version = time.strftime("%Y-%m-%d_%H-%M-%S")
        else:
            existing = [int(m.group(1)) for d in glob.glob(os.path.join(exp_dir, name, "version_*"))
                        if (m := re.search(r"version_(\d+)$", d))]
            version = f"version_{max(existing) + 1 if existing else 0}"
    os.environ["NEMO_EXPM_VERSION"] = version
    log_dir = Path(exp_dir) / name / version
    return log_dir, exp_dir, name, version


def check_resume(trainer, log_dir: str, resume_if_exists=False, resume_past_end=False, resume_ignore_no_checkpoint=False,
                 dirpath: Optional[str] = None, resume_from_checkpoint: Optional[str] = None):
    if not log_dir:
        raise ValueError(f"Resuming requires the log_dir {log_dir} to be passed to exp_manager")
    checkpoint = None
    if resume_from_checkpoint:
        checkpoint = resume_from_checkpoint
    if resume_if_exists:
        ck_dir = Path(dirpath) if dirpath else Path(log_dir) / "checkpoints"
        all_ckpts = list(ck_dir.rglob("*.ckpt")) if ck_dir.exists() else []
        ok = [c for c in all_ckpts if not NeMoModelCheckpoint.is_checkpoint_unfinished(str(c)) and not str(c).endswith("-EMA.ckpt")]
        end_ckpts = [c for c in ok if re.search(r"end(-v\d+)?\.ckpt$", c.name)]
        last_ckpts = [c for c in ok if re.search(r"last(-v\d+)?\.ckpt$", c.name)]
        if not ck_dir.exists() or (not end_ckpts and not last_ckpts):
            if resume_ignore_no_checkpoint:
                logging.warning(f"There were no checkpoints found in checkpoint_dir or no checkpoint folder at "
                                f"checkpoint_dir :{ck_dir}. Training from scratch.")
            elif checkpoint is None:
                raise NotFoundError(f"There were no checkpoints found in checkpoint_dir or no checkpoint folder at "
                                    f"checkpoint_dir :{ck_dir}. Cannot resume.")
        elif end_ckpts:
            if resume_past_end:
                if len(end_ckpts) > 1:
                    raise ValueError(f"Multiple checkpoints {end_ckpts} that matches *end.ckpt.")
                checkpoint = str(end_ckpts[0])
            else:
                raise ValueError(f"Found {end_ckpts[0]} indicating that the last training run has already completed.")
        else:
            if len(last_ckpts) > 1:
                raise ValueError(f"Multiple checkpoints {last_ckpts} that matches *last.ckpt.")
            checkpoint = str(last_ckpts[0])
            logging.info(f"Resuming training from checkpoint in {log_dir}, checkpoint: {checkpoint}")
    if checkpoint is not None:
        trainer.ckpt_path = str(checkpoint)
    if is_global_rank_zero() and Path(log_dir).exists():
        files = [c for c in Path(log_dir).iterdir() if c.is_file()]
        if files:
            runs = [int(m.group(1)) for c in Path(log_dir).iterdir() if c.is_dir() and (m := re.match(r"run_(\d+)$", c.name))]
            dst = Path(log_dir) / f"run_{max(runs) + 1 if runs else 0}"
            dst.mkdir()
            for f in files:
                shutil.move(str(f), str(dst))


def configure_checkpointing(trainer, log_dir, name, resume: bool, params: DictConfig, create_preemption_callback: bool):
    for cb in trainer.callbacks:
        if isinstance(cb, NeMoModelCheckpoint):
            raise CheckpointMisconfigurationError(
                "The trainer already contains a checkpoint callback; either set create_checkpoint_callback=False "
                "or remove it from the trainer callbacks.")
    p = to_container(params, resolve=True) if isinstance(params, DictConfig) else dict(params or {})
    if p.get("filepath"):
        if p.get("dirpath") is None:
            p["dirpath"] = str(Path(p["filepath"]).parent)
        if p.get("filename") is None:
            p["filename"] = Path(p["filepath"]).name
    p.pop("filepath", None)
    if p.get("dirpath") is None:
        p["dirpath"] = str(Path(log_dir) / "checkpoints")
    if p.get("filename") is None:
        p["filename"] = f"{name}--{{{p.get('monitor', 'val_loss')}:.4f}}-{{epoch}}"
    if p.get("prefix") is None:
        p["prefix"] = name
    if "val" in (p.get("monitor") or "") and trainer.max_epochs and trainer.max_epochs != -1 and \
            trainer.max_epochs < trainer.check_val_every_n_epoch:
        logging.error("The checkpoint callback was told to monitor a validation value but trainer.max_epochs is "
                      "less than trainer.check_val_every_n_epoch: no checkpoint will be saved.")
    cb = NeMoModelCheckpoint(**p)
    cb.last_model_path = trainer.ckpt_path or ""
    trainer.callbacks.append(cb)
    trainer.checkpoint_callback = cb
    if create_preemption_callback:
        trainer.callbacks.append(PreemptionCallback(cb))
    return cb


def exp_manager(trainer, cfg: Optional[Union[DictConfig, Dict]] = None) -> Optional[Path]:
    """Set up logging / checkpointing for ``trainer`` from an ``exp_manager`` config block."""
    if cfg is None:
        logging.error("exp_manager did not receive a cfg argument. It will be disabled.")
        return None
    if trainer.fast_dev_run:
        logging.info("Trainer was called with fast_dev_run. exp_manager will return without any functionality.")
        return None
    schema = OmegaConf.structured(ExpManagerConfig)
    if isinstance(cfg, dict):
        cfg = OmegaConf.create(cfg)
    else:
        # interpolations such as ``name: ${name}`` point into the tree this block came from: resolve them there, before the
        # block becomes a tree of its own
        from ..core.config import to_container

        cfg = OmegaConf.create(to_container(cfg, resolve=True))
    unknown = [k for k in cfg.keys() if k not in schema]
    if unknown:
        raise ValueError(f"Unknown exp_manager config keys: {unknown}")
    cfg = OmegaConf.merge(schema, cfg)
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    global_rank = trainer.global_rank
    log_dir, exp_dir, name, version = get_log_dir(trainer, cfg.exp_dir, cfg.name, cfg.version, cfg.explicit_log_dir,
                                                  cfg.use_datetime_version, cfg.resume_if_exists)
    ck_dir = None
    if cfg.checkpoint_callback_params is not None:
        ck_dir = cfg.checkpoint_callback_params.get("dirpath", None)
    if cfg.resume_if_exists or cfg.resume_from_checkpoint:
        check_resume(trainer, str(log_dir), cfg.resume_if_exists, cfg.resume_past_end, cfg.resume_ignore_no_checkpoint,
                     ck_dir, cfg.resume_from_checkpoint)
    app = AppState()
    app.log_dir, app.exp_dir, app.name, app.version = str(log_dir), exp_dir, name, version
    app.create_checkpoint_callback = cfg.create_checkpoint_callback
    os.makedirs(log_dir, exist_ok=True)
    trainer.default_root_dir = str(log_dir)
    logging.info(f"Experiments will be logged at {log_dir}")
    # per-rank log files
    if cfg.log_global_rank_0_only and cfg.log_local_rank_0_only:
        raise ValueError("Cannot set both log_local_rank_0_only and log_global_rank_0_only to True.")
    nemo_testing = os.environ.get("NEMO_TESTING", "0") == "1"
    log_file = log_dir / f"nemo_log_globalrank-{global_rank}_localrank-{local_rank}.txt"
    if cfg.log_local_rank_0_only and not nemo_testing:
        if local_rank == 0:
            logging.add_file_handler(str(log_file))
    elif cfg.log_global_rank_0_only and not nemo_testing:
        if global_rank == 0:
            logging.add_file_handler(str(log_file))
    else:
        logging.add_file_handler(str(log_file))
    configure_loggers(trainer, exp_dir, log_dir, name, version, cfg)
    if cfg.log_step_timing:
        kw = to_container(cfg.step_timing_kwargs) if cfg.step_timing_kwargs else {}
        trainer.callbacks.insert(0, TimingCallback(timer_kwargs={k: v for k, v in kw.items() if k != "sync_cuda"},
                                                   sync_cuda=kw.get("sync_cuda", False)))
    if cfg.ema is not None and cfg.ema.enable:
        trainer.callbacks.append(EMA(decay=cfg.ema.decay, validate_original_weights=cfg.ema.validate_original_weights,
                                     cpu_offload=cfg.ema.cpu_offload, every_n_steps=cfg.ema.every_n_steps))
    if cfg.create_early_stopping_callback:
        trainer.callbacks.append(EarlyStopping(**to_container(cfg.early_stopping_callback_params)))
    if cfg.create_checkpoint_callback:
        configure_checkpointing(trainer, log_dir, name or "default", cfg.resume_if_exists, cfg.checkpoint_callback_params,
                                cfg.create_preemption_callback)
    if cfg.max_time_per_run is not None:
        trainer.callbacks.append(StatelessTimer(cfg.max_time_per_run))
    if cfg.create_straggler_detection_callback or cfg.create_fault_tolerance_callback:
        from ..parallel.resiliency import FaultToleranceCallback, StragglerDetectionCallback

        if cfg.create_straggler_detection_callback:
            trainer.callbacks.append(StragglerDetectionCallback())
        if cfg.create_fault_tolerance_callback:
            trainer.callbacks.append(FaultToleranceCallback())
    if is_global_rank_zero():
        if cfg.files_to_copy:
            for f in cfg.files_to_copy:
                shutil.copy(f, log_dir)
        with open(log_dir / "cmd-args.log", "w", encoding="utf-8") as f:
            f.write(" ".join(sys.argv))
        try:
            sha = subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5)
            if sha.returncode == 0:
                diff = subprocess.run(["git", "diff", "--stat"], capture_output=True, text=True, timeout=5).stdout
                with open(log_dir / "git-info.log", "w", encoding="utf-8") as f:
                    f.write(f"commit hash: {sha.stdout.strip()}\n{diff}")
        except Exception:
            pass
        logging.add_err_file_handler(str(log_dir / "nemo_error_log.txt"))
    return log_dir

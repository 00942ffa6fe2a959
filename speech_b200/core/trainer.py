"""Training loop with Lightning-compatible hook names.

The reference drives every model through ``lightning.pytorch.Trainer``
(``examples/asr/asr_transducer/speech_to_text_rnnt_bpe.py:72-85``).  This trainer keeps the
same constructor keys (``devices, max_steps, max_epochs, precision, accumulate_grad_batches,
gradient_clip_val, val_check_interval, log_every_n_steps, limit_*_batches, strategy, callbacks``)
and callback protocol, but owns the step itself so that gradient buckets, the flat optimizer
arena, CUDA streams and whole-step CUDA graphs belong to the framework:

* one process per GPU; rank / world size come from the ``torchrun`` environment,
* gradients are exchanged by a :class:`speech_b200.parallel.ddp.GradSync` strategy (gloo on CPU,
  NCCL or the peer-memory kernel on GPUs) instead of a wrapped ``DistributedDataParallel``,
* precision ``bf16`` / ``bf16-mixed`` keeps fp32 master weights and runs activations in bf16;
  batch entries whose key contains ``audio`` stay fp32 (reference: ``nemo/utils/trainer_utils.py:115``).
"""
from __future__ import annotations

import contextlib
import math
import os
import signal
import time
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Union

import torch
import torch.distributed as dist

from ..utils.logging import AppState, logging
from .config import DictConfig, OmegaConf, to_container


class Callback:
    """Base callback; every hook gets ``(trainer, model, ...)``."""

    def setup(self, trainer, model, stage: str): ...
    def on_fit_start(self, trainer, model): ...
    def on_fit_end(self, trainer, model): ...
    def on_train_start(self, trainer, model): ...
    def on_train_end(self, trainer, model): ...
    def on_train_epoch_start(self, trainer, model): ...
    def on_train_epoch_end(self, trainer, model): ...
    def on_train_batch_start(self, trainer, model, batch, batch_idx): ...
    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx): ...
    def on_before_backward(self, trainer, model, loss): ...
    def on_after_backward(self, trainer, model): ...
    def on_before_optimizer_step(self, trainer, model, optimizer): ...
    def on_before_zero_grad(self, trainer, model, optimizer): ...
    def on_validation_start(self, trainer, model): ...
    def on_validation_end(self, trainer, model): ...
    def on_validation_batch_end(self, trainer, model, outputs, batch, batch_idx, dataloader_idx=0): ...
    def on_test_start(self, trainer, model): ...
    def on_test_end(self, trainer, model): ...
    def on_save_checkpoint(self, trainer, model, checkpoint: Dict[str, Any]): ...
    def on_load_checkpoint(self, trainer, model, checkpoint: Dict[str, Any]): ...
    def on_exception(self, trainer, model, exception): ...
    def state_dict(self) -> Dict[str, Any]:
        return {}

    def load_state_dict(self, state: Dict[str, Any]): ...


def move_to_device(batch: Any, device: torch.device, dtype: Optional[torch.dtype] = None, key: str = "") -> Any:
    """Recursive H2D copy; float tensors are cast to ``dtype`` unless their key mentions ``audio``."""
    if torch.is_tensor(batch):
        if dtype is not None and batch.is_floating_point() and "audio" not in key:
            return batch.to(device=device, dtype=dtype, non_blocking=True)
        return batch.to(device, non_blocking=True)
    if isinstance(batch, dict):
        return {k: move_to_device(v, device, dtype, str(k)) for k, v in batch.items()}
    if isinstance(batch, tuple) and hasattr(batch, "_fields"):
        return type(batch)(*(move_to_device(v, device, dtype, f) for v, f in zip(batch, batch._fields)))
    if isinstance(batch, (list, tuple)):
        return type(batch)(move_to_device(v, device, dtype, key) for v in batch)
    if hasattr(batch, "to") and not isinstance(batch, str):
        try:
            return batch.to(device)
        except Exception:
            return batch
    return batch


class Trainer:
    def __init__(self, devices: Union[int, str, List[int]] = 1, accelerator: str = "auto", num_nodes: int = 1,
                 max_epochs: Optional[int] = None, max_steps: int = -1, precision: Union[str, int] = 32,
                 accumulate_grad_batches: int = 1, gradient_clip_val: Optional[float] = None,
                 val_check_interval: Union[int, float] = 1.0, check_val_every_n_epoch: Optional[int] = 1,
                 log_every_n_steps: int = 50, limit_train_batches: Union[int, float] = 1.0,
                 limit_val_batches: Union[int, float] = 1.0, limit_test_batches: Union[int, float] = 1.0,
                 num_sanity_val_steps: int = 0, enable_checkpointing: bool = False, logger: Any = False,
                 callbacks: Optional[List[Callback]] = None, strategy: Any = "auto", fast_dev_run: Union[bool, int] = False,
                 enable_progress_bar: bool = False, sync_batchnorm: bool = False, benchmark: bool = False,
                 use_distributed_sampler: bool = False, default_root_dir: Optional[str] = None,
                 max_time: Optional[Any] = None, detect_anomaly: bool = False, **_ignored):
        self.callbacks: List[Callback] = list(callbacks or [])
        self.max_epochs = max_epochs if max_epochs is not None else (-1 if max_steps and max_steps > 0 else 1000)
        self.max_steps = max_steps if max_steps is not None else -1
        self.precision = str(precision)
        self.accumulate_grad_batches = int(accumulate_grad_batches or 1)
        self.gradient_clip_val = float(gradient_clip_val or 0.0)
        self.val_check_interval = val_check_interval
        self.check_val_every_n_epoch = check_val_every_n_epoch or 1
        self.log_every_n_steps = log_every_n_steps
        self.limit_train_batches, self.limit_val_batches, self.limit_test_batches = (
            limit_train_batches, limit_val_batches, limit_test_batches)
        self.num_sanity_val_steps = num_sanity_val_steps
        self.sync_batchnorm = sync_batchnorm
        self.default_root_dir = default_root_dir or os.getcwd()
        self.fast_dev_run = fast_dev_run
        if fast_dev_run:
            n = 1 if fast_dev_run is True else int(fast_dev_run)
            self.max_steps, self.limit_val_batches, self.limit_test_batches = n, n, n
            self.max_epochs = 1
        self.loggers: List[Any] = [] if not logger else (list(logger) if isinstance(logger, (list, tuple)) else [logger])
        self.strategy_spec = strategy
        self.accelerator = accelerator
        self.devices = devices
        self.num_nodes = num_nodes
        # --- distributed identity (torchrun env)
        self.global_rank = int(os.environ.get("RANK", 0))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        if accelerator in ("auto", "gpu", "cuda") and torch.cuda.is_available() and accelerator != "cpu":
            self.device = torch.device("cuda", self.local_rank % max(1, torch.cuda.device_count()))
        else:
            self.device = torch.device("cpu")
        self.global_step = 0
        self.current_epoch = 0
        self.batch_idx = 0
        self.should_stop = False
        self.model = None
        self.optimizers: List[torch.optim.Optimizer] = []
        self.lr_scheduler_configs: List[Dict[str, Any]] = []
        self.callback_metrics: Dict[str, Any] = {}
        self.logged_metrics: Dict[str, Any] = {}
        self._step_logs: Dict[str, Any] = {}
        self.ckpt_path: Optional[str] = None
        self.grad_sync = None
        self.state_fn = "idle"
        self.training = False
        self.validating = False
        self.testing = False
        self.sanity_checking = False
        self.interrupted = False
        self._resume_skip_batches = 0
        self._batches_in_epoch = 0           # batches of the current epoch already trained on (saved in checkpoints)
        self.checkpoint_callback = next((c for c in self.callbacks if hasattr(c, "best_model_path")), None)

    # ------------------------------------------------------------------ properties
    @property
    def is_global_zero(self) -> bool:
        return self.global_rank == 0

    @property
    def logger(self):
        return self.loggers[0] if self.loggers else None

    @property
    def log_dir(self) -> Optional[str]:
        lg = self.logger
        return getattr(lg, "log_dir", None) if lg is not None else self.default_root_dir

    @property
    def lightning_module(self):
        return self.model

    @property
    def compute_dtype(self) -> Optional[torch.dtype]:
        p = self.precision
        if p in ("bf16", "bf16-mixed", "bf16-true", "bf16-flash"):
            return torch.bfloat16
        if p in ("16", "16-mixed", "fp16"):
            return torch.float16
        return None

    @property
    def num_training_batches(self) -> float:
        dl = self.model.train_dataloader() if self.model is not None else None
        try:
            n = len(dl)
        except Exception:
            return float("inf")
        lim = self.limit_train_batches
        return min(n, lim) if isinstance(lim, int) else int(n * lim)

    # ------------------------------------------------------------------ logging plumbing
    def _collect_log(self, name: str, value: Any, sync_dist: bool = False):
        if sync_dist and torch.is_tensor(value) and self.world_size > 1 and dist.is_initialized():
            value = value.clone().float()
            dist.all_reduce(value)
            value /= self.world_size
        self._step_logs[name] = value
        self.callback_metrics[name] = value

    def _flush_logs(self, step: int):
        if not self._step_logs:
            return
        flat = {}
        for k, v in self._step_logs.items():
            if torch.is_tensor(v):
                if v.numel() != 1:
                    continue
                v = float(v)
            if isinstance(v, (int, float)):
                flat[k] = v
        self.logged_metrics.update(flat)
        if self.is_global_zero:
            for lg in self.loggers:
                lg.log_metrics(flat, step)
        self._step_logs = {}

    def _call(self, hook: str, *args, **kw):
        for cb in self.callbacks:
            fn = getattr(cb, hook, None)
            if fn is not None:
                fn(self, self.model, *args, **kw)

    # ------------------------------------------------------------------ setup
    def _init_distributed(self):
        if self.world_size > 1 and not dist.is_initialized():
            backend = "nccl" if self.device.type == "cuda" else "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            dist.init_process_group(backend, rank=self.global_rank, world_size=self.world_size)
        app = AppState()
        app.global_rank, app.local_rank, app.world_size = self.global_rank, self.local_rank, self.world_size

    def _attach(self, model, stage: str):
        self.model = model
        model.set_trainer(self)
        self._init_distributed()
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        model.to(self.device)
        if hasattr(self.strategy_spec, "setup_model") and getattr(self.strategy_spec, "_model_set_up", None) is not model:
            self.strategy_spec.setup_model(model)            # device mesh: the model shards itself before optimizers exist
            self.strategy_spec._model_set_up = model
        for cb in self.callbacks:
            if hasattr(cb, "setup"):
                cb.setup(self, model, stage)

    def _configure_optimizers(self):
        out = self.model.configure_optimizers()
        opts, scheds = [], []
        if out is None:
            pass
        elif isinstance(out, torch.optim.Optimizer):
            opts = [out]
        elif isinstance(out, (tuple, list)) and len(out) == 2 and isinstance(out[0], (list, tuple)):
            opts, scheds = list(out[0]), list(out[1])
        elif isinstance(out, dict):
            opts = [out["optimizer"]]
            if out.get("lr_scheduler") is not None:
                scheds = [out["lr_scheduler"]]
        else:
            opts = list(out)
        self.optimizers = opts
        self.lr_scheduler_configs = [s if isinstance(s, dict) else {"scheduler": s, "interval": "step", "frequency": 1}
                                     for s in scheds]

    def _setup_grad_sync(self):
        from ..parallel.ddp import build_grad_sync

        if not getattr(self.model, "automatic_optimization", True):
            self.grad_sync = None                       # manual_step averages the gradients of the optimizer it updates
            return

        if hasattr(self.strategy_spec, "build_grad_sync"):
            self.grad_sync = self.strategy_spec.build_grad_sync(self.model, self.optimizers, self.device, sync_batchnorm=self.sync_batchnorm)
            return
        self.grad_sync = build_grad_sync(self.model, self.optimizers, self.strategy_spec, self.world_size, self.device,
                                         sync_batchnorm=self.sync_batchnorm)

    # ------------------------------------------------------------------ contexts
    def precision_context(self):
        from .. import ops

        dt = self.compute_dtype
        if dt is None:
            return contextlib.nullcontext()
        stack = contextlib.ExitStack()
        stack.enter_context(ops.compute_dtype(dt))
        if self.device.type == "cuda":
            stack.enter_context(torch.autocast("cuda", dtype=dt))
        return stack

    # ------------------------------------------------------------------ fit
    def fit(self, model, train_dataloaders=None, val_dataloaders=None, ckpt_path: Optional[str] = None):
        self._attach(model, "fit")
        if train_dataloaders is not None:
            model._train_dl = train_dataloaders
        if val_dataloaders is not None:
            model._validation_dl = val_dataloaders
        self._configure_optimizers()
        self._setup_grad_sync()
        ckpt_path = ckpt_path or self.ckpt_path
        if ckpt_path:
            self._restore_checkpoint(ckpt_path)
        self.training = True
        self.state_fn = "fit"
        try:
            model.on_fit_start()
            self._call("on_fit_start")
            if self.num_sanity_val_steps and model.val_dataloader() is not None and not ckpt_path:
                self.sanity_checking = True
                self._run_eval("val", limit=self.num_sanity_val_steps)
                self.sanity_checking = False
            model.on_train_start()
            self._call("on_train_start")
            self._fit_loop()
            model.on_train_end()
            self._call("on_train_end")
            self._call("on_fit_end")
        except BaseException as e:  # noqa: BLE001 - callbacks get a chance to save state
            self._call("on_exception", e)
            raise
        finally:
            self.training = False
            self.state_fn = "idle"
        return self

    def _should_stop_steps(self) -> bool:
        return self.max_steps is not None and self.max_steps > 0 and self.global_step >= self.max_steps

    def _fit_loop(self):
        model = self.model
        while not self.should_stop:
            if self.max_epochs is not None and self.max_epochs >= 0 and self.current_epoch >= self.max_epochs:
                break
            if self._should_stop_steps():
                break
            dl = model.train_dataloader()
            if dl is None:
                raise RuntimeError("fit() needs a training dataloader (cfg.train_ds or train_dataloaders=...)")
            if hasattr(dl, "sampler") and hasattr(dl.sampler, "set_epoch"):
                dl.sampler.set_epoch(self.current_epoch)
            model.train()
            model.on_train_epoch_start()
            self._call("on_train_epoch_start")
            n_batches = self.num_training_batches
            val_every = self.val_check_interval
            if isinstance(val_every, float):
                val_every = max(1, int(n_batches * val_every)) if n_batches != float("inf") else None
            epoch_complete = True
            for batch_idx, batch in enumerate(dl):
                if batch_idx >= n_batches:
                    break
                if self._resume_skip_batches > 0:
                    self._resume_skip_batches -= 1      # resumed inside an epoch: these batches were trained on before the checkpoint
                    continue
                self.batch_idx = batch_idx
                self._train_batch(batch, batch_idx)
                self._batches_in_epoch = batch_idx + 1
                stepped = (batch_idx + 1) % self.accumulate_grad_batches == 0
                if stepped and val_every and isinstance(self.val_check_interval, int) and \
                        self.global_step % val_every == 0 and model.val_dataloader() is not None:
                    self._validate_in_fit()
                elif val_every and isinstance(self.val_check_interval, float) and (batch_idx + 1) % val_every == 0 \
                        and (self.current_epoch + 1) % self.check_val_every_n_epoch == 0 \
                        and model.val_dataloader() is not None:
                    self._validate_in_fit()
                if self.should_stop or self._should_stop_steps():
                    epoch_complete = n_batches != float("inf") and batch_idx + 1 >= n_batches
                    break
            model.on_train_epoch_end()
            self._call("on_train_epoch_end")
            if epoch_complete:
                # a run that stops inside an epoch (max_steps, early stop) stays in that epoch: a checkpoint taken now resumes
                # with the remaining batches of the same epoch and the same shuffling order
                self.current_epoch += 1
                self._batches_in_epoch = 0

    def _validate_in_fit(self):
        self._run_eval("val")
        self.model.train()

    def _train_batch(self, batch, batch_idx: int):
        model = self.model
        accum = self.accumulate_grad_batches
        first_micro = batch_idx % accum == 0
        last_micro = (batch_idx + 1) % accum == 0
        batch = move_to_device(batch, self.device, None)
        model.on_train_batch_start(batch, batch_idx)
        self._call("on_train_batch_start", batch, batch_idx)
        if not getattr(model, "automatic_optimization", True):
            # the model drives its optimizers itself (several optimizers updated in turn, as in adversarial training): its
            # training_step calls ``trainer.manual_step(loss, optimizer)`` for every update
            self._in_manual_step = True
            try:
                with self.precision_context():
                    out = model.training_step(batch, batch_idx)
            finally:
                self._in_manual_step = False
            for sc in self.lr_scheduler_configs:
                if sc.get("interval", "step") == "step" and (self.global_step + 1) % sc.get("frequency", 1) == 0 and not sc.get("reduce_on_plateau", False):
                    sc["scheduler"].step()
            self.global_step += 1
            if self.optimizers:
                self._collect_log("lr", self.optimizers[0].param_groups[0]["lr"])
            model.on_train_batch_end(out, batch, batch_idx)
            self._call("on_train_batch_end", out, batch, batch_idx)
            if self.global_step % max(1, self.log_every_n_steps) == 0 or self.global_step == 1:
                self._flush_logs(self.global_step)
            return
        if first_micro:
            for opt in self.optimizers:
                self._call("on_before_zero_grad", opt)
                opt.zero_grad(set_to_none=not hasattr(opt, "arena"))
            if self.grad_sync is not None:
                self.grad_sync.begin_step()
        with self.precision_context():
            out = model.training_step(batch, batch_idx)
        loss = out["loss"] if isinstance(out, dict) else out
        if loss is None:
            return
        self._call("on_before_backward", loss)
        sync_now = last_micro
        ctx = self.grad_sync.no_sync() if (self.grad_sync is not None and not sync_now) else contextlib.nullcontext()
        with ctx:
            (loss / accum if accum > 1 else loss).backward()
        if last_micro and self.grad_sync is not None:
            # the bucket reductions launched during backward are joined BEFORE any hook looks at (or zeroes) the gradients
            self.grad_sync.finish_step()
        model.on_after_backward()
        self._call("on_after_backward")
        if last_micro:
            self._check_kernel_status()
            for opt in self.optimizers:
                self._clip_gradients(opt)
                self._call("on_before_optimizer_step", opt)
                opt.step()
            for sc in self.lr_scheduler_configs:
                if sc.get("interval", "step") == "step" and (self.global_step + 1) % sc.get("frequency", 1) == 0:
                    if not sc.get("reduce_on_plateau", False):
                        sc["scheduler"].step()
            self.global_step += 1
            if self.optimizers:
                self._collect_log("lr", self.optimizers[0].param_groups[0]["lr"])
        model.on_train_batch_end(out, batch, batch_idx)
        self._call("on_train_batch_end", out, batch, batch_idx)
        if last_micro and (self.global_step % max(1, self.log_every_n_steps) == 0 or self.global_step == 1):
            self._flush_logs(self.global_step)

    @property
    def in_manual_step(self) -> bool:
        """True while a model with ``automatic_optimization = False`` runs its ``training_step`` under ``fit``."""
        return bool(getattr(self, "_in_manual_step", False))

    def manual_step(self, loss: torch.Tensor, optimizer, retain_graph: bool = False) -> None:
        """One update of ``optimizer`` from ``loss`` for models that optimise manually: clears that optimizer's gradients, runs
        backward, averages the gradients over data-parallel ranks, clips and steps."""
        optimizer.zero_grad(set_to_none=True)
        self._call("on_before_backward", loss)
        loss.backward(retain_graph=retain_graph)
        if self.world_size > 1 and torch.distributed.is_available() and torch.distributed.is_initialized():
            for g in optimizer.param_groups:
                for p in g["params"]:
                    if p.grad is not None:
                        torch.distributed.all_reduce(p.grad)
                        p.grad.div_(self.world_size)
        self._clip_gradients(optimizer)
        self._call("on_before_optimizer_step", optimizer)
        optimizer.step()

    def _check_kernel_status(self):
        """Fail the run when a kernel of an earlier step gave up a bounded wait (a peer rank that never arrived).

        The kernels themselves keep such a step harmless: the update kernel and the gradient unpack return without writing once
        the device status word is set.  Here the word of the PREVIOUS step is read (an asynchronous copy into pinned memory
        made at that step, so this never waits for the GPU's current work) and turned into an exception on every rank that
        sees it; ranks that did not time out themselves run into the missing rank at their next bucket and fail the same way."""
        if self.device.type != "cuda" or self.grad_sync is None:
            return
        from ..ops import native

        st = getattr(self, "_status_probe", None)
        if st is None:
            st = self._status_probe = native.StatusProbe(self.device)
        code = st.poll()
        if code:
            raise RuntimeError(f"a device kernel gave up a bounded wait in an earlier step: {native.status_message(code)}; "
                               "the optimizer update of that step was skipped on this rank")
        st.record()

    def _clip_gradients(self, opt):
        if self.gradient_clip_val <= 0 or getattr(opt, "max_grad_norm", 0.0) > 0:
            return  # fused optimizers clip inside their update kernel
        custom = getattr(self.model, "configure_gradient_clipping", None)
        if custom is not None:
            custom(opt, self.gradient_clip_val)       # models on a device mesh compute the norm over the right groups
            return
        params = [p for g in opt.param_groups for p in g["params"] if p.grad is not None]
        if params:
            torch.nn.utils.clip_grad_norm_(params, self.gradient_clip_val)

    # ------------------------------------------------------------------ evaluation
    def _run_eval(self, which: str, limit: Optional[int] = None, dataloaders=None):
        model = self.model
        dls = dataloaders if dataloaders is not None else (model.val_dataloader() if which == "val" else model.test_dataloader())
        if dls is None:
            return {}
        multi = isinstance(dls, (list, tuple))
        dls = list(dls) if multi else [dls]
        was_training = model.training
        model.eval()
        self.validating, self.testing = which == "val", which == "test"
        (model.on_validation_epoch_start if which == "val" else model.on_test_epoch_start)()
        self._call("on_validation_start" if which == "val" else "on_test_start")
        outputs_attr = "validation_step_outputs" if which == "val" else "test_step_outputs"
        setattr(model, outputs_attr, [[] for _ in dls] if multi else [])
        lim_cfg = self.limit_val_batches if which == "val" else self.limit_test_batches
        with torch.no_grad():
            for di, dl in enumerate(dls):
                try:
                    n = len(dl)
                    n = min(n, lim_cfg) if isinstance(lim_cfg, int) else int(math.ceil(n * lim_cfg))
                except Exception:
                    n = lim_cfg if isinstance(lim_cfg, int) else float("inf")
                if limit is not None:
                    n = min(n, limit)
                for bi, batch in enumerate(dl):
                    if bi >= n:
                        break
                    batch = move_to_device(batch, self.device, None)
                    with self.precision_context():
                        step = model.validation_step if which == "val" else model.test_step
                        out = step(batch, bi, di) if multi else step(batch, bi)
                    store = getattr(model, outputs_attr)
                    tgt = store[di] if multi else store
                    if out is not None and not tgt_contains(tgt, out):
                        tgt.append(out)
                    if which == "val":
                        self._call("on_validation_batch_end", out, batch, bi, di)
        res = model.on_validation_epoch_end() if which == "val" else model.on_test_epoch_end()
        if not self.sanity_checking:
            self._flush_logs(self.global_step)
            self._call("on_validation_end" if which == "val" else "on_test_end")
        self.validating = self.testing = False
        model.train(was_training)
        return res or {}

    def validate(self, model=None, dataloaders=None, ckpt_path=None):
        if model is not None:
            self._attach(model, "validate")
        if ckpt_path:
            self._restore_checkpoint(ckpt_path, weights_only=True)
        res = self._run_eval("val", dataloaders=dataloaders)
        return [_to_float_dict(res)]

    def test(self, model=None, dataloaders=None, ckpt_path=None):
        if model is not None:
            self._attach(model, "test")
        if ckpt_path:
            self._restore_checkpoint(ckpt_path, weights_only=True)
        res = self._run_eval("test", dataloaders=dataloaders)
        return [_to_float_dict(res)]

    def predict(self, model=None, dataloaders=None, return_predictions: bool = True):
        if model is not None:
            self._attach(model, "predict")
        model = self.model
        dls = dataloaders if dataloaders is not None else model.test_dataloader()
        dls = list(dls) if isinstance(dls, (list, tuple)) else [dls]
        model.eval()
        preds = []
        with torch.no_grad():
            for di, dl in enumerate(dls):
                for bi, batch in enumerate(dl):
                    batch = move_to_device(batch, self.device, None)
                    with self.precision_context():
                        preds.append(model.predict_step(batch, bi, di) if len(dls) > 1 else model.predict_step(batch, bi))
        return preds

    # ------------------------------------------------------------------ checkpoints
    def dump_checkpoint(self, weights_only: bool = False) -> Dict[str, Any]:
        model = self.model
        ckpt: Dict[str, Any] = {
            "epoch": self.current_epoch,
            "global_step": self.global_step,
            "batch_idx": self.batch_idx,
            "batches_in_epoch": self._batches_in_epoch,
            "state_dict": self._model_state_dict(),
            "hyper_parameters": {"cfg": to_container(model.cfg, resolve=True)},
            "pytorch-lightning_version": "speech_b200",
        }
        if not weights_only:
            ckpt["optimizer_states"] = [_cpu_tree(o.state_dict()) for o in self.optimizers]
            ckpt["lr_schedulers"] = [sc["scheduler"].state_dict() for sc in self.lr_scheduler_configs]
            ckpt["callbacks"] = {type(cb).__name__: cb.state_dict() for cb in self.callbacks if hasattr(cb, "state_dict")}
        self._call("on_save_checkpoint", ckpt)
        return ckpt

    def _model_state_dict(self) -> Dict[str, Any]:
        """Parameters of a fully-sharded model live as slices inside the optimizer: it assembles the full values (a collective,
        which is why every rank builds the checkpoint dictionary although only rank 0 writes it)."""
        for o in getattr(self, "optimizers", []) or []:
            if hasattr(o, "full_model_state_dict"):
                return o.full_model_state_dict()
        sd = {k: v.detach() for k, v in self.model.state_dict().items()}
        mp = {n: p for n, p in self.model.named_parameters() if getattr(p, "_mp_gather", None) is not None}
        for n, p in mp.items():                      # tensor- / expert-parallel slices are written as whole tensors
            if n in sd:
                sd[n] = p._mp_gather(sd[n])
        return {k: v.cpu() for k, v in sd.items()}

    def save_checkpoint(self, filepath: str, weights_only: bool = False, checkpoint_format: Optional[str] = None):
        """``checkpoint_format="dcp"`` (or a path ending in ``.dcp``) writes a distributed-checkpoint directory: the model tensors in
        PyTorch's DCP layout, written cooperatively by all ranks, plus ``trainer_state.pt`` (optimizers, schedulers, counters) from
        rank 0.  The default is one ``.ckpt`` file from rank 0."""
        ckpt = self.dump_checkpoint(weights_only)
        if (checkpoint_format or getattr(self, "checkpoint_format", None)) == "dcp" or str(filepath).endswith(".dcp"):
            from ..utils.dcp_io import DCPCheckpointIO

            tensors = {k: v for k, v in ckpt["state_dict"].items() if torch.is_tensor(v)}
            DCPCheckpointIO().save_checkpoint(tensors, filepath, extra={"global_step": self.global_step, "epoch": self.current_epoch})
            if self.is_global_zero:
                rest = {k: v for k, v in ckpt.items() if k != "state_dict"}
                rest["state_dict_extra"] = {k: v for k, v in ckpt["state_dict"].items() if not torch.is_tensor(v)}
                torch.save(rest, os.path.join(filepath, "trainer_state.pt.tmp"))
                os.replace(os.path.join(filepath, "trainer_state.pt.tmp"), os.path.join(filepath, "trainer_state.pt"))
            if self.world_size > 1 and dist.is_initialized():
                dist.barrier()
            return
        if self.is_global_zero:
            os.makedirs(os.path.dirname(os.path.abspath(filepath)), exist_ok=True)
            tmp = filepath + ".tmp"
            torch.save(ckpt, tmp)
            os.replace(tmp, filepath)
        if self.world_size > 1 and dist.is_initialized():
            dist.barrier()

    def _restore_checkpoint(self, path: str, weights_only: bool = False):
        if os.path.isdir(path):
            from ..utils.dcp_io import DCPCheckpointIO

            state, _ = DCPCheckpointIO().load_checkpoint(path)
            ckpt = torch.load(os.path.join(path, "trainer_state.pt"), map_location="cpu", weights_only=False)
            ckpt["state_dict"] = dict(state, **ckpt.pop("state_dict_extra", {}))
        else:
            ckpt = torch.load(path, map_location="cpu", weights_only=False)
        sharded = [o for o in (getattr(self, "optimizers", []) or []) if hasattr(o, "load_full_params")]
        if sharded:
            # sharded parameters are taken slice-wise by their optimizer; the module only loads what the optimizer does not own
            owned = set(sharded[0]._names().values())
            rest = {k: v for k, v in ckpt["state_dict"].items() if k not in owned}
            missing, unexpected = self.model.load_state_dict(rest, strict=False)
            bad = [k for k in missing if k not in owned] + list(unexpected)
            if bad:
                raise KeyError(f"checkpoint does not match the model: {bad[:8]}")
            sharded[0].load_full_params(ckpt["state_dict"])
        else:
            sd = ckpt["state_dict"]
            mp = {n: p for n, p in self.model.named_parameters() if getattr(p, "_mp_slice", None) is not None}
            if mp:
                from ..parallel.tp import mp_local

                sd = dict(sd)
                for n, p in mp.items():
                    if n in sd:
                        sd[n] = mp_local(p, sd[n], p.shape)
            self.model.load_state_dict(sd, strict=True)
        if weights_only:
            return
        self.global_step = int(ckpt.get("global_step", 0))
        self.current_epoch = int(ckpt.get("epoch", 0))
        self._resume_skip_batches = self._batches_in_epoch = int(ckpt.get("batches_in_epoch", 0))
        for o, s in zip(self.optimizers, ckpt.get("optimizer_states", [])):
            o.load_state_dict(s)
        for o in self.optimizers:
            if hasattr(o, "arena"):
                o.arena.refresh_lowp()
        for sc, s in zip(self.lr_scheduler_configs, ckpt.get("lr_schedulers", [])):
            sc["scheduler"].load_state_dict(s)
        cb_states = ckpt.get("callbacks", {})
        for cb in self.callbacks:
            if type(cb).__name__ in cb_states and hasattr(cb, "load_state_dict"):
                cb.load_state_dict(cb_states[type(cb).__name__])
        self._call("on_load_checkpoint", ckpt)
        logging.info(f"Restored trainer state from {path} at global_step={self.global_step}")


def tgt_contains(store: list, out: Any) -> bool:
    """Models may append to ``validation_step_outputs`` themselves; avoid storing the same object twice."""
    return any(o is out for o in store[-1:])


def _to_float_dict(d: Dict[str, Any]) -> Dict[str, float]:
    out = {}
    for k, v in (d or {}).items():
        if torch.is_tensor(v) and v.numel() == 1:
            out[k] = float(v)
        elif isinstance(v, (int, float)):
            out[k] = float(v)
    return out


def _cpu_tree(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _cpu_tree(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_cpu_tree(v) for v in obj)
    return obj

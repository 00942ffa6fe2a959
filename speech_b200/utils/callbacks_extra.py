"""Further trainer callbacks and IO helpers: whole-iteration CUDA-graph capture, a process-wide callback fan-out, profiler range
control, object-store checkpoint IO and the Hugging Face directory / hub mixin.

Reference: ``utils/callbacks/cuda_graph.py:88,251`` (``StaticBufferLoader``, ``CUDAGraphCallback``: static input buffers, warm-up
iterations on a side stream, the forward + backward of a training iteration captured once and replayed),
``lightning/callback_group.py`` (``CallbackGroup`` singleton: ``on_model_init_start`` … ``on_app_end`` fanned out to registered
callbacks, ``hook_class_init_with_callbacks``), ``speechlm2/parts/nsight.py:18`` (``NsightProfiling``: profiler start / stop at
given steps), ``utils/callbacks/s3_checkpoint_io.py`` / ``msc_utils.py`` (checkpoint IO on object stores),
``core/classes/mixins/hf_io_mixin.py`` (``HuggingFaceFileIO``: ``save_pretrained`` / ``from_pretrained`` / ``push_to_hub``).
"""
from __future__ import annotations

import json
import os
import shutil
import threading
from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..core.trainer import Callback
from .logging import logging


# ---------------------------------------------------------------------------------------------- CUDA graphs for training
def _tensors(batch) -> List[torch.Tensor]:
    if isinstance(batch, torch.Tensor):
        return [batch]
    if isinstance(batch, (list, tuple)):
        return [t for b in batch for t in _tensors(b)]
    if isinstance(batch, dict):
        return [t for k in sorted(batch) for t in _tensors(batch[k])]
    return []


class StaticBufferLoader:
    """Copies every batch into the same device buffers (one set per batch signature) so that a captured graph sees stable
    addresses."""

    def __init__(self, device: torch.device):
        self.device = device
        self.buffers: Dict[Tuple, Any] = {}

    @staticmethod
    def signature(batch) -> Tuple:
        return tuple((tuple(t.shape), str(t.dtype)) for t in _tensors(batch))

    def _like(self, batch):
        if isinstance(batch, torch.Tensor):
            return torch.empty_like(batch, device=self.device)
        if isinstance(batch, (list, tuple)):
            return type(batch)(self._like(b) for b in batch)
        if isinstance(batch, dict):
            return {k: self._like(v) for k, v in batch.items()}
        return batch

    def load(self, batch):
        sig = self.signature(batch)
        if sig not in self.buffers:
            self.buffers[sig] = self._like(batch)
        static = self.buffers[sig]
        for dst, src in zip(_tensors(static), _tensors(batch)):
            dst.copy_(src, non_blocking=True)
        return static


class CUDAGraphCallback(Callback):
    """Replays the forward + backward pass of a training iteration from a CUDA graph.

    One graph per batch signature (shapes and dtypes of all tensors in the batch), at most ``max_graphs`` of them — other
    batches run eagerly, so bucketed data with a handful of shapes benefits and arbitrary shapes still train.  Gradient
    zeroing, forward and backward are captured; gradient exchange, clipping, the optimizer update and the scheduler stay
    outside the graph (their host-side arguments — learning rate, step count — change every iteration).  Stateless dropout
    draws its seeds on the host, so a captured dropout mask would repeat: models with active dropout are refused unless
    ``allow_fixed_dropout_mask`` is set."""

    def __init__(self, warmup_steps: int = 3, max_graphs: int = 8, allow_fixed_dropout_mask: bool = False):
        self.warmup_steps, self.max_graphs, self.allow_fixed = warmup_steps, max_graphs, allow_fixed_dropout_mask
        self.graphs: "OrderedDict[Tuple, Dict[str, Any]]" = OrderedDict()
        self.seen: Dict[Tuple, int] = {}
        self.replays = 0
        self.loader: Optional[StaticBufferLoader] = None

    def setup(self, trainer, model, stage=None):
        if trainer.device.type != "cuda":
            logging.warning("CUDAGraphCallback: not a CUDA device, the callback stays inactive")
            return
        if not self.allow_fixed and any(isinstance(m, torch.nn.Dropout) and m.p > 0 for m in model.modules()):
            raise ValueError("CUDAGraphCallback: the model has active dropout; a captured mask would repeat every iteration "
                             "(set dropout to 0 or pass allow_fixed_dropout_mask=True)")
        self.loader = StaticBufferLoader(trainer.device)
        self._eager = trainer._train_batch
        trainer._train_batch = lambda batch, batch_idx: self._train_batch(trainer, batch, batch_idx)

    def on_fit_end(self, trainer, model):
        if self.loader is not None:
            trainer._train_batch = self._eager
            self.loader = None

    def _fwd_bwd(self, trainer, batch, batch_idx):
        for opt in trainer.optimizers:
            opt.zero_grad(set_to_none=False)
        with trainer.precision_context():
            out = trainer.model.training_step(batch, batch_idx)
        loss = out["loss"] if isinstance(out, dict) else out
        loss.backward()
        return loss

    def _train_batch(self, trainer, batch, batch_idx):
        from ..core.trainer import move_to_device

        if trainer.accumulate_grad_batches != 1:
            return self._eager(batch, batch_idx)
        batch = move_to_device(batch, trainer.device, None)
        sig = StaticBufferLoader.signature(batch)
        n = self.seen.get(sig, 0)
        self.seen[sig] = n + 1
        entry = self.graphs.get(sig)
        if entry is None and (n < self.warmup_steps or len(self.graphs) >= self.max_graphs):
            return self._eager(batch, batch_idx)
        static = self.loader.load(batch)
        sync = trainer.grad_sync
        if entry is None:
            g = torch.cuda.CUDAGraph()
            ctx = sync.no_sync() if sync is not None else _null()
            torch.cuda.synchronize()
            with ctx, torch.cuda.graph(g):
                loss = self._fwd_bwd(trainer, static, batch_idx)
            entry = self.graphs[sig] = {"graph": g, "loss": loss}
            logging.info(f"CUDAGraphCallback: captured a training graph for batch signature #{len(self.graphs)}")
        trainer.model.on_train_batch_start(batch, batch_idx)
        trainer._call("on_train_batch_start", batch, batch_idx)
        entry["graph"].replay()
        self.replays += 1
        loss = entry["loss"]
        if sync is not None:                        # gradients are final only now: exchange all buckets after the replay
            sync.begin_step()
            sync.finish_step()
        for opt in trainer.optimizers:
            trainer._clip_gradients(opt)
            trainer._call("on_before_optimizer_step", opt)
            opt.step()
        for sc in trainer.lr_scheduler_configs:
            if sc.get("interval", "step") == "step" and not sc.get("reduce_on_plateau", False):
                sc["scheduler"].step()
        trainer.global_step += 1
        out = {"loss": loss.detach()}
        trainer.model.on_train_batch_end(out, batch, batch_idx)
        trainer._call("on_train_batch_end", out, batch, batch_idx)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# ---------------------------------------------------------------------------------------------- callback group
class CallbackGroup:
    """Process-wide fan-out of application life-cycle events (model / data loader / optimizer initialisation, checkpoint load
    and save, start and end of the application) to registered observers, e.g. a telemetry logger."""

    _instance: Optional["CallbackGroup"] = None
    _lock = threading.Lock()
    EVENTS = ("on_app_start", "on_app_end", "on_model_init_start", "on_model_init_end", "on_dataloader_init_start", "on_dataloader_init_end",
              "on_optimizer_init_start", "on_optimizer_init_end", "on_load_checkpoint_start", "on_load_checkpoint_end",
              "on_save_checkpoint_start", "on_save_checkpoint_end", "on_save_checkpoint_success", "update_config")

    def __init__(self):
        self._callbacks: List[Any] = []

    @classmethod
    def get_instance(cls) -> "CallbackGroup":
        with cls._lock:
            if cls._instance is None:
                cls._instance = cls()
            return cls._instance

    def register(self, cb) -> None:
        if cb not in self._callbacks:
            self._callbacks.append(cb)

    def clear(self) -> None:
        self._callbacks.clear()

    def __getattr__(self, name: str) -> Callable:
        if name.startswith("_"):
            raise AttributeError(name)

        def fan_out(*a, **kw):
            for cb in list(self._callbacks):
                fn = getattr(cb, name, None)
                if callable(fn):
                    fn(*a, **kw)

        return fan_out


def hook_class_init_with_callbacks(cls, start_event: str, end_event: str):
    """Wrap ``cls.__init__`` so the group hears ``start_event`` before and ``end_event`` after every construction."""
    if getattr(cls.__init__, "_callback_group_wrapped", False):
        return cls
    orig = cls.__init__

    def wrapped(self, *a, **kw):
        group = CallbackGroup.get_instance()
        getattr(group, start_event)()
        orig(self, *a, **kw)
        getattr(group, end_event)()

    wrapped._callback_group_wrapped = True
    cls.__init__ = wrapped
    return cls


class EventRecorder:
    """Minimal observer: timestamps of every event, as a telemetry back-end would collect them."""

    def __init__(self, clock: Callable[[], float] = None):
        import time

        self.clock = clock or time.time
        self.events: List[Tuple[str, float]] = []

    def __getattr__(self, name):
        if name.startswith("on_") or name == "update_config":
            return lambda *a, **kw: self.events.append((name, self.clock()))
        raise AttributeError(name)


# ---------------------------------------------------------------------------------------------- profiler control
class NsightProfiling(Callback):
    """Opens the CUDA profiler range (``cudaProfilerStart``) at ``begin_step`` and closes it at ``end_step`` on the chosen ranks,
    optionally with NVTX shape annotations, so that an external profiler launched with capture-range=cudaProfilerApi records
    exactly those iterations."""

    def __init__(self, begin_step: int, end_step: int, ranks: Optional[List[int]] = None, gen_shape: bool = False):
        if end_step < begin_step:
            raise ValueError("end_step must be >= begin_step")
        self.begin_step, self.end_step, self.ranks, self.gen_shape = begin_step, end_step, list(ranks or [0]), gen_shape
        self.active = False
        self._nvtx_ctx = None

    def on_train_batch_start(self, trainer, model, batch, batch_idx):
        if trainer.global_step == self.begin_step and getattr(trainer, "global_rank", 0) in self.ranks and trainer.device.type == "cuda":
            torch.cuda.cudart().cudaProfilerStart()
            if self.gen_shape:
                self._nvtx_ctx = torch.autograd.profiler.emit_nvtx(record_shapes=True)
                self._nvtx_ctx.__enter__()
            self.active = True

    def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
        if self.active and trainer.global_step >= self.end_step:
            if self._nvtx_ctx is not None:
                self._nvtx_ctx.__exit__(None, None, None)
                self._nvtx_ctx = None
            torch.cuda.cudart().cudaProfilerStop()
            self.active = False


# ---------------------------------------------------------------------------------------------- object-store checkpoint IO
class ObjectStoreCheckpointIO:
    """``save_checkpoint`` / ``load_checkpoint`` / ``remove_checkpoint`` for ``s3://bucket/key`` and ``msc://profile/path`` URLs.
    Checkpoints are written to a local staging directory first and uploaded by a background thread (``async_checkpointing``);
    plain paths are handled locally.  The transfer client is injected (an object with ``upload_file(local, bucket, key)``,
    ``download_file(bucket, key, local)`` and ``delete_object(Bucket=, Key=)``) or created from ``boto3`` when installed."""

    def __init__(self, client=None, staging_dir: Optional[str] = None, async_checkpointing: bool = False):
        self.client, self.async_checkpointing = client, async_checkpointing
        self.staging_dir = staging_dir or os.path.join(os.environ.get("TMPDIR", "/tmp"), "speech_b200_ckpt_staging")
        self._threads: List[threading.Thread] = []

    @staticmethod
    def is_remote(path: str) -> bool:
        return path.startswith("s3://") or path.startswith("msc://")

    @staticmethod
    def parse(path: str) -> Tuple[str, str]:
        rest = path.split("://", 1)[1]
        bucket, _, key = rest.partition("/")
        return bucket, key

    def _client(self):
        if self.client is None:
            try:
                import boto3
            except ImportError as e:
                raise ImportError("object-store checkpoint IO needs a transfer client (pass `client=`) or the boto3 package") from e
            self.client = boto3.client("s3")
        return self.client

    def save_checkpoint(self, checkpoint: Dict[str, Any], path: str, storage_options=None) -> None:
        if not self.is_remote(path):
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            torch.save(checkpoint, path)
            return
        bucket, key = self.parse(path)
        os.makedirs(self.staging_dir, exist_ok=True)
        local = os.path.join(self.staging_dir, key.replace("/", "__"))
        torch.save(checkpoint, local)

        def upload():
            self._client().upload_file(local, bucket, key)
            os.remove(local)

        if self.async_checkpointing:
            t = threading.Thread(target=upload, daemon=True)
            t.start()
            self._threads.append(t)
        else:
            upload()

    def wait(self) -> None:
        for t in self._threads:
            t.join()
        self._threads = []

    def load_checkpoint(self, path: str, map_location="cpu") -> Dict[str, Any]:
        if not self.is_remote(path):
            return torch.load(path, map_location=map_location, weights_only=False)
        bucket, key = self.parse(path)
        os.makedirs(self.staging_dir, exist_ok=True)
        local = os.path.join(self.staging_dir, "dl__" + key.replace("/", "__"))
        self._client().download_file(bucket, key, local)
        try:
            return torch.load(local, map_location=map_location, weights_only=False)
        finally:
            os.remove(local)

    def remove_checkpoint(self, path: str) -> None:
        if not self.is_remote(path):
            if os.path.isdir(path):
                shutil.rmtree(path)
            elif os.path.exists(path):
                os.remove(path)
            return
        bucket, key = self.parse(path)
        self._client().delete_object(Bucket=bucket, Key=key)


# ---------------------------------------------------------------------------------------------- Hugging Face directory / hub IO
class HuggingFaceFileIO:
    """Mixin for ``ModelPT`` subclasses: a model directory in the Hugging Face layout (``config.json`` with the model config and
    class path, ``model.safetensors``-style weights saved with torch, tokenizer artifacts) that ``from_pretrained`` reads back;
    ``push_to_hub`` / hub downloads need the optional ``huggingface_hub`` package and network access."""

    def save_pretrained(self, save_directory: str) -> str:
        from ..core.config import OmegaConf

        os.makedirs(save_directory, exist_ok=True)
        cfg = OmegaConf.to_container(self.cfg, resolve=True) if hasattr(self, "cfg") else {}
        with open(os.path.join(save_directory, "config.json"), "w", encoding="utf-8") as f:
            json.dump({"target": f"{type(self).__module__}.{type(self).__qualname__}", "model_config": cfg}, f, indent=1, default=str)
        torch.save({k: v.detach().cpu() for k, v in self.state_dict().items()}, os.path.join(save_directory, "model_weights.pt"))
        return save_directory

    @classmethod
    def from_pretrained(cls, model_name_or_path: str, map_location="cpu", strict: bool = True, **kw):
        path = model_name_or_path
        if not os.path.isdir(path):
            try:
                from huggingface_hub import snapshot_download
            except ImportError as e:
                raise FileNotFoundError(f"{path} is not a local model directory and huggingface_hub is not installed") from e
            path = snapshot_download(repo_id=model_name_or_path, **kw)
        from ..core.config import OmegaConf
        from ..core.instantiate import locate

        meta = json.load(open(os.path.join(path, "config.json"), encoding="utf-8"))
        target = locate(meta["target"]) if cls is HuggingFaceFileIO or not hasattr(cls, "state_dict") else cls
        model = target(OmegaConf.create(meta["model_config"]))
        model.load_state_dict(torch.load(os.path.join(path, "model_weights.pt"), map_location=map_location), strict=strict)
        return model

    def push_to_hub(self, repo_id: str, **kw):
        try:
            from huggingface_hub import HfApi
        except ImportError as e:
            raise ImportError("push_to_hub needs the huggingface_hub package") from e
        import tempfile

        with tempfile.TemporaryDirectory() as d:
            self.save_pretrained(d)
            return HfApi().upload_folder(repo_id=repo_id, folder_path=d, **kw)


class IPLEpochStopper(Callback):
    """Stops training at the end of every ``stop_every_n_epochs``-th epoch when ``enable_stop`` is set.  Iterative pseudo-labelling
    alternates training with re-labelling of the unlabelled data: the trainer stops here, labels are regenerated with the current
    model, and training resumes from the checkpoint (reference: ``common/callbacks/ipl_epoch_stopper.py``)."""

    def __init__(self, enable_stop: bool = False, stop_every_n_epochs: int = 1):
        self.enable_stop, self.every = bool(enable_stop), int(stop_every_n_epochs)
        self._left = self.every

    def on_train_epoch_end(self, trainer, model):
        if not self.enable_stop:
            return
        self._left -= 1
        if self._left <= 0:
            trainer.should_stop = True
            self._left = self.every

    def state_dict(self):
        return {"left": self._left}

    def load_state_dict(self, sd):
        self._left = int(sd.get("left", self.every))

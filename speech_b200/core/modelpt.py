"""``ModelPT``: the base class of every trainable model.

Behaviour modelled on the reference's base class (``nemo/core/classes/modelPT.py:52``):
configs become ``DictConfig`` and are stored on the model (``:105-125``); train / validation /
test loaders are built from ``cfg.{train,validation,test}_ds`` (``:149-171``); artifacts are
registered for packing into ``.nemo`` files (``:233``); ``save_to`` / ``restore_from``
(``:391,433``); optimizer + scheduler from ``cfg.optim`` (``:627-792``); multi-dataloader
validation / test epoch end (``:961,1057``); partial initialisation from other checkpoints
(``:1262``).  The hook names are the Lightning ones so user code written against the reference
carries over; they are driven by :class:`speech_b200.core.trainer.Trainer`.
"""
from __future__ import annotations

import copy
import inspect
import os
import uuid
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from ..utils.logging import AppState, is_global_rank_zero, logging
from .config import DictConfig, ListConfig, OmegaConf, open_dict, to_container
from .module import NeuralModule, Serialization, Typing
from .optim import lr_scheduler as _sched
from .optim import optimizers as _optim
from .save_restore import SaveRestoreConnector

__all__ = ["ModelPT", "PretrainedModelInfo"]


class PretrainedModelInfo:
    def __init__(self, pretrained_model_name: str, description: str = "", location: str = "", class_=None,
                 aliases: Optional[List[str]] = None):
        self.pretrained_model_name, self.description, self.location = pretrained_model_name, description, location
        self.class_, self.aliases = class_, aliases

    def __repr__(self):
        return f"PretrainedModelInfo(name={self.pretrained_model_name}, location={self.location})"


class ModelPT(nn.Module, Typing, Serialization):
    _save_restore_connector = SaveRestoreConnector()
    _is_model_being_restored = False
    _nemo_file_folder: Optional[str] = None

    def __init__(self, cfg: DictConfig, trainer=None):
        if trainer is not None and not hasattr(trainer, "fit"):
            raise ValueError(f"trainer must be a Trainer-like object, got {type(trainer)}")
        super().__init__()
        if isinstance(cfg, dict):
            cfg = OmegaConf.create(cfg)
        if not isinstance(cfg, DictConfig):
            raise ValueError(f"cfg constructor argument must be of type DictConfig/dict but got {type(cfg)} instead.")
        if "model" in cfg and "trainer" in cfg and "preprocessor" not in cfg:
            raise ValueError("Creating model config node is forbidden due to collision problem when loading from "
                             "checkpoint: pass cfg.model instead of the whole experiment config.")
        cfg = copy.deepcopy(cfg)
        OmegaConf.set_struct(cfg, False)
        if "target" not in cfg:
            cfg["target"] = f"{type(self).__module__}.{type(self).__name__}"
        if "nemo_version" not in cfg:
            from .. import __version__

            cfg["nemo_version"] = __version__
        self._cfg = cfg
        self.model_guid = str(uuid.uuid4())
        AppState().register_model_guid(self.model_guid, AppState().model_restore_path if self._is_model_being_restored else None)
        self._restore_folder = type(self)._nemo_file_folder if self._is_model_being_restored else None
        self.artifacts: Dict[str, Dict[str, Any]] = self.__dict__.get("artifacts", None) or {}
        self._trainer = trainer
        self.world_size = 1
        if trainer is not None:
            self.set_world_size(trainer)
        self._train_dl = self._validation_dl = self._test_dl = None
        self._optimizer = None
        self._scheduler = None
        self._optimizer_param_groups = None
        self._validation_names = self._test_names = None
        self._validation_dl_idx = self._test_dl_idx = 0
        self.validation_step_outputs: Any = []
        self.test_step_outputs: Any = []
        self._logged: Dict[str, Any] = {}
        self.global_step_override: Optional[int] = None
        self._nemo_submodule_fields: List[str] = []
        if not self._is_model_being_restored:
            self._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ trainer plumbing
    @property
    def trainer(self):
        return self._trainer

    def set_trainer(self, trainer) -> None:
        self._trainer = trainer
        self.set_world_size(trainer)

    def set_world_size(self, trainer) -> None:
        self.world_size = 1
        if trainer is not None:
            self.world_size = max(1, int(getattr(trainer, "world_size", 1) or 1))

    @property
    def device(self) -> torch.device:
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")

    @property
    def global_step(self) -> int:
        if self.global_step_override is not None:
            return self.global_step_override
        return int(getattr(self._trainer, "global_step", 0)) if self._trainer is not None else 0

    @property
    def current_epoch(self) -> int:
        return int(getattr(self._trainer, "current_epoch", 0)) if self._trainer is not None else 0

    @property
    def local_rank(self) -> int:
        return int(getattr(self._trainer, "local_rank", 0)) if self._trainer is not None else 0

    @property
    def global_rank(self) -> int:
        return int(getattr(self._trainer, "global_rank", 0)) if self._trainer is not None else 0

    def log(self, name: str, value: Any, prog_bar: bool = False, sync_dist: bool = False, batch_size=None, **kw):
        if torch.is_tensor(value):
            value = value.detach()
        self._logged[name] = value
        if self._trainer is not None and hasattr(self._trainer, "_collect_log"):
            self._trainer._collect_log(name, value, sync_dist=sync_dist)

    def log_dict(self, d: Dict[str, Any], **kw):
        for k, v in d.items():
            self.log(k, v, **kw)

    # ------------------------------------------------------------------ cfg
    @property
    def cfg(self) -> DictConfig:
        return self._cfg

    @cfg.setter
    def cfg(self, cfg):
        self._cfg = cfg if isinstance(cfg, DictConfig) else OmegaConf.create(cfg)
        OmegaConf.set_struct(self._cfg, False)

    @property
    def hparams(self):
        return {"cfg": self._cfg}

    def to_config_file(self, path2yaml_file: str):
        OmegaConf.save(self._cfg, path2yaml_file, resolve=True)

    @classmethod
    def from_config_file(cls, path2yaml_file: str, trainer=None):
        conf = OmegaConf.load(path2yaml_file)
        if "model" in conf:
            conf = conf.model
        return cls.from_config_dict(conf, trainer=trainer)

    @classmethod
    def from_config_dict(cls, config, trainer=None):
        if isinstance(config, dict):
            config = OmegaConf.create(config)
        target = config.get("target", None) if isinstance(config, DictConfig) else None
        use_cls = cls
        if target is not None:
            from .instantiate import locate

            try:
                cand = locate(target)
                if isinstance(cand, type) and issubclass(cand, cls):
                    use_cls = cand
            except Exception:
                pass
        return use_cls(cfg=config, trainer=trainer)

    # ------------------------------------------------------------------ artifacts / nested models
    def register_artifact(self, config_path: str, src: str, verify_src_exists: bool = True):
        if src is None or src == "":
            return src
        return self._save_restore_connector.register_artifact(self, config_path, src, verify_src_exists)

    def has_artifacts(self) -> bool:
        return len(self.artifacts) > 0

    def register_nemo_submodule(self, name: str, config_field: str, model: "ModelPT") -> None:
        if not isinstance(model, ModelPT):
            raise ValueError(f"Model {name} is not and instance of ModelPT")
        setattr(self, name, model)
        model._nemo_config_field = config_field
        self._nemo_submodule_fields.append(name)
        with open_dict(self._cfg):
            self._cfg[config_field] = model.cfg

    def has_nemo_submodules(self) -> bool:
        return any(True for n, _ in self.named_nemo_modules() if n != "")

    def named_nemo_modules(self, prefix_name: str = ""):
        yield prefix_name, self
        for name, mod in self.named_children():
            if isinstance(mod, ModelPT):
                yield from mod.named_nemo_modules((prefix_name + "." if prefix_name else "") + name)

    # ------------------------------------------------------------------ save / restore
    def save_to(self, save_path: str):
        return self._save_restore_connector.save_to(self, save_path)

    @classmethod
    def restore_from(cls, restore_path: str, override_config_path=None, map_location=None, strict: bool = True,
                     return_config: bool = False, save_restore_connector: Optional[SaveRestoreConnector] = None,
                     trainer=None, validate_access_integrity: bool = True):
        connector = save_restore_connector or SaveRestoreConnector()
        if not os.path.exists(restore_path):
            raise FileNotFoundError(f"Can't find {restore_path}")
        cls.update_save_restore_connector(connector)
        instance = connector.restore_from(cls, restore_path, override_config_path, map_location, strict,
                                          return_config, trainer, validate_access_integrity)
        if isinstance(instance, ModelPT):
            instance._save_restore_connector = connector
        return instance

    @classmethod
    def update_save_restore_connector(cls, connector):
        cls._save_restore_connector = connector

    @classmethod
    def _set_model_restore_state(cls, is_being_restored: bool, folder: Optional[str] = None):
        ModelPT._is_model_being_restored = is_being_restored
        ModelPT._nemo_file_folder = folder

    @classmethod
    def list_available_models(cls) -> List[PretrainedModelInfo]:
        """Published checkpoints of this class (``core/model_catalog.py``); a subclass that overrides this with ``[]`` has none."""
        from .model_catalog import entries_for_class

        return [PretrainedModelInfo(pretrained_model_name=e.name, description=e.description, location=e.location, class_=cls) for e in entries_for_class(cls)]

    @classmethod
    def from_pretrained(cls, model_name: str, refresh_cache: bool = False, override_config_path=None,
                        map_location=None, strict: bool = True, return_config: bool = False, trainer=None,
                        save_restore_connector=None):
        """Load by name.  A path to a ``.nemo`` file or an extracted directory is used directly; a
        ``org/name`` id is looked up in the local Hugging Face cache (this build has no network)."""
        from .model_catalog import resolve_local

        path = None
        if os.path.exists(model_name):
            path = model_name
        elif resolve_local(model_name) is not None:
            path = resolve_local(model_name)
        elif "/" in model_name:
            try:
                from huggingface_hub import snapshot_download

                snap = snapshot_download(repo_id=model_name, local_files_only=True)
                nemo_files = [f for f in os.listdir(snap) if f.endswith(".nemo")]
                path = os.path.join(snap, nemo_files[0]) if nemo_files else snap
            except Exception as e:
                raise FileNotFoundError(f"Model '{model_name}' is not in the local Hugging Face cache: {e}")
        else:
            for info in cls.list_available_models():
                if info.pretrained_model_name == model_name and os.path.exists(info.location):
                    path = info.location
        if path is None:
            raise FileNotFoundError(f"Model {model_name} was not found. No network access: pass a local .nemo path.")
        return cls.restore_from(path, override_config_path, map_location, strict, return_config,
                                save_restore_connector, trainer)

    @classmethod
    def load_from_checkpoint(cls, checkpoint_path: str, map_location=None, strict: bool = True, trainer=None, **kw):
        """Load a trainer ``.ckpt`` (``{"state_dict", "hyper_parameters": {"cfg": ...}}``)."""
        ckpt = torch.load(checkpoint_path, map_location=map_location or "cpu", weights_only=False)
        cfg = ckpt.get("hyper_parameters", {}).get("cfg", None)
        if cfg is None:
            raise ValueError(f"{checkpoint_path} has no hyper_parameters.cfg")
        cfg = OmegaConf.create(cfg) if not isinstance(cfg, DictConfig) else cfg
        cls._set_model_restore_state(True)
        try:
            model = cls.from_config_dict(cfg, trainer=trainer)
        finally:
            cls._set_model_restore_state(False)
        model.load_state_dict(ckpt["state_dict"], strict=strict)
        return model

    def maybe_init_from_pretrained_checkpoint(self, cfg: DictConfig, map_location: str = "cpu"):
        """``init_from_nemo_model`` / ``init_from_pretrained_model`` / ``init_from_ptl_ckpt`` with
        optional ``include`` / ``exclude`` name filters per source."""
        keys = [k for k in ("init_from_nemo_model", "init_from_pretrained_model", "init_from_ptl_ckpt") if cfg.get(k)]
        if len(keys) > 1:
            raise ValueError(f"Cannot pass more than one model initialization arguments to config! Found : {keys}")
        if not keys:
            return
        key = keys[0]
        spec = cfg[key]
        entries: List[Tuple[str, List[str], List[str]]] = []
        if isinstance(spec, str):
            entries.append((spec, [""], []))
        else:
            for _, v in (spec.items() if isinstance(spec, DictConfig) else dict(spec).items()):
                entries.append((v["path"] if "path" in v else v["name"], list(v.get("include", [""]) or [""]),
                                list(v.get("exclude", []) or [])))
        for path, include, exclude in entries:
            if key == "init_from_ptl_ckpt":
                sd = torch.load(path, map_location=map_location, weights_only=False)["state_dict"]
            else:
                loader = ModelPT.restore_from if key == "init_from_nemo_model" else ModelPT.from_pretrained
                other = loader(path, map_location=map_location, strict=False)
                sd = other.state_dict()
                del other
            self.load_part_of_state_dict(sd, include, exclude, f"{key}:{path}")

    def load_part_of_state_dict(self, state_dict, include, exclude, load_from_string=None):
        own = self.state_dict()
        picked = {}
        for k, v in state_dict.items():
            if not any(k.startswith(i) or i == "" for i in include):
                continue
            if any(k.startswith(e) for e in exclude):
                continue
            if k in own and own[k].shape == v.shape:
                picked[k] = v
        own.update(picked)
        self.load_state_dict(own, strict=False)
        logging.info(f"Model checkpoint partially restored from {load_from_string}: {len(picked)} tensors")

    # ------------------------------------------------------------------ data
    def _setup_dataloaders_from_cfg(self):
        cfg = self._cfg
        if "train_ds" in cfg and cfg.train_ds is not None and not cfg.train_ds.get("defer_setup", False):
            self.setup_training_data(cfg.train_ds)
        if "validation_ds" in cfg and cfg.validation_ds is not None and not cfg.validation_ds.get("defer_setup", False):
            self.setup_multiple_validation_data(val_data_config=cfg.validation_ds)
        if "test_ds" in cfg and cfg.test_ds is not None and not cfg.test_ds.get("defer_setup", False):
            self.setup_multiple_test_data(test_data_config=cfg.test_ds)

    def setup_training_data(self, train_data_config):
        pass

    def setup_validation_data(self, val_data_config):
        pass

    def setup_test_data(self, test_data_config):
        pass

    def _multi(self, config, setup_fn, names_attr: str, dl_attr: str):
        """Manifest lists -> one dataloader per entry, remembering a short name for each."""
        key = None
        for cand in ("manifest_filepath", "tarred_audio_filepaths", "cuts_path", "input_cfg"):
            if config is not None and cand in config and isinstance(config[cand], (list, ListConfig)) and cand != "input_cfg":
                key = cand
                break
        if key is None or len(config[key]) <= 1:
            setup_fn(config)
            return
        dls, names = [], []
        for entry in config[key]:
            sub = copy.deepcopy(config)
            sub[key] = entry
            setup_fn(sub)
            dls.append(getattr(self, dl_attr))
            names.append(os.path.splitext(os.path.basename(str(entry)))[0])
        setattr(self, dl_attr, dls)
        setattr(self, names_attr, names)

    def setup_multiple_validation_data(self, val_data_config):
        self._validation_dl_idx = 0
        self._validation_names = None
        self._multi(val_data_config, self.setup_validation_data, "_validation_names", "_validation_dl")

    def setup_multiple_test_data(self, test_data_config):
        self._test_dl_idx = 0
        self._test_names = None
        self._multi(test_data_config, self.setup_test_data, "_test_names", "_test_dl")

    def train_dataloader(self):
        return self._train_dl

    def val_dataloader(self):
        return self._validation_dl

    def test_dataloader(self):
        return self._test_dl

    # ------------------------------------------------------------------ optimisation
    def setup_optimizer_param_groups(self):
        """Per-module parameter groups when ``cfg.optim_param_groups`` is given (``modelPT.py:794``)."""
        known_groups = []
        param_groups = []
        if "optim_param_groups" in self.cfg:
            param_groups_cfg = self.cfg.optim_param_groups
            for group, group_cfg in param_groups_cfg.items():
                module = getattr(self, group, None)
                if module is None:
                    raise ValueError(f"{group} not found in model.")
                if not hasattr(module, "parameters"):
                    raise ValueError(f"{group} does not have parameters.")
                known_groups.append(group)
                new_group = {"params": list(module.parameters())}
                for k, v in group_cfg.items():
                    new_group[k] = v
                param_groups.append(new_group)
            other = [p for n, p in self.named_parameters() if n.split(".")[0] not in known_groups]
            if other:
                param_groups = [{"params": other}] + param_groups
        else:
            param_groups = [{"params": list(self.parameters())}]
        self._optimizer_param_groups = param_groups

    def setup_optimization(self, optim_config: Optional[Union[DictConfig, Dict]] = None,
                           optim_kwargs: Optional[Dict[str, Any]] = None):
        self.setup_optimizer_param_groups()
        if optim_config is None:
            optim_config = self._cfg.get("optim", None)
        if optim_config is None:
            logging.info("No optimizer config provided, therefore no optimizer was created")
            return None, None
        optim_config = OmegaConf.create(to_container(optim_config, resolve=True)) if isinstance(optim_config, DictConfig) \
            else OmegaConf.create(dict(optim_config))
        if optim_kwargs:
            for k, v in optim_kwargs.items():
                optim_config[k] = v
        sched_cfg = optim_config.get("sched", None)
        tr = self._trainer
        if sched_cfg is not None and tr is not None:
            with open_dict(optim_config):
                ms = getattr(tr, "max_steps", -1)
                if ms is not None and ms > 0:
                    optim_config.sched["max_steps"] = optim_config.sched.get("max_steps", None) or ms
                    if optim_config.sched["max_steps"] is None or optim_config.sched["max_steps"] < 0:
                        optim_config.sched["max_steps"] = ms
                else:
                    optim_config.sched["t_max_epochs"] = getattr(tr, "max_epochs", None)
                    optim_config.sched["t_accumulate_grad_batches"] = getattr(tr, "accumulate_grad_batches", 1)
                    optim_config.sched["t_limit_train_batches"] = getattr(tr, "limit_train_batches", 1.0)
                    optim_config.sched["t_num_workers"] = getattr(tr, "world_size", 1)
        name = optim_config.get("name", None)
        target = optim_config.get("_target_", None)
        kwargs = _optim.parse_optimizer_args(name, optim_config)
        lr = kwargs.pop("lr", None)
        if lr is None:
            raise ValueError("`lr` must be passed to `optimizer_config` when setting up the optimization !")
        groups = [g for g in self._optimizer_param_groups if len(g["params"]) > 0]
        groups = [{**g, "params": [p for p in g["params"] if p.requires_grad]} for g in groups]
        groups = [g for g in groups if g["params"]]
        if target is not None:
            from .instantiate import locate

            optimizer = locate(target)(groups, lr=lr, **kwargs)
        else:
            if name is None:
                raise ValueError("optim config needs `name` or `_target_`")
            use_fused = name in ("adamw",) and self._cfg.get("fused_optimizer", None) is not False and \
                all(p.dtype == torch.float32 for g in groups for p in g["params"]) and \
                (self.device.type == "cuda" or self._cfg.get("fused_optimizer", False))
            if use_fused:
                kwargs.pop("foreach", None), kwargs.pop("fused", None)
                clip = getattr(tr, "gradient_clip_val", 0.0) if tr is not None else 0.0
                fusion = [fg for m in self.modules() if hasattr(m, "arena_fusion_groups") for fg in m.arena_fusion_groups()]
                optimizer = _optim.get_optimizer("fused_adamw")(groups, lr=lr, max_grad_norm=clip or 0.0,
                                                                fusion_groups=fusion, **kwargs)
            elif name in ("fully_sharded_adamw", "fsdp2_adamw"):
                clip = getattr(tr, "gradient_clip_val", 0.0) if tr is not None else 0.0
                optimizer = _optim.get_optimizer(name)(groups, model=self, lr=lr, max_grad_norm=clip or 0.0, device=self.device,
                                                       **{**kwargs, **self._sharded_optimizer_kwargs()})
            else:
                optimizer = _optim.get_optimizer(name)(groups, lr=lr, **kwargs)
        self._optimizer = optimizer
        self._scheduler = _sched.prepare_lr_scheduler(optimizer, sched_cfg and optim_config, self._train_dl) \
            if sched_cfg is not None else None
        return self._optimizer, self._scheduler

    def load_state_dict(self, state_dict, strict: bool = True, **kw):
        """Adapters listed in ``cfg.adapters`` are rebuilt before the weights are loaded, so a check-point written with adapters
        restores into a freshly constructed model."""
        if hasattr(self, "restore_adapters_from_cfg"):
            self.restore_adapters_from_cfg()
        return super().load_state_dict(state_dict, strict=strict, **kw)

    def _sharded_optimizer_kwargs(self) -> Dict[str, Any]:
        """Extra arguments of the fully-sharded optimizer (``group``, ``replicate_group``, ``units``); models that live on a
        device mesh override this."""
        return {}

    def configure_optimizers(self):
        self.setup_optimization()
        if self._scheduler is None:
            return self._optimizer
        return [self._optimizer], [self._scheduler]

    # ------------------------------------------------------------------ hooks (no-ops by default)
    def on_fit_start(self):
        pass

    def on_train_start(self):
        pass

    def on_train_end(self):
        if getattr(self, "_step_hooks", None) is not None:
            self._step_hooks.close()

    def on_train_epoch_start(self):
        pass

    def on_train_epoch_end(self):
        pass

    def _hooks(self):
        """Profiling windows and scheduled freezing read from ``cfg`` on first use (see :mod:`speech_b200.core.profiling`)."""
        h = getattr(self, "_step_hooks", None)
        if h is None:
            from .profiling import StepHooks

            rank = torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0
            h = StepHooks(getattr(self, "cfg", None), rank=rank)
            object.__setattr__(self, "_step_hooks", h)
        return h

    def on_train_batch_start(self, batch, batch_idx: int):
        h = self._hooks()
        if h.active:
            h.batch_start(self, batch_idx, self.trainer.global_step if self.trainer is not None else batch_idx)

    def on_train_batch_end(self, outputs, batch, batch_idx: int):
        h = self._hooks()
        if h.active:
            h.batch_end(self, batch_idx, self.trainer.global_step if self.trainer is not None else batch_idx + 1)

    def on_after_backward(self):
        pass

    def on_validation_epoch_start(self):
        pass

    def on_test_epoch_start(self):
        pass

    def training_step(self, batch, batch_idx):
        raise NotImplementedError

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        raise NotImplementedError

    def test_step(self, batch, batch_idx, dataloader_idx=0):
        return self.validation_step(batch, batch_idx, dataloader_idx)

    def predict_step(self, batch, batch_idx, dataloader_idx=0):
        raise NotImplementedError

    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0) -> Optional[Dict[str, Any]]:
        return None

    def multi_test_epoch_end(self, outputs, dataloader_idx: int = 0) -> Optional[Dict[str, Any]]:
        return self.multi_validation_epoch_end(outputs, dataloader_idx)

    def get_validation_dataloader_prefix(self, dataloader_idx: int = 0) -> str:
        return (self._validation_names[dataloader_idx] + "_") if self._validation_names else ""

    def get_test_dataloader_prefix(self, dataloader_idx: int = 0) -> str:
        return (self._test_names[dataloader_idx] + "_") if self._test_names else ""

    @staticmethod
    def reduce_sums(values, device=None):
        """Sum a short list of python numbers over all ranks (identity without a process group).  Metrics that are ratios of
        sums (WER = errors / words, mean loss = sum / count) are formed from the reduced numerators and denominators, as the
        reference's torchmetrics-based WER does with ``dist_reduce_fx='sum'`` (``collections/asr/metrics/wer.py``)."""
        import torch.distributed as dist

        vals = [float(v) for v in values]
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            return vals
        on_gpu = dist.get_backend() == "nccl"
        t = torch.tensor(vals, dtype=torch.float64, device=device if (on_gpu and device is not None) else ("cuda" if on_gpu else "cpu"))
        dist.all_reduce(t)
        return [float(x) for x in t.cpu()]

    def _sync_logged(self, log: Dict[str, Any]) -> Dict[str, Any]:
        """Mean over ranks of every scalar about to be logged at an epoch end (``sync_dist=True`` of the reference,
        ``core/classes/modelPT.py:991``), so that ``trainer.callback_metrics``, and with it every checkpoint and early-stopping
        decision, is identical on all ranks."""
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            return log
        keys = sorted(k for k, v in log.items() if isinstance(v, (int, float)) or (torch.is_tensor(v) and v.numel() == 1))
        if not keys:
            return log
        world = dist.get_world_size()
        red = self.reduce_sums([float(log[k]) for k in keys], getattr(self, "device", None))
        out = dict(log)
        for k, v in zip(keys, red):
            out[k] = torch.tensor(v / world, dtype=torch.float32)
        return out

    def _epoch_end(self, outputs, multi_fn, prefix_fn, which: str):
        if not outputs:
            return {}
        single = not (isinstance(outputs[0], list))
        if single:
            out = multi_fn(outputs, 0) or {}
            log = out.pop("log", {}) if isinstance(out, dict) else {}
            log = self._sync_logged(log)
            out = self._sync_logged(out) if isinstance(out, dict) else out
            self.log_dict(log)
            for k, v in (out.items() if isinstance(out, dict) else []):
                self.log(k, v)
            return {**out, **log}
        merged: Dict[str, Any] = {}
        primary = self._validation_dl_idx if which == "val" else self._test_dl_idx
        for idx, douts in enumerate(outputs):
            if not douts:
                continue
            out = multi_fn(douts, idx) or {}
            prefix = prefix_fn(idx)
            log = out.pop("log", {}) if isinstance(out, dict) else {}
            for k, v in {**out, **log}.items():
                if idx == primary and k in (f"{which}_loss", f"{which}_wer"):
                    merged[k] = v
                merged[prefix + k] = v
        merged = self._sync_logged(merged)
        self.log_dict(merged)
        return merged

    def on_validation_epoch_end(self):
        out = self._epoch_end(self.validation_step_outputs, self.multi_validation_epoch_end,
                              self.get_validation_dataloader_prefix, "val")
        self.validation_step_outputs = [] if not (self.validation_step_outputs and isinstance(self.validation_step_outputs[0], list)) \
            else [[] for _ in self.validation_step_outputs]
        return out

    def on_test_epoch_end(self):
        out = self._epoch_end(self.test_step_outputs, self.multi_test_epoch_end, self.get_test_dataloader_prefix, "test")
        self.test_step_outputs = [] if not (self.test_step_outputs and isinstance(self.test_step_outputs[0], list)) \
            else [[] for _ in self.test_step_outputs]
        return out

    # ------------------------------------------------------------------ misc helpers
    def prepare_test(self, trainer) -> bool:
        self.eval()
        return True

    def summarize(self) -> str:
        total = sum(p.numel() for p in self.parameters())
        train = sum(p.numel() for p in self.parameters() if p.requires_grad)
        lines = [f"{type(self).__name__}: {total / 1e6:.1f} M params ({train / 1e6:.1f} M trainable)"]
        for n, m in self.named_children():
            lines.append(f"  {n:<24s}{type(m).__name__:<40s}{sum(p.numel() for p in m.parameters()) / 1e6:9.2f} M")
        return "\n".join(lines)

    @property
    def num_weights(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    def freeze(self):
        for p in self.parameters():
            p.requires_grad = False
        self.eval()

    def unfreeze(self):
        for p in self.parameters():
            p.requires_grad = True
        self.train()

"""``.nemo`` archive reader / writer.

A ``.nemo`` file is an *uncompressed* tar holding ``model_config.yaml``, ``model_weights.ckpt``
(a ``torch.save`` of the state dict) and any registered artifact files renamed to
``<uuid4hex>_<basename>`` with the config value rewritten to ``nemo:<uuid4hex>_<basename>``
(reference: ``nemo/core/connectors/save_restore_connector.py:48-49,455-615``).  Old archives
that were gzip-compressed are still readable (``:670-688``).  Extraction is guarded against
path traversal (reference: ``nemo/utils/tar_utils.py``).
"""
from __future__ import annotations

import os
import shutil
import tarfile
import tempfile
import uuid
from typing import Any, Dict, Optional, Tuple, Union

import torch

from ..utils.logging import AppState, logging
from .config import DictConfig, OmegaConf, open_dict


def safe_extract(tar: tarfile.TarFile, out_folder: str, members=None) -> None:
    base = os.path.realpath(out_folder)
    members = members if members is not None else tar.getmembers()
    for m in members:
        target = os.path.realpath(os.path.join(out_folder, m.name))
        if not (target == base or target.startswith(base + os.sep)):
            raise RuntimeError(f"Refusing to extract '{m.name}': path escapes the extraction directory")
        if m.issym() or m.islnk():
            link = os.path.realpath(os.path.join(os.path.dirname(target), m.linkname))
            if not link.startswith(base + os.sep):
                raise RuntimeError(f"Refusing to extract link '{m.name}' -> '{m.linkname}'")
        if m.isdev():
            raise RuntimeError(f"Refusing to extract device file '{m.name}'")
    try:
        tar.extractall(out_folder, members=members, filter="data")
    except TypeError:  # pragma: no cover (python < 3.12)
        tar.extractall(out_folder, members=members)


class SaveRestoreConnector:
    def __init__(self) -> None:
        self._model_config_yaml = "model_config.yaml"
        self._model_weights_ckpt = "model_weights.ckpt"
        self._model_extracted_dir: Optional[str] = None

    # ------------------------------------------------------------------ properties
    @property
    def model_config_yaml(self) -> str:
        return self._model_config_yaml

    @model_config_yaml.setter
    def model_config_yaml(self, v: str) -> None:
        self._model_config_yaml = v

    @property
    def model_weights_ckpt(self) -> str:
        return self._model_weights_ckpt

    @model_weights_ckpt.setter
    def model_weights_ckpt(self, v: str) -> None:
        self._model_weights_ckpt = v

    @property
    def model_extracted_dir(self) -> Optional[str]:
        return self._model_extracted_dir

    @model_extracted_dir.setter
    def model_extracted_dir(self, path: Optional[str]) -> None:
        self._model_extracted_dir = path

    # ------------------------------------------------------------------ save
    def save_to(self, model, save_path: str) -> str:
        from ..utils.logging import is_global_rank_zero

        # a fully-sharded model keeps its parameters as slices inside the optimizer: every rank takes part in assembling the
        # full values (a collective), then only rank 0 writes the archive
        opt = getattr(model, "_optimizer", None)
        full_sd = opt.full_model_state_dict() if hasattr(opt, "full_model_state_dict") else None
        if not is_global_rank_zero():
            return save_path
        save_path = os.path.abspath(os.path.expanduser(save_path))
        os.makedirs(os.path.dirname(save_path), exist_ok=True)
        with tempfile.TemporaryDirectory() as tmpdir:
            cfg_path = os.path.join(tmpdir, self.model_config_yaml)
            weights_path = os.path.join(tmpdir, self.model_weights_ckpt)
            model.to_config_file(path2yaml_file=cfg_path)
            if getattr(model, "has_nemo_submodules", lambda: False)():
                self._update_subconfigs(model, cfg_path)
            if getattr(model, "artifacts", None):
                self._handle_artifacts(model, nemo_file_folder=tmpdir)
                self._update_artifact_paths(model, path2yaml_file=cfg_path)
            self._save_state_dict_to_disk(full_sd if full_sd is not None else model.state_dict(), weights_path)
            self._make_nemo_file_from_folder(save_path, tmpdir)
        return save_path

    # ------------------------------------------------------------------ restore
    def load_config_and_state_dict(self, calling_cls, restore_path: str, override_config_path=None,
                                   map_location: Optional[torch.device] = None, strict: bool = True,
                                   return_config: bool = False, trainer=None, validate_access_integrity: bool = True):
        cwd = os.getcwd()
        if map_location is None:
            map_location = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
        app_state = AppState()
        tmp_ctx = None
        if self.model_extracted_dir is not None and os.path.isdir(self.model_extracted_dir):
            tmpdir = self.model_extracted_dir
        elif os.path.isdir(restore_path):
            tmpdir = restore_path
        else:
            tmp_ctx = tempfile.TemporaryDirectory()
            tmpdir = tmp_ctx.name
        try:
            if tmp_ctx is not None:
                members = None
                if return_config:
                    members = [self.model_config_yaml]
                self._unpack_nemo_file(restore_path, tmpdir, members=members)
            if override_config_path is None:
                config_yaml = os.path.join(tmpdir, self.model_config_yaml)
            else:
                config_yaml = override_config_path
            conf = OmegaConf.load(config_yaml) if not isinstance(config_yaml, (DictConfig,)) else config_yaml
            if override_config_path is not None and "model" in conf:
                conf = conf.model
            if return_config:
                return conf
            prev_folder = app_state.nemo_file_folder
            prev_restoring = app_state.is_model_being_restored
            app_state.nemo_file_folder = tmpdir
            app_state.is_model_being_restored = True
            app_state.model_restore_path = restore_path
            try:
                OmegaConf.set_struct(conf, True)
                calling_cls._set_model_restore_state(is_being_restored=True, folder=tmpdir)
                instance = calling_cls.from_config_dict(config=conf, trainer=trainer)
                instance = instance.to(map_location)
                weights = os.path.join(tmpdir, self.model_weights_ckpt)
                state_dict = self._load_state_dict_from_disk(weights, map_location=map_location)
            finally:
                calling_cls._set_model_restore_state(is_being_restored=False)
                app_state.nemo_file_folder = prev_folder
                app_state.is_model_being_restored = prev_restoring
        finally:
            os.chdir(cwd)
            if tmp_ctx is not None:
                tmp_ctx.cleanup()
        return conf, instance, state_dict

    def modify_state_dict(self, conf, state_dict):
        # Older checkpoints stored the CTC head under "decoder." in hybrid models etc.; nothing to do by default.
        return state_dict

    def load_instance_with_state_dict(self, instance, state_dict, strict: bool):
        missing, unexpected = instance.load_state_dict(state_dict, strict=False)
        # Non-persistent buffers from older versions are tolerated; anything else is a hard error in strict mode.
        if strict and (missing or unexpected):
            raise RuntimeError(
                f"Error(s) in loading state_dict for {type(instance).__name__}: "
                f"missing keys {list(missing)}, unexpected keys {list(unexpected)}"
            )
        if missing:
            logging.warning(f"Missing keys when restoring: {list(missing)[:8]}{'...' if len(missing) > 8 else ''}")
        if unexpected:
            logging.warning(f"Unexpected keys when restoring: {list(unexpected)[:8]}{'...' if len(unexpected) > 8 else ''}")
        instance._set_model_restore_state(is_being_restored=False)

    def restore_from(self, calling_cls, restore_path: str, override_config_path=None, map_location=None,
                     strict: bool = True, return_config: bool = False, trainer=None,
                     validate_access_integrity: bool = True):
        loaded = self.load_config_and_state_dict(calling_cls, restore_path, override_config_path, map_location,
                                                 strict, return_config, trainer, validate_access_integrity)
        if not isinstance(loaded, tuple):
            return loaded
        conf, instance, state_dict = loaded
        state_dict = self.modify_state_dict(conf, state_dict)
        self.load_instance_with_state_dict(instance, state_dict, strict)
        logging.info(f"Model {type(instance).__name__} was successfully restored from {restore_path}.")
        return instance

    def extract_state_dict_from(self, restore_path: str, save_dir: str, split_by_module: bool = False):
        os.makedirs(save_dir, exist_ok=True)
        with tempfile.TemporaryDirectory() as tmpdir:
            self._unpack_nemo_file(restore_path, tmpdir)
            state_dict = self._load_state_dict_from_disk(os.path.join(tmpdir, self.model_weights_ckpt), "cpu")
        if not split_by_module:
            self._save_state_dict_to_disk(state_dict, os.path.join(save_dir, self.model_weights_ckpt))
            return state_dict
        tops = sorted({k.split(".")[0] for k in state_dict})
        for top in tops:
            sub = {k[len(top) + 1:]: v for k, v in state_dict.items() if k.startswith(top + ".")}
            self._save_state_dict_to_disk(sub, os.path.join(save_dir, f"{top}.ckpt"))
        return state_dict

    # ------------------------------------------------------------------ artifacts
    def register_artifact(self, model, config_path: str, src: str, verify_src_exists: bool = True) -> Optional[str]:
        app_state = AppState()
        artifacts = model.artifacts
        if config_path in artifacts:
            logging.warning(f"Artifact '{config_path}' registered twice; keeping the first registration")
            return artifacts[config_path]["path"]
        if src is None or src == "":
            return src
        item: Dict[str, Any] = {"path": None, "path_type": None, "hashed_path": None}
        src_abs = os.path.abspath(src)
        if os.path.exists(src_abs):
            item.update(path=src_abs, path_type="LOCAL_PATH")
            ret = src_abs
        elif src.startswith("nemo:"):
            folder = app_state.nemo_file_folder or getattr(model, "_restore_folder", None)
            if folder is None:
                raise FileNotFoundError(f"'{src}' can only be resolved while a .nemo file is being restored")
            ret = os.path.abspath(os.path.join(folder, src[5:]))
            item.update(path=src, path_type="TAR_PATH")
            if not os.path.exists(ret) and verify_src_exists:
                raise FileNotFoundError(f"Artifact {src} not found inside the restored archive ({ret})")
        else:
            if verify_src_exists:
                raise FileNotFoundError(f"src path does not exist or it is not a path in nemo file. src value: {src}")
            return None
        artifacts[config_path] = item
        return ret

    def _handle_artifacts(self, model, nemo_file_folder: str) -> None:
        app_state = AppState()
        for conf_path, item in model.artifacts.items():
            if item["path_type"] == "LOCAL_PATH":
                src = item["path"]
            else:  # TAR_PATH: the file lives in the folder the model was restored from
                folder = getattr(model, "_restore_folder", None) or app_state.nemo_file_folder
                src = os.path.join(folder, item["path"][5:]) if folder else None
                if src is None or not os.path.exists(src):
                    restore = app_state.model_restore_path
                    if restore and os.path.isfile(restore):
                        with tarfile.open(restore, "r:*") as tar:
                            name = item["path"][5:]
                            mem = [m for m in tar.getmembers() if os.path.basename(m.name) == name]
                            safe_extract(tar, nemo_file_folder, members=mem)
                        item["hashed_path"] = item["path"]
                        continue
                    raise FileNotFoundError(f"Cannot find artifact {item['path']} to re-pack")
            base = os.path.basename(src)
            if item["path_type"] == "TAR_PATH":
                hashed = base  # keep the already-hashed name
            else:
                hashed = f"{uuid.uuid4().hex}_{base}"
            shutil.copy2(src, os.path.join(nemo_file_folder, hashed))
            item["hashed_path"] = "nemo:" + hashed

    def _update_artifact_paths(self, model, path2yaml_file: str) -> None:
        conf = OmegaConf.load(path2yaml_file)
        for conf_path, item in model.artifacts.items():
            if item.get("hashed_path"):
                OmegaConf.update(conf, conf_path, item["hashed_path"])
        OmegaConf.save(conf, path2yaml_file)

    def _update_subconfigs(self, model, path2yaml_file: str) -> None:
        conf = OmegaConf.load(path2yaml_file)
        for name, sub in model.named_nemo_modules():
            if name == "" or not getattr(sub, "cfg", None):
                continue
            key = getattr(sub, "_nemo_config_field", name)
            if key in conf:
                with open_dict(conf):
                    conf[key] = sub.cfg
        OmegaConf.save(conf, path2yaml_file)

    # ------------------------------------------------------------------ io helpers
    @staticmethod
    def _make_nemo_file_from_folder(filename: str, source_dir: str) -> None:
        with tarfile.open(filename, "w:") as tar:
            tar.add(source_dir, arcname=".")

    @staticmethod
    def _unpack_nemo_file(path2file: str, out_folder: str, members=None) -> str:
        if not os.path.exists(path2file):
            raise FileNotFoundError(f"{path2file} does not exist")
        try:
            tar = tarfile.open(path2file, "r:")
        except tarfile.ReadError:
            tar = tarfile.open(path2file, "r:gz")
        with tar:
            if members is not None:
                wanted = []
                for m in tar.getmembers():
                    if os.path.normpath(m.name) in {os.path.normpath(x) for x in members}:
                        wanted.append(m)
                safe_extract(tar, out_folder, members=wanted)
            else:
                safe_extract(tar, out_folder)
        return out_folder

    @staticmethod
    def _save_state_dict_to_disk(state_dict, filepath: str) -> None:
        torch.save({k: v.detach().cpu() if torch.is_tensor(v) else v for k, v in state_dict.items()}, filepath)

    @staticmethod
    def _load_state_dict_from_disk(model_weights: str, map_location="cpu"):
        try:
            return torch.load(model_weights, map_location=map_location, weights_only=True)
        except Exception:
            if os.environ.get("TORCH_FORCE_NO_WEIGHTS_ONLY_LOAD", "0") == "1":
                return torch.load(model_weights, map_location=map_location, weights_only=False)
            raise

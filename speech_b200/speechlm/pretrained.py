"""Initialising speech-LM models from what exists on disk.

* ``load_checkpoint(path)`` — a state dict from a ``.safetensors`` file, a ``.ckpt`` / ``.pt`` file (its ``state_dict`` key when
  present), a ``.nemo`` archive, a directory of safetensors shards (Hugging Face layout, with or without an index file) or a
  distributed-checkpoint directory.
* ``set_model_dict_for_partial_init`` — keeps the entries whose names and shapes match the model (optionally after stripping or
  adding a prefix) and reports what was skipped.
* ``init_model_from_checkpoint`` / ``init_perception_from_checkpoint`` / ``init_from_training_checkpoint`` — whole model, only the
  perception module (e.g. from an ASR checkpoint: ``encoder.*`` / ``preprocessor.*`` names are mapped under ``perception.``), or a
  trainer checkpoint of the same model.
* ``maybe_load_pretrained_models(model)`` — reads ``cfg.pretrained_s2s_model`` / ``cfg.pretrained_perception_from_s2s`` /
  ``cfg.init_from_checkpoint`` and applies the matching loader.
* ``update_perception_output_dim`` / ``move_embedding`` — the two config / module fix-ups the model constructors share.

Reference: ``speechlm2/parts/pretrained.py``.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..core.config import cfg_get, open_dict
from ..utils.logging import logging

__all__ = ["init_from_training_checkpoint", "init_model_from_checkpoint", "init_perception_from_checkpoint", "load_checkpoint", "maybe_load_pretrained_models",
           "move_embedding", "set_model_dict_for_partial_init", "update_perception_output_dim"]


def _load_safetensors_dir(path: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        files = sorted(set(json.load(open(idx))["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    out: Dict[str, torch.Tensor] = {}
    for f in files:
        out.update(load_file(os.path.join(path, f)))
    return out


def load_checkpoint(path: str) -> Dict[str, torch.Tensor]:
    if os.path.isdir(path):
        from ..utils.dcp_io import DCPCheckpointIO, is_dcp_checkpoint

        if is_dcp_checkpoint(path):
            return DCPCheckpointIO().load_checkpoint(path)[0]
        return _load_safetensors_dir(path)
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        return load_file(path)
    if path.endswith(".nemo"):
        import tempfile

        from ..core.save_restore import SaveRestoreConnector

        conn = SaveRestoreConnector()
        with tempfile.TemporaryDirectory() as tmp:
            conn._unpack_nemo_file(path, tmp, members=[conn.model_weights_ckpt])
            return conn._load_state_dict_from_disk(os.path.join(tmp, conn.model_weights_ckpt), "cpu")
    obj = torch.load(path, map_location="cpu", weights_only=False)
    return obj["state_dict"] if isinstance(obj, dict) and "state_dict" in obj else obj


def set_model_dict_for_partial_init(pretrained: Dict[str, torch.Tensor], model_dict: Dict[str, torch.Tensor], strip_prefix: str = "", add_prefix: str = ""
                                    ) -> Tuple[Dict[str, torch.Tensor], List[str], List[str]]:
    """-> ``(model_dict updated with every usable entry, names taken, names skipped with the reason)``."""
    taken, skipped = [], []
    out = dict(model_dict)
    for k, v in pretrained.items():
        name = k[len(strip_prefix):] if strip_prefix and k.startswith(strip_prefix) else k
        name = add_prefix + name
        if name not in model_dict:
            skipped.append(f"{k}: no parameter {name}")
        elif tuple(model_dict[name].shape) != tuple(v.shape):
            skipped.append(f"{k}: shape {tuple(v.shape)} vs {tuple(model_dict[name].shape)}")
        else:
            out[name] = v
            taken.append(name)
    return out, taken, skipped


def init_model_from_checkpoint(model: torch.nn.Module, checkpoint_path: str, strict: bool = False) -> Tuple[int, int]:
    sd, taken, skipped = set_model_dict_for_partial_init(load_checkpoint(checkpoint_path), model.state_dict())
    if strict and skipped:
        raise RuntimeError(f"{len(skipped)} entries of {checkpoint_path} do not fit the model, e.g. {skipped[:3]}")
    model.load_state_dict(sd, strict=False)
    logging.info(f"{checkpoint_path}: {len(taken)} tensors loaded, {len(skipped)} skipped")
    return len(taken), len(skipped)


def init_perception_from_checkpoint(model: torch.nn.Module, checkpoint_path: str) -> int:
    """Loads only ``perception.*``.  The checkpoint may be a speech LM (names already under ``perception.``) or an ASR model, whose
    ``encoder.*`` / ``preprocessor.*`` / ``spec_augmentation.*`` modules sit directly under the perception module here."""
    src = load_checkpoint(checkpoint_path)
    own = {k: v for k, v in model.state_dict().items() if k.startswith("perception.")}
    if any(k.startswith("perception.") for k in src):
        src = {k: v for k, v in src.items() if k.startswith("perception.")}
        sd, taken, _ = set_model_dict_for_partial_init(src, own)
    else:
        src = {k: v for k, v in src.items() if k.startswith(("encoder.", "preprocessor.", "spec_augmentation."))}
        sd, taken, _ = set_model_dict_for_partial_init(src, own, add_prefix="perception.")
    if not taken:
        raise RuntimeError(f"nothing in {checkpoint_path} matches the perception module")
    model.load_state_dict(sd, strict=False)
    logging.info(f"perception initialised from {checkpoint_path}: {len(taken)} tensors")
    return len(taken)


def init_from_training_checkpoint(model: torch.nn.Module, checkpoint_path: str) -> int:
    """A checkpoint written by the trainer for this very model (file or distributed directory): everything must match."""
    sd = load_checkpoint(checkpoint_path)
    missing, unexpected = model.load_state_dict({k: v for k, v in sd.items() if torch.is_tensor(v)}, strict=False)
    missing = [k for k in missing if "lora_" not in k]
    if missing or unexpected:
        raise RuntimeError(f"training checkpoint does not match: missing {missing[:5]}, unexpected {list(unexpected)[:5]}")
    return len(sd)


def maybe_load_pretrained_models(model: torch.nn.Module) -> None:
    cfg = model.cfg
    if cfg_get(cfg, "pretrained_s2s_model", None):
        init_model_from_checkpoint(model, cfg.pretrained_s2s_model)
    if cfg_get(cfg, "pretrained_perception_from_s2s", None):
        init_perception_from_checkpoint(model, cfg.pretrained_perception_from_s2s)
    if cfg_get(cfg, "init_from_checkpoint", None):
        init_from_training_checkpoint(model, cfg.init_from_checkpoint)


def update_perception_output_dim(model) -> None:
    """The modality adapter must end in the LLM's hidden size."""
    with open_dict(model.cfg):
        model.cfg.perception.output_dim = int(model.llm.config.hidden_size)


def move_embedding(model) -> None:
    """The token embedding moves from the LLM to the wrapper: the LLM is then called with embeddings only (audio and text mixed),
    and parameter-efficient tuning of the LLM leaves the table alone."""
    if getattr(model.llm.model, "embed_tokens", None) is not None:
        model.embed_tokens = model.llm.model.embed_tokens
        model.llm.model.embed_tokens = None

"""Serving a speech-LLM (SALM) through an external LLM engine: the pieces the engine plug-in needs.

An LLM serving engine schedules by token count, so before the encoder ever runs it must know how many placeholder positions
an audio of N samples will occupy; it loads weights by Hugging Face names; and it asks the model for "multimodal embeddings"
that it splices into the token embeddings itself.  This module provides exactly those pieces, engine-independent and testable
on a CPU, plus ``register()`` which hands them to vLLM when that package is importable:

* ``AudioTokenEstimator`` — integer arithmetic for the perception module's output length (STFT framing, then the strided
  convolution stack), the chunked variant for long audio (fixed-size chunks, a short tail folded into the previous chunk) and
  the inverse (smallest sample count that yields a given number of tokens, by bisection) used to size the engine's encoder cache.
* ``merge_lora_into_base`` — folds ``lora_A`` / ``lora_B`` pairs into their base weights (``W + scale · B A``).
* ``export_for_serving`` — writes ``config.json`` + ``model.safetensors``-style state (``torch.save`` when safetensors is
  missing) with the LLM under ``llm.`` in Hugging Face naming, the perception module under ``perception.`` and the external
  embedding table restored into the LLM.
* ``SpeechLMServingModel`` — engine-facing wrapper: ``get_multimodal_embeddings(audio, lengths)`` and
  ``get_input_embeddings(input_ids, multimodal_embeddings)``.
* ``register()`` — registers the architecture name with vLLM's model registry (lazy import; raises with guidance when vLLM
  is not installed).  The registered class path points at ``build_vllm_model_class``, which derives the engine-side class
  from vLLM's multimodal interfaces at call time, so importing this module never imports vLLM.

Reference: ``speechlm2/vllm/salm/__init__.py:29-49`` (registration), ``audio.py:218-308`` (token estimators, tail folding),
``backends.py:82-147`` (LoRA merge, name mapping), ``model.py`` (embedding splice).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

ARCHITECTURE = "SpeechB200SALMForConditionalGeneration"
MODEL_TYPE = "speech_b200_salm"


@dataclass
class AudioTokenEstimator:
    sample_rate: int = 16000
    n_fft: int = 512
    hop_length: int = 160
    conv_kernel: int = 3
    conv_stride: int = 2
    conv_repeat: int = 3
    conv_padding: int = 2                      # total padding of one convolution (left + right)
    min_chunk_seconds: float = 0.5             # a tail shorter than this joins the previous chunk
    max_seconds: float = 3600.0

    def single_pass(self, n_samples: int) -> int:
        frames = (int(n_samples) + 2 * (self.n_fft // 2) - self.n_fft) // self.hop_length
        length = float(frames)
        for _ in range(self.conv_repeat):
            length = float(int((length + self.conv_padding - self.conv_kernel) / self.conv_stride + 1.0))
        return max(1, int(length))

    def spans(self, n_samples: int, chunk_seconds: Optional[float]) -> List[Tuple[int, int]]:
        if chunk_seconds is None or n_samples <= 0:
            return [(0, max(0, int(n_samples)))]
        if chunk_seconds <= 0:
            raise ValueError("encoder chunk size must be positive when set")
        min_chunk = int(self.min_chunk_seconds * self.sample_rate)
        chunk = max(int(round(chunk_seconds * self.sample_rate)), min_chunk, 1)
        out = [(b, min(b + chunk, n_samples)) for b in range(0, n_samples, chunk)]
        if len(out) > 1 and out[-1][1] - out[-1][0] < min_chunk:
            out[-2] = (out[-2][0], out[-1][1])
            out.pop()
        return out

    def tokens(self, n_samples: int, chunk_seconds: Optional[float] = None) -> int:
        return sum(self.single_pass(e - b) for b, e in self.spans(n_samples, chunk_seconds))

    def samples_for_tokens(self, target_tokens: int, chunk_seconds: Optional[float] = None) -> int:
        target = max(1, int(target_tokens))
        cap = int(self.max_seconds * self.sample_rate)
        lo, hi = 1, min(self.sample_rate, cap)
        while hi < cap and self.tokens(hi, chunk_seconds) < target:
            hi = min(hi * 2, cap)
        if self.tokens(hi, chunk_seconds) < target:
            raise ValueError(f"cannot produce {target} audio tokens within {self.max_seconds:g} s")
        while lo < hi:
            mid = (lo + hi) // 2
            if self.tokens(mid, chunk_seconds) >= target:
                hi = mid
            else:
                lo = mid + 1
        return lo


def merge_lora_into_base(state: Dict[str, torch.Tensor], scale: float) -> Dict[str, torch.Tensor]:
    """``{name.base.weight | name.weight, name.lora_A, name.lora_B}`` -> ``{name.weight: W + scale · B A}``; other entries pass."""
    out: Dict[str, torch.Tensor] = {}
    lora: Dict[str, Dict[str, torch.Tensor]] = {}
    for k, v in state.items():
        for tag in ("lora_A", "lora_B"):
            for suffix in (f".{tag}", f".{tag}.weight", f".{tag}.default.weight"):
                if k.endswith(suffix):
                    lora.setdefault(k[: -len(suffix)], {})[tag] = v
                    break
            else:
                continue
            break
        else:
            out[k.replace(".base.weight", ".weight").replace(".base.bias", ".bias").replace(".base_layer.", ".")] = v
    for name, ab in lora.items():
        if "lora_A" not in ab or "lora_B" not in ab:
            raise KeyError(f"incomplete LoRA pair for {name}")
        w = out.get(name + ".weight")
        if w is None:
            raise KeyError(f"LoRA weights for {name} have no base weight")
        out[name + ".weight"] = (w.float() + scale * (ab["lora_B"].float() @ ab["lora_A"].float())).to(w.dtype)
    return out


@dataclass
class SpeechLMServingConfig:
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])
    model_type: str = MODEL_TYPE
    llm: Dict[str, Any] = field(default_factory=dict)
    perception: Dict[str, Any] = field(default_factory=dict)
    audio_locator_tag: str = "<|audioplaceholder|>"
    audio_locator_tag_id: int = -1
    encoder_chunk_size_seconds: Optional[float] = None
    estimator: Dict[str, Any] = field(default_factory=dict)


def export_for_serving(model, path: str, lora_scale: Optional[float] = None) -> SpeechLMServingConfig:
    """Write a serving directory for a SALM-style model (``llm``, ``embed_tokens`` kept outside it, ``perception``)."""
    from ..core.config import OmegaConf

    os.makedirs(path, exist_ok=True)
    llm_state = {k: v.detach().cpu() for k, v in model.llm.state_dict().items()}
    if lora_scale is not None:
        llm_state = merge_lora_into_base(llm_state, lora_scale)
    llm_state["model.embed_tokens.weight"] = model.embed_tokens.weight.detach().cpu()
    state = {"llm." + k: v for k, v in llm_state.items()}
    state.update({"perception." + k: v.detach().cpu() for k, v in model.perception.state_dict().items()})
    pcfg = getattr(model.perception, "cfg", None) or getattr(model.cfg, "perception", {})
    cfg = SpeechLMServingConfig(llm=asdict(model.llm.config) if hasattr(model.llm.config, "__dataclass_fields__") else dict(model.llm.config),
                                perception=OmegaConf.to_container(pcfg, resolve=True) if not isinstance(pcfg, dict) else pcfg,
                                audio_locator_tag=model.audio_locator_tag, audio_locator_tag_id=int(model.audio_locator_tag_id),
                                encoder_chunk_size_seconds=getattr(model, "encoder_chunk_size_seconds", None))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(asdict(cfg), f, indent=1, default=str)
    try:
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in state.items()}, os.path.join(path, "model.safetensors"))
    except ImportError:
        torch.save(state, os.path.join(path, "pytorch_model.bin"))
    return cfg


def load_serving_state(path: str) -> Tuple[Dict[str, Any], Dict[str, torch.Tensor]]:
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    st = os.path.join(path, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file

        return cfg, load_file(st)
    return cfg, torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu")


class SpeechLMServingModel(nn.Module):
    """What the engine calls: audio -> embeddings, and the splice of those embeddings into the prompt's token embeddings."""

    def __init__(self, perception: nn.Module, embed_tokens: nn.Module, placeholder_id: int, estimator: Optional[AudioTokenEstimator] = None,
                 encoder_chunk_size_seconds: Optional[float] = None):
        super().__init__()
        self.perception, self.embed_tokens, self.placeholder_id = perception, embed_tokens, int(placeholder_id)
        self.estimator = estimator or AudioTokenEstimator()
        self.chunk_seconds = encoder_chunk_size_seconds

    @torch.no_grad()
    def get_multimodal_embeddings(self, audio: torch.Tensor, audio_lens: torch.Tensor) -> List[torch.Tensor]:
        """One tensor [tokens_i, hidden] per audio; long audio goes through the encoder chunk by chunk."""
        out = []
        for b in range(audio.shape[0]):
            n = int(audio_lens[b])
            parts = []
            for s, e in self.estimator.spans(n, self.chunk_seconds):
                emb, ln = self.perception(input_signal=audio[b:b + 1, s:e], input_signal_length=torch.tensor([e - s], device=audio.device))
                parts.append(emb[0, : int(ln[0])])
            out.append(torch.cat(parts, dim=0))
        return out

    def get_input_embeddings(self, input_ids: torch.Tensor, multimodal_embeddings: Optional[Sequence[torch.Tensor]] = None) -> torch.Tensor:
        """input_ids [T] (flattened batch, as engines pass it) with one placeholder id per audio token."""
        ids = input_ids.reshape(-1)
        is_audio = ids == self.placeholder_id
        emb = self.embed_tokens(torch.where(is_audio, torch.zeros_like(ids), ids))
        if multimodal_embeddings:
            flat = torch.cat(list(multimodal_embeddings), dim=0).to(emb.dtype)
            if int(is_audio.sum()) != flat.shape[0]:
                raise ValueError(f"{int(is_audio.sum())} placeholder positions but {flat.shape[0]} audio embeddings")
            emb = emb.clone()
            emb[is_audio] = flat
        return emb.view(*input_ids.shape, -1)

    def expand_placeholders(self, input_ids: List[int], audio_samples: Sequence[int]) -> List[int]:
        """Replace each single locator token by as many placeholders as its audio will produce (what the engine's prompt
        processor does before scheduling)."""
        out, k = [], 0
        for t in input_ids:
            if t == self.placeholder_id:
                if k >= len(audio_samples):
                    raise ValueError("more audio locator tokens than audios")
                out.extend([t] * self.estimator.tokens(int(audio_samples[k]), self.chunk_seconds))
                k += 1
            else:
                out.append(t)
        if k != len(audio_samples):
            raise ValueError("more audios than audio locator tokens")
        return out


def build_vllm_model_class():
    """Derive the engine-side class from vLLM's interfaces (called by vLLM through the registry's lazy import)."""
    from vllm.model_executor.models.interfaces import SupportsMultiModal  # noqa: F401  (raises ImportError without vLLM)
    from vllm.model_executor.models.utils import init_vllm_registered_model, maybe_prefix

    class SpeechB200SALMForConditionalGeneration(nn.Module, SupportsMultiModal):
        def __init__(self, *, vllm_config, prefix: str = ""):
            super().__init__()
            hf = vllm_config.model_config.hf_config
            from ..core.config import OmegaConf
            from .perception import AudioPerceptionModule

            self.config = hf
            self.language_model = init_vllm_registered_model(vllm_config=vllm_config, hf_config=getattr(hf, "text_config", hf),
                                                             prefix=maybe_prefix(prefix, "language_model"))
            self.perception = AudioPerceptionModule(OmegaConf.create(dict(hf.perception)))
            self.serving = SpeechLMServingModel(self.perception, self.language_model.get_input_embeddings, int(hf.audio_locator_tag_id),
                                                AudioTokenEstimator(**dict(getattr(hf, "estimator", {}) or {})),
                                                getattr(hf, "encoder_chunk_size_seconds", None))

        def get_multimodal_embeddings(self, **kwargs):
            audio, lens = kwargs.get("audio"), kwargs.get("audio_lens")
            return None if audio is None else self.serving.get_multimodal_embeddings(audio, lens)

        def get_input_embeddings(self, input_ids, multimodal_embeddings=None, **_):
            return self.serving.get_input_embeddings(input_ids, multimodal_embeddings)

        def forward(self, input_ids, positions, intermediate_tensors=None, inputs_embeds=None, **kwargs):
            return self.language_model.model(input_ids, positions, intermediate_tensors, inputs_embeds=inputs_embeds)

        def compute_logits(self, hidden_states, *a, **kw):
            return self.language_model.compute_logits(hidden_states, *a, **kw)

        def load_weights(self, weights):
            llm, perc = [], {}
            for name, w in weights:
                if name.startswith("llm."):
                    llm.append((name[4:], w))
                elif name.startswith("perception."):
                    perc[name[len("perception."):]] = w
            self.perception.load_state_dict(perc, strict=False)
            return self.language_model.load_weights(llm)

    return SpeechB200SALMForConditionalGeneration


def __getattr__(name):
    if name == ARCHITECTURE:
        return build_vllm_model_class()
    raise AttributeError(name)


def register(registry=None) -> None:
    """Register the architecture with vLLM (``vllm.general_plugins`` entry point target).  ``registry`` is injectable for tests."""
    if registry is None:
        try:
            from vllm.model_executor.models.registry import ModelRegistry as registry  # type: ignore
        except ImportError as e:
            raise ImportError("vLLM is not installed: install it to serve speech_b200 SALM models through vLLM, or use "
                              "`SpeechLMServingModel` with the built-in `CausalLM.generate`") from e
    registry.register_model(ARCHITECTURE, f"{__name__}:{ARCHITECTURE}")

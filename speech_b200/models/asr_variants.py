"""ASR model variants built on the CTC / transducer / AED base classes.

* ``EncDecRNNTBPEModelWithPrompt`` / ``EncDecHybridRNNTCTCBPEModelWithPrompt`` — a language-id (or task) prompt vector per
  utterance is projected and combined with the encoder output before the decoders
  (``models/rnnt_bpe_models_prompt.py``, ``hybrid_rnnt_ctc_bpe_models_prompt.py``).
* ``EncDecRNNTBPEEOUModel`` / ``EncDecHybridRNNTCTCBPEEOUModel`` — end-of-utterance training: the vocabulary carries
  ``<EOU>`` / ``<EOB>`` tokens and validation reports EOU latency / early / miss statistics (``models/asr_eou_models.py``).
* ``EncDecMultiTalkerRNNTBPEModel`` — speaker-kernel injection: per-layer learned "speaker kernels" add a projection of
  the frames where the target speaker (from diarization activity) is active (``models/multitalker_asr_models.py``).
* ``EncDecTransfModelBPE`` — the older encoder + Transformer decoder speech-translation model
  (``models/transformer_bpe_models.py``).
* ``ConfidenceEnsembleModel`` — runs several models and keeps, per utterance, the output of the most confident one
  (``models/confidence_ensemble.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn as nn

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.modelpt import ModelPT
from .aed_models import EncDecMultiTaskModel
from .hybrid_models import EncDecHybridRNNTCTCBPEModel
from .rnnt_models import EncDecRNNTBPEModel


# ---------------------------------------------------------------------------------------------- prompt models
class _PromptMixin:
    """Adds ``prompt_kernel``: ``enc' = Linear([enc ; onehot(prompt)])`` applied to every encoder frame."""

    def _init_prompt(self, cfg):
        self.num_prompts = int(cfg_get(cfg, "num_prompts", cfg_get(cfg.get("model_defaults", {}), "num_prompts", 128)))
        d = self.encoder._feat_out
        self.prompt_kernel = nn.Sequential(nn.Linear(d + self.num_prompts, d * 2), nn.ReLU(), nn.Linear(d * 2, d))
        self._current_prompt: Optional[torch.Tensor] = None

    def set_prompt(self, prompt_ids: Optional[torch.Tensor]):
        """``prompt_ids`` [B] (class index) or [B, num_prompts] (soft vector) used by the next forward calls."""
        self._current_prompt = prompt_ids

    def _apply_prompt(self, encoded: torch.Tensor, prompt) -> torch.Tensor:
        if prompt is None:
            return encoded
        x = encoded.transpose(1, 2)
        if prompt.dim() == 1:
            prompt = torch.nn.functional.one_hot(prompt.long(), self.num_prompts)
        p = prompt.to(x.dtype).unsqueeze(1).expand(-1, x.shape[1], -1)
        h = torch.cat([x, p], dim=-1)
        l0, l2 = self.prompt_kernel[0], self.prompt_kernel[2]
        h = ops.linear(h, l0.weight, l0.bias, act="relu")
        h = ops.linear(h, l2.weight, l2.bias)
        return h.transpose(1, 2).to(encoded.dtype)

    def forward(self, input_signal=None, input_signal_length=None, processed_signal=None, processed_signal_length=None,
                prompt=None):
        encoded, encoded_len = super().forward(input_signal=input_signal, input_signal_length=input_signal_length,
                                               processed_signal=processed_signal, processed_signal_length=processed_signal_length)
        prompt = prompt if prompt is not None else self._current_prompt
        return self._apply_prompt(encoded, prompt), encoded_len

    def training_step(self, batch, batch_idx):
        self.set_prompt(batch[4] if len(batch) > 4 else None)
        try:
            return super().training_step(batch[:4], batch_idx)
        finally:
            self.set_prompt(None)

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        self.set_prompt(batch[4] if len(batch) > 4 else None)
        try:
            return super().validation_pass(batch[:4], batch_idx, dataloader_idx)
        finally:
            self.set_prompt(None)


class EncDecRNNTBPEModelWithPrompt(_PromptMixin, EncDecRNNTBPEModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self._init_prompt(self._cfg)


class EncDecHybridRNNTCTCBPEModelWithPrompt(_PromptMixin, EncDecHybridRNNTCTCBPEModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self._init_prompt(self._cfg)


# ---------------------------------------------------------------------------------------------- end of utterance
EOU_STRING, EOB_STRING = "<EOU>", "<EOB>"


@dataclass
class EOUResult:
    latency: List[float]
    early_cutoff: List[float]
    true_positives: int = 0
    false_negatives: int = 0
    false_positives: int = 0
    num_utterances: int = 0
    num_predictions: int = 0
    missing: int = 0


def evaluate_eou(prediction: Sequence[Dict[str, float]], reference: Sequence[Dict[str, float]], threshold: float = 0.5,
                 collar: float = 0.0, do_sorting: bool = True) -> EOUResult:
    """Match predicted EOU events (``{"start_time","end_time","eou_prob","eou_pred"}``) to reference utterance ends.
    A prediction inside ``[ref_end - collar, next_start)`` is a hit with latency ``pred_end - ref_end``; before the window it
    is an early cut-off (``parts/utils/eou_utils.py``)."""
    preds = [p for p in prediction if p.get("eou_pred", p.get("eou_prob", 0.0) >= threshold)]
    refs = list(reference)
    if do_sorting:
        preds.sort(key=lambda p: p["end_time"])
        refs.sort(key=lambda r: r["end_time"])
    res = EOUResult([], [], num_utterances=len(refs), num_predictions=len(preds))
    used = set()
    for i, r in enumerate(refs):
        nxt = refs[i + 1]["start_time"] if i + 1 < len(refs) else float("inf")
        hit = None
        for j, p in enumerate(preds):
            if j in used:
                continue
            if r["start_time"] < p["end_time"] < r["end_time"] - collar:
                res.early_cutoff.append(r["end_time"] - p["end_time"])
                used.add(j)
                res.false_positives += 1
                continue
            if r["end_time"] - collar <= p["end_time"] < max(nxt, r["end_time"] + 1e-9):
                hit = j
                break
        if hit is None:
            res.false_negatives += 1
            res.missing += 1
        else:
            used.add(hit)
            res.true_positives += 1
            res.latency.append(max(0.0, preds[hit]["end_time"] - r["end_time"]))
    res.false_positives += len([j for j in range(len(preds)) if j not in used])
    return res


class _EOUMixin:
    def _init_eou(self):
        tok = self.tokenizer
        self.eou_token = tok.token_to_id(EOU_STRING) if hasattr(tok, "token_to_id") else -1
        self.eob_token = tok.token_to_id(EOB_STRING) if hasattr(tok, "token_to_id") else -1
        self.frame_seconds = None

    def _frame_seconds(self) -> float:
        feat = getattr(self.preprocessor, "featurizer", self.preprocessor)
        return feat.hop_length / feat.sample_rate * self.encoder.subsampling_factor

    def eou_predictions_from_hypothesis(self, hyp) -> List[Dict[str, float]]:
        ys = hyp.y_sequence.tolist() if torch.is_tensor(hyp.y_sequence) else list(hyp.y_sequence)
        ts = hyp.timestamp.tolist() if torch.is_tensor(hyp.timestamp) else list(hyp.timestamp)
        fs = self._frame_seconds()
        return [{"start_time": t * fs, "end_time": (t + 1) * fs, "eou_prob": 1.0, "eou_pred": True}
                for y, t in zip(ys, ts) if y in (self.eou_token, self.eob_token)]

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        out = super().validation_pass(batch[:4], batch_idx, dataloader_idx)
        signal, signal_len = batch[0], batch[1]
        encoded, encoded_len = self.forward(input_signal=signal, input_signal_length=signal_len)
        hyps = self.decoding.rnnt_decoder_predictions_tensor(encoded, encoded_len, return_hypotheses=True)
        lat, early, miss = [], [], 0
        for b, h in enumerate(hyps):
            dur = float(signal_len[b]) / cfg_get(self._cfg, "sample_rate", 16000)
            r = evaluate_eou(self.eou_predictions_from_hypothesis(h), [{"start_time": 0.0, "end_time": dur}], collar=0.2)
            lat += r.latency
            early += r.early_cutoff
            miss += r.missing
        out.update({"val_eou_latency": torch.tensor(float(np.mean(lat)) if lat else 0.0),
                    "val_eou_early_cutoff": torch.tensor(float(len(early))), "val_eou_missing": torch.tensor(float(miss))})
        return out


class EncDecRNNTBPEEOUModel(_EOUMixin, EncDecRNNTBPEModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self._init_eou()


class EncDecHybridRNNTCTCBPEEOUModel(_EOUMixin, EncDecHybridRNNTCTCBPEModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        self._init_eou()


# ---------------------------------------------------------------------------------------------- multitalker
class SpeakerKernel(nn.Module):
    """``x + mask * FF(x)``: a feed-forward branch that only sees (and only changes) the frames of one speaker."""

    def __init__(self, d_model: int, dropout: float = 0.1):
        super().__init__()
        self.ff = nn.Sequential(nn.Linear(d_model, d_model), nn.ReLU(), nn.Dropout(dropout), nn.Linear(d_model, d_model))

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        m = mask.unsqueeze(-1).to(x.dtype)
        return x + m * self.ff(x * m)


class EncDecMultiTalkerRNNTBPEModel(EncDecRNNTBPEModel):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        layers = list(cfg_get(cfg, "spk_kernel_layers", [0]))
        d = self.encoder.d_model
        self.spk_kernel_type = cfg_get(cfg, "spk_kernel_type", "ff")
        self.add_bg_spk_kernel = cfg_get(cfg, "add_bg_spk_kernel", True)
        self.spk_kernels = nn.ModuleDict({str(i): SpeakerKernel(d) for i in layers})
        self.bg_spk_kernels = nn.ModuleDict({str(i): SpeakerKernel(d) for i in layers}) if self.add_bg_spk_kernel else None
        self._spk_targets: Optional[torch.Tensor] = None
        self._bg_targets: Optional[torch.Tensor] = None
        self._spk_hook_handles = []
        for i in layers:
            self._spk_hook_handles.append(self.encoder.layers[i].register_forward_pre_hook(self._make_hook(str(i)), with_kwargs=True))

    def set_speaker_targets(self, spk_targets: Optional[torch.Tensor], bg_spk_targets: Optional[torch.Tensor] = None):
        """``spk_targets`` [B, T'] activity (0..1) of the speaker to transcribe; ``bg_spk_targets`` everyone else."""
        self._spk_targets, self._bg_targets = spk_targets, bg_spk_targets

    def _make_hook(self, key: str):
        def hook(module, args, kwargs):
            if self._spk_targets is None:
                return None
            x = kwargs.get("x", args[0] if args else None)
            T = x.shape[1]
            def fit(m):
                m = m.to(x.device)
                return m[:, :T] if m.shape[1] >= T else torch.nn.functional.pad(m, (0, T - m.shape[1]))
            x = self.spk_kernels[key](x, fit(self._spk_targets))
            if self.bg_spk_kernels is not None and self._bg_targets is not None:
                x = self.bg_spk_kernels[key](x, fit(self._bg_targets))
            if "x" in kwargs:
                kwargs = dict(kwargs, x=x)
                return args, kwargs
            return (x,) + tuple(args[1:]), kwargs
        return hook

    def training_step(self, batch, batch_idx):
        if len(batch) > 4:
            self.set_speaker_targets(batch[4], batch[5] if len(batch) > 5 else None)
        try:
            return super().training_step(batch[:4], batch_idx)
        finally:
            self.set_speaker_targets(None)

    def validation_pass(self, batch, batch_idx, dataloader_idx=0):
        if len(batch) > 4:
            self.set_speaker_targets(batch[4], batch[5] if len(batch) > 5 else None)
        try:
            return super().validation_pass(batch[:4], batch_idx, dataloader_idx)
        finally:
            self.set_speaker_targets(None)

    @torch.no_grad()
    def transcribe_with_speaker_targets(self, audio: torch.Tensor, lens: torch.Tensor, spk_targets: torch.Tensor,
                                        bg_spk_targets: Optional[torch.Tensor] = None):
        """Hypotheses of the speaker whose activity is ``spk_targets`` [B, T'] (``multitalker_asr_models.py`` ``_transcribe_forward``)."""
        self.set_speaker_targets(spk_targets, bg_spk_targets)
        try:
            return self._transcribe_forward_and_decode(audio, lens, None)
        finally:
            self.set_speaker_targets(None)


# ---------------------------------------------------------------------------------------------- confidence ensemble
def entropy_confidence(log_probs: torch.Tensor, alpha: float = 0.33, kind: str = "tsallis") -> torch.Tensor:
    """Per-frame confidence in [0, 1] from a distribution (``parts/utils/asr_confidence_utils.py``): normalised
    exponential of the Gibbs (alpha = 1), Tsallis or Renyi entropy."""
    p = log_probs.float().exp()
    V = log_probs.shape[-1]
    if kind == "max_prob":
        return (p.max(-1).values * V - 1) / (V - 1)
    if kind == "gibbs" or abs(alpha - 1.0) < 1e-6:
        ent = -(p * log_probs.float()).sum(-1)
        return 1 - ent / np.log(V)
    s = p.pow(alpha).sum(-1)
    if kind == "renyi":
        ent = torch.log2(s) / (1 - alpha)
        return 1 - ent / np.log2(V)
    ent = (s - 1) / (1 - alpha)                      # Tsallis entropy (1 - sum p^alpha) / (alpha - 1)
    return 1 - ent / ((V ** (1 - alpha) - 1) / (1 - alpha))


class ConfidenceEnsembleModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None, models: Optional[Sequence[ModelPT]] = None):
        super().__init__(cfg=cfg, trainer=trainer)
        self.num_models = len(models) if models is not None else len(cfg_get(self._cfg, "load_models", []))
        mods = list(models) if models is not None else [ModelPT.restore_from(p) for p in self._cfg.load_models]
        for i, m in enumerate(mods):
            self.add_module(f"model{i}", m)
        self.alpha = cfg_get(self._cfg, "confidence_alpha", 0.33)
        self.kind = cfg_get(self._cfg, "confidence_kind", "tsallis")
        self.model_selection_block = None       # optional sklearn pipeline (``predict_proba``) on the confidence features

    def list_models(self):
        return [getattr(self, f"model{i}") for i in range(self.num_models)]

    @torch.no_grad()
    def _confidence(self, model, audio, lens) -> torch.Tensor:
        out = model.forward(input_signal=audio, input_signal_length=lens)
        if len(out) == 3:                         # CTC: log_probs, lengths, greedy
            lp, ln = out[0], out[1]
        else:                                     # transducer: use the auxiliary CTC head when there is one
            enc, ln = out
            head = getattr(model, "ctc_decoder", None)
            if head is None:
                return torch.ones(audio.shape[0])
            lp = head(encoder_output=enc)
        conf = entropy_confidence(lp, self.alpha, self.kind)
        mask = torch.arange(conf.shape[1], device=conf.device)[None] < ln[:, None]
        return ((conf * mask).sum(1) / ln.clamp(min=1)).cpu()

    @torch.no_grad()
    def transcribe(self, audio: Sequence[Any], batch_size: int = 4, return_hypotheses: bool = False, **kw):
        outs = [m.transcribe(audio, batch_size=batch_size, return_hypotheses=True, **kw) for m in self.list_models()]
        from ..data.audio_to_text import load_audio

        confs = []
        for m in self.list_models():
            c = []
            for a in audio:
                x = torch.as_tensor(load_audio(a) if isinstance(a, str) else a, dtype=torch.float32).reshape(1, -1).to(m.device)
                c.append(float(self._confidence(m, x, torch.tensor([x.shape[1]], device=m.device))[0]))
            confs.append(c)
        confs_t = torch.tensor(confs)                           # [models, utterances]
        if self.model_selection_block is not None:
            pick = torch.as_tensor(self.model_selection_block.predict(confs_t.T.numpy()))
        else:
            pick = confs_t.argmax(dim=0)
        best = [outs[int(pick[i])][i] for i in range(len(audio))]
        return best if return_hypotheses else [h.text for h in best]

    def setup_training_data(self, c): ...
    def setup_validation_data(self, c): ...


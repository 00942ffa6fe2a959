"""Sortformer end-to-end speaker diarization: FastConformer encoder → projection → Transformer encoder → per-frame
speaker sigmoids, trained with arrival-time-sorted (ATS) and permutation-invariant (PIL) binary cross entropy; offline and
streaming (speaker cache + FIFO) inference.

Reference: ``models/sortformer_diar_models.py``, ``modules/sortformer_modules.py`` and
``parts/utils/asr_multispeaker_utils.py`` (target construction), ``parts/utils/vad_utils.py`` (post-processing).
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

from .. import ops
from ..core.config import DictConfig, cfg_get, open_dict
from ..core.instantiate import from_config_dict
from ..core.modelpt import ModelPT
from ..core.module import NeuralModule
from ..losses.misc import BCELoss
from ..modules.transformer import TransformerEncoder


class SortformerModules(NeuralModule):
    def __init__(self, num_spks: int = 4, dropout_rate: float = 0.5, fc_d_model: int = 512, tf_d_model: int = 192,
                 subsampling_factor: int = 8, spkcache_len: int = 188, fifo_len: int = 0, chunk_len: int = 376,
                 spkcache_update_period: int = 376, chunk_left_context: int = 1, chunk_right_context: int = 1,
                 spkcache_sil_frames_per_spk: int = 3, causal_attn_rate: float = 0.0, causal_attn_rc: int = 7,
                 scores_add_rnd: float = 0.0, pred_score_threshold: float = 0.25, max_index: int = 99999,
                 scores_boost_latest: float = 0.05, sil_threshold: float = 0.2, strong_boost_rate: float = 0.75,
                 weak_boost_rate: float = 1.5, min_pos_scores_rate: float = 0.5):
        super().__init__()
        self.n_spk, self.fc_d_model, self.tf_d_model = num_spks, fc_d_model, tf_d_model
        self.subsampling_factor = subsampling_factor
        self.encoder_proj = nn.Linear(fc_d_model, tf_d_model)
        self.first_hidden_to_hidden = nn.Linear(tf_d_model, tf_d_model)
        self.single_hidden_to_spks = nn.Linear(tf_d_model, num_spks)
        self.hidden_to_spks = nn.Linear(2 * tf_d_model, num_spks)
        self.dropout = nn.Dropout(dropout_rate)
        self.spkcache_len, self.fifo_len, self.chunk_len = spkcache_len, fifo_len, chunk_len
        self.chunk_left_context, self.chunk_right_context = chunk_left_context, chunk_right_context
        self.spkcache_update_period = spkcache_update_period
        self.spkcache_sil_frames_per_spk = spkcache_sil_frames_per_spk
        self.pred_score_threshold, self.sil_threshold = pred_score_threshold, sil_threshold
        self.scores_boost_latest = scores_boost_latest

    @staticmethod
    def length_to_mask(lengths: torch.Tensor, max_length: int) -> torch.Tensor:
        return torch.arange(max_length, device=lengths.device)[None, :] < lengths[:, None]

    def forward_speaker_sigmoids(self, hidden_out: torch.Tensor) -> torch.Tensor:
        h = self.dropout(torch.relu(hidden_out))
        h = self.dropout(torch.relu(ops.linear(h, self.first_hidden_to_hidden.weight, self.first_hidden_to_hidden.bias)))
        return torch.sigmoid(ops.linear(h, self.single_hidden_to_spks.weight, self.single_hidden_to_spks.bias).float())

    # ------------------------------------------------------------------ streaming state
    @dataclass
    class StreamingState:
        spkcache: Optional[torch.Tensor] = None          # [B, n, D] embeddings kept as long-term speaker memory
        spkcache_preds: Optional[torch.Tensor] = None    # [B, n, S]
        fifo: Optional[torch.Tensor] = None              # [B, m, D] most recent frames not yet folded into the cache
        fifo_preds: Optional[torch.Tensor] = None

    def init_streaming_state(self, batch_size: int, device) -> "SortformerModules.StreamingState":
        z = lambda n, d: torch.zeros((batch_size, n, d), device=device)  # noqa: E731
        return self.StreamingState(z(0, self.fc_d_model), z(0, self.n_spk), z(0, self.fc_d_model), z(0, self.n_spk))

    def compress_spkcache(self, emb: torch.Tensor, preds: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Keep ``spkcache_len`` frames: for every speaker the frames where it is most confidently the only one talking,
        plus a few silence frames, in time order (``sortformer_modules.py`` ``_compress_spkcache``)."""
        B, N, D = emb.shape
        if N <= self.spkcache_len:
            return emb, preds
        per_spk = (self.spkcache_len - self.spkcache_sil_frames_per_spk * self.n_spk) // self.n_spk
        p = preds.clamp(1e-6, 1 - 1e-6)
        # log-score of "speaker s alone": log p_s + sum_{r != s} log (1 - p_r)
        log1m = torch.log1p(-p)
        scores = torch.log(p) - log1m + log1m.sum(dim=-1, keepdim=True)
        scores = scores + self.scores_boost_latest * torch.linspace(0, 1, N, device=emb.device).view(1, N, 1)
        scores = torch.where(preds > self.pred_score_threshold, scores, torch.full_like(scores, float("-inf")))
        keep = torch.zeros((B, N), dtype=torch.bool, device=emb.device)
        for s in range(self.n_spk):
            k = min(per_spk, N)
            top = scores[..., s].topk(k, dim=1).indices
            valid = torch.gather(scores[..., s], 1, top) > float("-inf")
            keep.scatter_(1, top, valid)
        sil = (preds.sum(-1) < self.sil_threshold)
        need = self.spkcache_len - keep.sum(1)
        out_e, out_p = [], []
        for b in range(B):
            idx = keep[b].nonzero().squeeze(-1)
            extra_pool = (~keep[b]).nonzero().squeeze(-1)
            sil_first = extra_pool[sil[b][extra_pool]]
            rest = extra_pool[~sil[b][extra_pool]]
            extra = torch.cat([sil_first, rest.flip(0)])[: int(need[b])]
            sel = torch.cat([idx, extra]).sort().values[: self.spkcache_len]
            out_e.append(emb[b, sel])
            out_p.append(preds[b, sel])
        return torch.stack(out_e), torch.stack(out_p)

    def streaming_update(self, state, chunk_emb: torch.Tensor, chunk_preds: torch.Tensor):
        """Append the chunk to the FIFO; overflow moves into the speaker cache, which is then compressed."""
        state.fifo = torch.cat([state.fifo, chunk_emb], dim=1)
        state.fifo_preds = torch.cat([state.fifo_preds, chunk_preds], dim=1)
        over = state.fifo.shape[1] - self.fifo_len
        if over > 0:
            state.spkcache = torch.cat([state.spkcache, state.fifo[:, :over]], dim=1)
            state.spkcache_preds = torch.cat([state.spkcache_preds, state.fifo_preds[:, :over]], dim=1)
            state.fifo, state.fifo_preds = state.fifo[:, over:], state.fifo_preds[:, over:]
            state.spkcache, state.spkcache_preds = self.compress_spkcache(state.spkcache, state.spkcache_preds)
        return state


# ---------------------------------------------------------------------------------------------- targets
def get_ats_targets(labels: torch.Tensor, preds: torch.Tensor, speaker_permutations: torch.Tensor) -> torch.Tensor:
    """Arrival-time sort: order the target speakers by the frame of their first activity (silent speakers last)."""
    B, T, S = labels.shape
    first = torch.where(labels > 0.5, torch.arange(T, device=labels.device).view(1, T, 1).expand(B, T, S),
                        torch.full((B, T, S), T + 1, device=labels.device)).min(dim=1).values
    order = first.argsort(dim=1, stable=True)
    return torch.gather(labels, 2, order.unsqueeze(1).expand(B, T, S))


def get_pil_targets(labels: torch.Tensor, preds: torch.Tensor, speaker_permutations: torch.Tensor) -> torch.Tensor:
    """Permutation-invariant: pick, per sample, the speaker permutation of the targets that best matches the predictions."""
    perms = speaker_permutations.to(labels.device)                                  # [P, S]
    cand = labels[:, :, perms]                                                       # [B, T, P, S]
    score = (cand * preds.unsqueeze(2) + (1 - cand) * (1 - preds.unsqueeze(2))).sum(dim=(1, 3))
    best = score.argmax(dim=1)
    return cand[torch.arange(labels.shape[0], device=labels.device), :, best]


def find_segments(probs: np.ndarray, frame_sec: float, onset: float = 0.5, offset: float = 0.5, pad_onset: float = 0.0,
                  pad_offset: float = 0.0, min_duration_on: float = 0.0, min_duration_off: float = 0.0) -> List[Tuple[float, float]]:
    """Hysteresis thresholding + padding + short gap / short segment removal (``vad_utils.binarization`` + ``filtering``)."""
    segs, on, start = [], False, 0.0
    for t, p in enumerate(probs):
        if not on and p >= onset:
            on, start = True, t * frame_sec
        elif on and p < offset:
            on = False
            segs.append((max(0.0, start - pad_onset), t * frame_sec + pad_offset))
    if on:
        segs.append((max(0.0, start - pad_onset), len(probs) * frame_sec + pad_offset))
    merged: List[Tuple[float, float]] = []
    for s, e in segs:
        if merged and s - merged[-1][1] <= min_duration_off:
            merged[-1] = (merged[-1][0], max(e, merged[-1][1]))
        else:
            merged.append((s, e))
    return [(s, e) for s, e in merged if e - s >= min_duration_on]


class SortformerEncLabelModel(ModelPT):
    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.preprocessor = from_config_dict(cfg.preprocessor)
        self.spec_augmentation = from_config_dict(cfg.spec_augment) if cfg.get("spec_augment") is not None else None
        self.encoder = from_config_dict(cfg.encoder)
        self.sortformer_modules = from_config_dict(cfg.sortformer_modules)
        self.transformer_encoder = from_config_dict(cfg.transformer_encoder)
        self.loss = BCELoss(**(dict(cfg.loss) if cfg.get("loss") is not None and "_target_" not in cfg.loss else {}))
        self.max_num_of_spks = cfg.get("max_num_of_spks", 4)
        self.ats_weight = cfg.get("ats_weight", 0.5)
        self.pil_weight = cfg.get("pil_weight", 0.5)
        self.streaming_mode = cfg.get("streaming_mode", False)
        perms = list(itertools.permutations(range(self.max_num_of_spks)))
        self.register_buffer("speaker_permutations", torch.tensor(perms, dtype=torch.long), persistent=False)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if not hasattr(self, "transformer_encoder"):
            return
        super()._setup_dataloaders_from_cfg()

    # ------------------------------------------------------------------ data: (audio, audio_len, targets [B, T', S], target_len)
    def _loader(self, config):
        if config is None:
            return None
        from ..data.diarization import build_diarization_dataset
        from ..data.audio_to_text import get_dataloader_from_config

        ds = build_diarization_dataset(config, num_spks=self.max_num_of_spks,
                                       frame_sec=self.frame_seconds())
        rank = self.global_rank if self._trainer is not None else int(os.environ.get("RANK", 0))
        ws = self.world_size if self._trainer is not None else int(os.environ.get("WORLD_SIZE", 1))
        return get_dataloader_from_config(config, ds, rank, ws)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def setup_test_data(self, c):
        self._test_dl = self._loader(c)

    def frame_seconds(self) -> float:
        feat = getattr(self.preprocessor, "featurizer", self.preprocessor)
        return feat.hop_length / feat.sample_rate * self.encoder.subsampling_factor

    # ------------------------------------------------------------------ forward
    def frontend_encoder(self, processed_signal, processed_signal_length):
        emb, emb_len = self.encoder(audio_signal=processed_signal, length=processed_signal_length)[:2]
        return emb.transpose(1, 2), emb_len                     # [B, T', D]

    def forward_infer(self, emb_seq: torch.Tensor, emb_len: Optional[torch.Tensor] = None) -> torch.Tensor:
        sm = self.sortformer_modules
        x = ops.linear(emb_seq, sm.encoder_proj.weight, sm.encoder_proj.bias)
        mask = sm.length_to_mask(emb_len, x.shape[1]) if emb_len is not None else \
            torch.ones(x.shape[:2], dtype=torch.bool, device=x.device)
        h = self.transformer_encoder(encoder_states=x, encoder_mask=mask)
        preds = sm.forward_speaker_sigmoids(h)
        return preds * mask.unsqueeze(-1)

    def process_signal(self, audio_signal, audio_signal_length):
        feats, flen = self.preprocessor(input_signal=audio_signal, length=audio_signal_length)
        if self.spec_augmentation is not None and self.training:
            feats = self.spec_augmentation(input_spec=feats, length=flen)
        return feats, flen

    def forward(self, audio_signal, audio_signal_length):
        feats, flen = self.process_signal(audio_signal, audio_signal_length)
        if self.streaming_mode and not self.training:
            return self.forward_streaming(feats, flen)
        emb, emb_len = self.frontend_encoder(feats, flen)
        return self.forward_infer(emb, emb_len)

    @torch.no_grad()
    def forward_streaming(self, feats: torch.Tensor, flen: torch.Tensor) -> torch.Tensor:
        """Chunk-wise diarization with speaker cache + FIFO; output frames line up with the offline output."""
        sm = self.sortformer_modules
        sf = self.encoder.subsampling_factor
        B, _, T = feats.shape
        state = sm.init_streaming_state(B, feats.device)
        outs = []
        step = sm.chunk_len * sf
        lc, rc = sm.chunk_left_context * sf, sm.chunk_right_context * sf
        for s in range(0, T, step):
            lo, hi = max(0, s - lc), min(T, s + step + rc)
            chunk = feats[:, :, lo:hi]
            clen = (flen - lo).clamp(min=0, max=hi - lo)
            emb, emb_len = self.frontend_encoder(chunk, clen)
            drop_l = (s - lo) // sf
            n_new = min(sm.chunk_len, -(-(min(T, s + step) - s) // sf))
            emb_new = emb[:, drop_l:drop_l + n_new]
            ctx = torch.cat([state.spkcache, state.fifo, emb_new], dim=1)
            preds = self.forward_infer(ctx, None)
            n_ctx = state.spkcache.shape[1] + state.fifo.shape[1]
            new_preds = preds[:, n_ctx:]
            outs.append(new_preds)
            state = sm.streaming_update(state, emb_new, new_preds)
        out = torch.cat(outs, dim=1)
        valid = torch.div(flen + sf - 1, sf, rounding_mode="floor").clamp(max=out.shape[1])
        return out * sm.length_to_mask(valid, out.shape[1]).unsqueeze(-1)

    # ------------------------------------------------------------------ training
    def _loss(self, batch):
        audio, audio_len, targets, target_len = batch[:4]
        preds = self.forward(audio_signal=audio, audio_signal_length=audio_len)
        T = min(preds.shape[1], targets.shape[1])
        preds, targets = preds[:, :T], targets[:, :T].to(preds.dtype)
        target_len = target_len.clamp(max=T)
        ats = get_ats_targets(targets, preds, self.speaker_permutations)
        pil = get_pil_targets(targets, preds.detach(), self.speaker_permutations)
        l_ats = self.loss(probs=preds, labels=ats, target_lens=target_len)
        l_pil = self.loss(probs=preds, labels=pil, target_lens=target_len)
        loss = self.ats_weight * l_ats + self.pil_weight * l_pil
        with torch.no_grad():
            m = SortformerModules.length_to_mask(target_len, T).unsqueeze(-1)
            hard = (preds > 0.5).float()
            tp = (hard * pil * m).sum()
            f1 = 2 * tp / ((hard * m).sum() + (pil * m).sum()).clamp(min=1)
        return loss, {"ats_loss": l_ats.detach(), "pil_loss": l_pil.detach(), "f1_acc": f1}

    def training_step(self, batch, batch_idx):
        loss, logs = self._loss(batch)
        self.log_dict({"train_loss": loss.detach(), **{f"train_{k}": v for k, v in logs.items()}})
        return {"loss": loss}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        loss, logs = self._loss(batch)
        return {"val_loss": loss, **{f"val_{k}": v for k, v in logs.items()}}

    def multi_validation_epoch_end(self, outputs, dataloader_idx: int = 0):
        if not outputs:
            return {}
        keys = outputs[0].keys()
        avg = {k: torch.stack([torch.as_tensor(o[k]).float() for o in outputs]).mean() for k in keys}
        return {"val_loss": avg["val_loss"], "log": avg}

    # ------------------------------------------------------------------ inference API
    @torch.no_grad()
    def diarize(self, audio: Sequence, batch_size: int = 1, include_tensor_outputs: bool = False, postprocessing: Optional[dict] = None,
                sample_rate: int = 16000):
        """Returns, per recording, a list of ``"start end speaker_k"`` strings (and the probability tensors on request)."""
        from ..data.audio_to_text import load_audio

        self.eval()
        pp = dict(onset=0.5, offset=0.5, pad_onset=0.0, pad_offset=0.0, min_duration_on=0.0, min_duration_off=0.0)
        pp.update(postprocessing or {})
        fs = self.frame_seconds()
        results, tensors = [], []
        for s in range(0, len(audio), batch_size):
            xs = [torch.as_tensor(load_audio(a, target_sr=sample_rate) if isinstance(a, str) else a, dtype=torch.float32).reshape(-1)
                  for a in audio[s:s + batch_size]]
            lens = torch.tensor([x.numel() for x in xs], device=self.device)
            x = torch.nn.utils.rnn.pad_sequence(xs, batch_first=True).to(self.device)
            preds = self.forward(audio_signal=x, audio_signal_length=lens).float().cpu()
            for b in range(preds.shape[0]):
                n = int(np.ceil(int(lens[b]) / sample_rate / fs))
                p = preds[b, :n].numpy()
                segs = []
                for k in range(p.shape[1]):
                    segs += [(st, en, k) for st, en in find_segments(p[:, k], fs, **pp)]
                segs.sort()
                results.append([f"{st:.3f} {en:.3f} speaker_{k}" for st, en, k in segs])
                tensors.append(preds[b, :n])
        return (results, tensors) if include_tensor_outputs else results

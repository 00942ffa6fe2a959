"""CTC decoding: greedy (per-sample and batched) and prefix beam search, with timestamps.

Strategies follow ``nemo/collections/asr/parts/submodules/ctc_decoding.py`` (``greedy``, ``greedy_batch``,
``beam``); the batched greedy path collapses repeats and removes blanks fully on the device without a
per-utterance loop (reference: ``ctc_greedy_decoding.py:393``).
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ..core.config import DictConfig, OmegaConf, cfg_get
from .rnnt_decoding import Hypothesis, NBestHypotheses


@dataclass
class GreedyCTCInferConfig:
    preserve_alignments: bool = False
    compute_timestamps: bool = False
    preserve_frame_confidence: bool = False


@dataclass
class BeamCTCInferConfig:
    beam_size: int = 4
    search_type: str = "default"
    preserve_alignments: bool = False
    compute_timestamps: bool = False
    return_best_hypothesis: bool = True
    beam_alpha: float = 1.0
    beam_beta: float = 0.0
    kenlm_path: Optional[str] = None
    ngram_lm_model: Optional[str] = None
    ngram_lm_alpha: float = 0.0


@dataclass
class CTCDecodingConfig:
    strategy: str = "greedy_batch"
    preserve_alignments: Optional[bool] = None
    compute_timestamps: Optional[bool] = None
    word_seperator: str = " "
    segment_seperators: Optional[List[str]] = field(default_factory=lambda: [".", "!", "?"])
    segment_gap_threshold: Optional[int] = None
    ctc_timestamp_type: str = "all"
    batch_dim_index: int = 0
    greedy: GreedyCTCInferConfig = field(default_factory=GreedyCTCInferConfig)
    beam: BeamCTCInferConfig = field(default_factory=BeamCTCInferConfig)
    confidence_cfg: Optional[Dict[str, Any]] = None
    temperature: float = 1.0


@dataclass
class CTCBPEDecodingConfig(CTCDecodingConfig):
    pass


def greedy_batch_ctc(log_probs: torch.Tensor, lengths: torch.Tensor, blank: int):
    """log_probs [B,T,V+1] (or argmax ids [B,T]) -> padded token matrix, per-row counts, frame index per token, scores."""
    if log_probs.dim() == 3:
        scores, ids = log_probs.max(dim=-1)
    else:
        ids, scores = log_probs, torch.zeros_like(log_probs, dtype=torch.float32)
    B, T = ids.shape
    t = torch.arange(T, device=ids.device)[None, :]
    valid = t < lengths[:, None]
    prev = torch.cat([torch.full((B, 1), -1, device=ids.device, dtype=ids.dtype), ids[:, :-1]], dim=1)
    keep = valid & (ids != blank) & (ids != prev)
    counts = keep.sum(dim=1)
    pos = (keep.cumsum(dim=1) - 1).clamp(min=0)
    maxn = max(1, int(counts.max())) if B > 0 else 1
    out = torch.full((B, maxn + 1), blank, device=ids.device, dtype=torch.long)
    frames = torch.zeros((B, maxn + 1), device=ids.device, dtype=torch.long)
    dump = torch.full_like(pos, maxn)
    tgt = torch.where(keep, pos, dump)
    out.scatter_(1, tgt, torch.where(keep, ids, torch.full_like(ids, blank)))
    frames.scatter_(1, tgt, t.expand(B, T).contiguous())
    total = (scores * valid).sum(dim=1)
    return out[:, :maxn], counts, frames[:, :maxn], total


class AbstractCTCDecoding:
    def __init__(self, decoding_cfg, blank_id: int, supported_punctuation=None):
        if decoding_cfg is None:
            decoding_cfg = OmegaConf.structured(CTCDecodingConfig)
        elif not isinstance(decoding_cfg, DictConfig):
            decoding_cfg = OmegaConf.create(decoding_cfg)
        self.cfg = decoding_cfg
        self.blank_id = blank_id
        self.strategy = cfg_get(self.cfg, "strategy", "greedy_batch")
        if self.strategy not in ("greedy", "greedy_batch", "beam", "beam_batch", "pyctcdecode", "flashlight", "wfst"):
            raise ValueError(f"unknown CTC decoding strategy {self.strategy}")
        if self.strategy in ("pyctcdecode", "flashlight", "wfst"):
            raise NotImplementedError(f"CTC strategy '{self.strategy}' needs an external decoder that is not installed; "
                                      f"use 'beam' (built-in prefix beam search)")
        self.compute_timestamps = cfg_get(self.cfg, "compute_timestamps", None)
        self.preserve_alignments = cfg_get(self.cfg, "preserve_alignments", None)
        self.word_seperator = cfg_get(self.cfg, "word_seperator", " ")
        self.segment_seperators = list(cfg_get(self.cfg, "segment_seperators", [".", "?", "!"]) or [])
        self.segment_gap_threshold = cfg_get(self.cfg, "segment_gap_threshold", None)
        bm = cfg_get(self.cfg, "beam", None) or {}
        self.beam_size = cfg_get(bm, "beam_size", 4)
        self.return_best_hypothesis = cfg_get(bm, "return_best_hypothesis", True)

    def ctc_decoder_predictions_tensor(self, decoder_outputs: torch.Tensor, decoder_lengths: Optional[torch.Tensor] = None,
                                       fold_consecutive: bool = True, return_hypotheses: bool = False) -> List[Hypothesis]:
        if decoder_lengths is None:
            decoder_lengths = torch.full((decoder_outputs.shape[0],), decoder_outputs.shape[1],
                                         device=decoder_outputs.device, dtype=torch.long)
        if self.strategy == "beam_batch":
            from .batched_beam import BatchedBeamCTCComputer

            comp = BatchedBeamCTCComputer(self.blank_id, beam_size=self.beam_size,
                                          beam_beta=cfg_get(cfg_get(self.cfg, "beam", None) or {}, "beam_beta", 0.0),
                                          fusion_models=getattr(self, "fusion_models", None),
                                          fusion_models_alpha=getattr(self, "fusion_models_alpha", None))
            beams = comp(decoder_outputs, decoder_lengths.to(decoder_outputs.device))
            out = []
            for nbest in beams.to_hyps_list(score_norm=False):
                hs = [Hypothesis(score=s, y_sequence=torch.tensor(tok, dtype=torch.long),
                                 timestamp=torch.tensor(frm, dtype=torch.long)) for tok, frm, s in nbest]
                hs = hs or [Hypothesis(score=0.0, y_sequence=torch.zeros(0, dtype=torch.long))]
                out.append(self._finish(hs))
            return [h[0] for h in out] if self.return_best_hypothesis else [NBestHypotheses(h) for h in out]
        if self.strategy == "beam":
            hyps = [self._beam(decoder_outputs[b, : int(decoder_lengths[b])].float().cpu())
                    for b in range(decoder_outputs.shape[0])]
            if self.return_best_hypothesis:
                hyps = [h[0] for h in hyps]
            else:
                return [NBestHypotheses(self._finish(h)) for h in hyps]
            return self._finish(hyps)
        toks, counts, frames, total = greedy_batch_ctc(decoder_outputs, decoder_lengths.to(decoder_outputs.device), self.blank_id)
        toks, counts, frames, total = toks.cpu(), counts.cpu().tolist(), frames.cpu(), total.cpu().tolist()
        hyps = [Hypothesis(score=total[b], y_sequence=toks[b, : counts[b]], timestamp=frames[b, : counts[b]],
                           length=int(decoder_lengths[b])) for b in range(toks.shape[0])]
        return self._finish(hyps)

    __call__ = ctc_decoder_predictions_tensor

    def _finish(self, hyps: List[Hypothesis]) -> List[Hypothesis]:
        for h in hyps:
            ids = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
            h.text = self.decode_tokens_to_str(ids)
            if self.compute_timestamps:
                ts = h.timestamp.tolist() if torch.is_tensor(h.timestamp) else list(h.timestamp)
                toks = self.decode_ids_to_tokens(ids)
                chars = [{"char": [tk], "start_offset": t, "end_offset": t + 1} for tk, t in zip(toks, ts)]
                h.timestamp = {"timestep": ts, "char": chars, "word": self._words(chars)}
        return hyps

    def _words(self, chars):
        words, cur, start, end = [], "", None, None
        for c in chars:
            tok = c["char"][0]
            brk = tok.startswith("▁") or tok == self.word_seperator
            piece = tok.replace("▁", "") if tok != self.word_seperator else ""
            if brk and cur:
                words.append({"word": cur, "start_offset": start, "end_offset": end})
                cur = ""
            if piece:
                if not cur:
                    start = c["start_offset"]
                cur += piece
                end = c["end_offset"]
        if cur:
            words.append({"word": cur, "start_offset": start, "end_offset": end})
        return words

    def _beam(self, lp: torch.Tensor) -> List[Hypothesis]:
        """CTC prefix beam search over log-probs [T, V+1]."""
        NEG = -float("inf")

        def lse(*xs):
            m = max(xs)
            return m if m == NEG else m + math.log(sum(math.exp(x - m) for x in xs))

        beam = {(): (0.0, NEG)}  # prefix -> (log p_blank, log p_nonblank)
        T, V1 = lp.shape
        topk = min(V1, max(self.beam_size * 2, 8))
        for t in range(T):
            nxt: Dict[tuple, List[float]] = defaultdict(lambda: [NEG, NEG])
            vals, idxs = lp[t].topk(topk)
            for prefix, (pb, pnb) in beam.items():
                for v, k in zip(vals.tolist(), idxs.tolist()):
                    if k == self.blank_id:
                        e = nxt[prefix]
                        e[0] = lse(e[0], pb + v, pnb + v)
                        continue
                    last = prefix[-1] if prefix else None
                    np_ = prefix + (k,)
                    e = nxt[np_]
                    if k == last:
                        e[1] = lse(e[1], pb + v)
                        same = nxt[prefix]
                        same[1] = lse(same[1], pnb + v)
                    else:
                        e[1] = lse(e[1], pb + v, pnb + v)
            beam = dict(sorted(((p, (a, b)) for p, (a, b) in nxt.items()), key=lambda kv: lse(*kv[1]), reverse=True)[: self.beam_size])
        out = [Hypothesis(score=lse(a, b), y_sequence=torch.tensor(list(p), dtype=torch.long), timestamp=[], length=T)
               for p, (a, b) in beam.items()]
        return out

    def decode_tokens_to_str(self, tokens):
        raise NotImplementedError

    def decode_ids_to_tokens(self, tokens):
        raise NotImplementedError


class CTCDecoding(AbstractCTCDecoding):
    def __init__(self, decoding_cfg, vocabulary):
        self.labels_map = {i: vocabulary[i] for i in range(len(vocabulary))}
        super().__init__(decoding_cfg, blank_id=len(vocabulary))

    def decode_tokens_to_str(self, tokens):
        return "".join(self.labels_map[t] for t in tokens if t != self.blank_id)

    def decode_ids_to_tokens(self, tokens):
        return [self.labels_map[t] for t in tokens if t != self.blank_id]


class CTCBPEDecoding(AbstractCTCDecoding):
    def __init__(self, decoding_cfg, tokenizer):
        self.tokenizer = tokenizer
        super().__init__(decoding_cfg, blank_id=tokenizer.vocab_size)

    def decode_tokens_to_str(self, tokens):
        return self.tokenizer.ids_to_text([t for t in tokens if t != self.blank_id])

    def decode_ids_to_tokens(self, tokens):
        return self.tokenizer.ids_to_tokens([t for t in tokens if t != self.blank_id])

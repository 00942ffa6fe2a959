"""Transducer decoding front-end: strategies, hypotheses, timestamps, token -> text.

``RNNTDecoding`` / ``RNNTBPEDecoding`` dispatch on ``cfg.strategy`` (``greedy``, ``greedy_batch``, ``beam``,
``alsd``, ``maes``, ``tsd``, ``malsd_batch``, ``maes_batch``) like the reference
(``nemo/collections/asr/parts/submodules/rnnt_decoding.py:87,1256,1524``); defaults ``loop_labels=True`` and
``use_cuda_graph_decoder=True`` (``:456-457,477``).  Greedy strategies run the batched label-looping computer
(:mod:`speech_b200.decoding.label_looping`); beam strategies run the classic per-utterance searches
(reference: ``rnnt_beam_decoding.py:116``, ``tdt_beam_decoding.py:56``).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from .. import ops
from ..core.config import DictConfig, OmegaConf, cfg_get
from .label_looping import BatchedHyps, GreedyBatchedLabelLoopingComputer, LabelLoopingState


@dataclass
class Hypothesis:
    """One decoding hypothesis (reference: ``parts/utils/rnnt_utils.py:39+``)."""

    score: float
    y_sequence: Union[List[int], torch.Tensor]
    text: Optional[str] = None
    dec_out: Optional[List[torch.Tensor]] = None
    dec_state: Any = None
    timestamp: Union[List[int], torch.Tensor, dict] = field(default_factory=list)
    alignments: Any = None
    frame_confidence: Any = None
    token_confidence: Any = None
    word_confidence: Any = None
    length: Union[int, torch.Tensor] = 0
    y: Any = None
    lm_state: Any = None
    lm_scores: Any = None
    ngram_lm_state: Any = None
    tokens: Any = None
    last_token: Any = None
    token_duration: Any = None
    last_frame: Optional[int] = None

    @property
    def non_blank_frame_confidence(self):
        return []

    @property
    def words(self) -> List[str]:
        return [] if self.text is None else self.text.split()


@dataclass
class NBestHypotheses:
    n_best_hypotheses: Optional[List[Hypothesis]]


def batched_hyps_to_hypotheses(hyps: BatchedHyps, alignments=None, batch_size: Optional[int] = None) -> List[Hypothesis]:
    B = batch_size or hyps.scores.shape[0]
    lens = hyps.current_lengths.cpu().tolist()
    tr, ts = hyps.transcript.cpu(), hyps.timestamps.cpu()
    sc = hyps.scores.cpu().tolist()
    du = hyps.token_durations.cpu() if hyps.token_durations is not None else None
    out = []
    for i in range(B):
        out.append(Hypothesis(score=sc[i], y_sequence=tr[i, : lens[i]], timestamp=ts[i, : lens[i]],
                              token_duration=du[i, : lens[i]] if du is not None else None, alignments=None,
                              dec_state=None))
    return out


@dataclass
class GreedyBatchedRNNTInferConfig:
    max_symbols_per_step: Optional[int] = 10
    preserve_alignments: bool = False
    preserve_frame_confidence: bool = False
    loop_labels: bool = True
    use_cuda_graph_decoder: bool = True
    tdt_include_token_duration: bool = False
    ngram_lm_model: Optional[str] = None
    ngram_lm_alpha: float = 0.0
    boosting_tree: Any = None
    boosting_tree_alpha: float = 0.0


@dataclass
class BeamRNNTInferConfig:
    beam_size: int = 4
    search_type: str = "default"
    score_norm: bool = True
    return_best_hypothesis: bool = True
    tsd_max_sym_exp_per_step: Optional[int] = 50
    alsd_max_target_len: float = 1.0
    nsc_max_timesteps_expansion: int = 1
    nsc_prefix_alpha: int = 1
    maes_num_steps: int = 2
    maes_prefix_alpha: int = 1
    maes_expansion_gamma: float = 2.3
    maes_expansion_beta: int = 2
    language_model: Optional[Dict[str, Any]] = None
    softmax_temperature: float = 1.0
    preserve_alignments: bool = False
    ngram_lm_model: Optional[str] = None
    ngram_lm_alpha: Optional[float] = 0.0
    hat_subtract_ilm: bool = False
    hat_ilm_weight: float = 0.0
    max_symbols_per_step: Optional[int] = 10
    blank_lm_score_mode: Optional[str] = "no_score"
    pruning_mode: Optional[str] = "early"
    allow_cuda_graphs: bool = True


@dataclass
class RNNTDecodingConfig:
    model_type: str = "rnnt"
    strategy: str = "greedy_batch"
    compute_hypothesis_token_set: bool = False
    preserve_alignments: Optional[bool] = None
    tdt_include_token_duration: Optional[bool] = None
    confidence_cfg: Optional[Dict[str, Any]] = None
    fused_batch_size: Optional[int] = None
    compute_timestamps: Optional[bool] = None
    compute_langs: bool = False
    word_seperator: str = " "
    segment_seperators: Optional[List[str]] = field(default_factory=lambda: [".", "!", "?"])
    segment_gap_threshold: Optional[int] = None
    rnnt_timestamp_type: str = "all"
    greedy: GreedyBatchedRNNTInferConfig = field(default_factory=GreedyBatchedRNNTInferConfig)
    beam: BeamRNNTInferConfig = field(default_factory=BeamRNNTInferConfig)
    temperature: float = 1.0
    durations: Optional[List[int]] = field(default_factory=list)
    big_blank_durations: Optional[List[int]] = field(default_factory=list)


@dataclass
class RNNTBPEDecodingConfig(RNNTDecodingConfig):
    pass


class BeamRNNTInfer:
    """Per-utterance beam search (``default`` = the standard transducer beam search; ``alsd`` = alignment-length
    synchronous decoding).  Works for RNNT and TDT (duration argmax is taken greedily per expansion)."""

    def __init__(self, decoder, joint, blank_index: int, beam_size: int, search_type: str = "default",
                 score_norm: bool = True, return_best_hypothesis: bool = True, durations: Optional[List[int]] = None,
                 alsd_max_target_len: float = 1.0, max_symbols_per_step: Optional[int] = 10,
                 softmax_temperature: float = 1.0, ngram_lm=None, ngram_lm_alpha: float = 0.0, **_):
        self.decoder, self.joint, self.blank = decoder, joint, blank_index
        self.beam_size, self.search_type, self.score_norm = beam_size, search_type, score_norm
        self.return_best_hypothesis = return_best_hypothesis
        self.durations = list(durations or [])
        self.alsd_max_target_len = alsd_max_target_len
        self.max_symbols = max_symbols_per_step or 10
        self.temperature = softmax_temperature
        if search_type not in ("default", "alsd", "maes", "tsd"):
            raise NotImplementedError(f"beam search type '{search_type}' is not implemented; use default|alsd|maes|tsd")

    def _logp(self, f_t, dec_out):
        logits = self.joint.joint_after_projection(f_t.view(1, 1, -1), dec_out.view(1, 1, -1)).view(-1).float()
        nd = len(self.durations)
        if nd:
            return torch.log_softmax(logits[:-nd] / self.temperature, -1), torch.log_softmax(logits[-nd:], -1)
        if not (logits.exp().sum() - 1).abs() < 1e-3:
            logits = torch.log_softmax(logits / self.temperature, -1)
        return logits, None

    @torch.no_grad()
    def __call__(self, encoder_output: torch.Tensor, encoded_lengths: torch.Tensor):
        """encoder_output: [B, D, T]."""
        prev_log_softmax = self.joint.log_softmax
        self.joint.log_softmax = False
        try:
            enc = self.joint.project_encoder(encoder_output.transpose(1, 2).float())
            results = []
            for b in range(enc.shape[0]):
                nbest = self._search(enc[b, : int(encoded_lengths[b])])
                results.append(nbest[0] if self.return_best_hypothesis else NBestHypotheses(nbest))
        finally:
            self.joint.log_softmax = prev_log_softmax
        return (results,)

    def _search(self, f: torch.Tensor) -> List[Hypothesis]:
        T = f.shape[0]
        beam = self.beam_size
        dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=1)
        proj0 = self.joint.project_prednet(dec_out.float())[0, 0]
        init = Hypothesis(score=0.0, y_sequence=[], dec_state=state, timestamp=[], last_frame=0)
        init.dec_out = proj0
        # frame-synchronous search with per-hypothesis frame pointer (handles TDT jumps as well)
        hyps = [init]
        finished: List[Hypothesis] = []
        cache: Dict[Tuple[int, ...], Any] = {}
        steps = 0
        max_steps = T * (self.max_symbols + 1) + 8
        while hyps and steps < max_steps:
            steps += 1
            new: List[Hypothesis] = []
            for h in hyps:
                t = h.last_frame
                if t >= T:
                    finished.append(h)
                    continue
                logp, dlogp = self._logp(f[t], h.dec_out)
                topv, topi = logp.topk(min(beam + 1, logp.numel()))
                jump_b = 1
                jump_l = 0
                dsc = 0.0
                if dlogp is not None:
                    di = int(dlogp.argmax())
                    dsc = float(dlogp[di])
                    jump_l = self.durations[di]
                    jump_b = max(1, jump_l)
                # blank expansion
                nb = Hypothesis(score=h.score + float(logp[self.blank]) + dsc, y_sequence=h.y_sequence,
                                dec_state=h.dec_state, timestamp=h.timestamp, last_frame=t + jump_b)
                nb.dec_out = h.dec_out
                nb.token_duration = h.token_duration
                new.append(nb)
                same_frame = sum(1 for ts in h.timestamp[-self.max_symbols:] if ts == t)
                if same_frame >= self.max_symbols:
                    continue
                for v, k in zip(topv.tolist(), topi.tolist()):
                    if k == self.blank:
                        continue
                    seq = tuple(h.y_sequence) + (k,)
                    if seq in cache:
                        proj, st = cache[seq]
                    else:
                        tok = torch.tensor([[k]], device=f.device)
                        o, st = self.decoder.predict(tok, state=h.dec_state, add_sos=False, batch_size=1)
                        proj = self.joint.project_prednet(o.float())[0, 0]
                        cache[seq] = (proj, st)
                    nh = Hypothesis(score=h.score + v + dsc, y_sequence=list(seq), dec_state=st,
                                    timestamp=h.timestamp + [t], last_frame=t + jump_l)
                    nh.dec_out = proj
                    new.append(nh)
            # merge identical (sequence, frame) hypotheses, keep the best `beam`
            merged: Dict[Tuple[Tuple[int, ...], int], Hypothesis] = {}
            for h in new:
                key = (tuple(h.y_sequence), h.last_frame)
                if key in merged:
                    o = merged[key]
                    o.score = float(torch.logaddexp(torch.tensor(o.score), torch.tensor(h.score)))
                else:
                    merged[key] = h
            hyps = sorted(merged.values(), key=lambda h: h.score, reverse=True)[:beam]
        finished.extend(h for h in hyps if h.last_frame >= T)
        if not finished:
            finished = hyps or [init]
        best: Dict[Tuple[int, ...], Hypothesis] = {}
        for h in finished:
            k = tuple(h.y_sequence)
            if k not in best or h.score > best[k].score:
                best[k] = h
        out = list(best.values())
        if self.score_norm:
            out.sort(key=lambda h: h.score / max(1, len(h.y_sequence)), reverse=True)
        else:
            out.sort(key=lambda h: h.score, reverse=True)
        for h in out:
            h.y_sequence = torch.tensor(h.y_sequence, dtype=torch.long)
            h.timestamp = torch.tensor(h.timestamp, dtype=torch.long)
            h.dec_out = None
        return out[: self.beam_size]


class GreedyBatchedRNNTInfer:
    def __init__(self, decoder_model, joint_model, blank_index: int, durations=None, max_symbols_per_step=10,
                 preserve_alignments=False, preserve_frame_confidence=False, loop_labels=True,
                 use_cuda_graph_decoder=True, include_duration=False, fusion_models=None, fusion_models_alpha=None, **_):
        self.decoder, self.joint = decoder_model, joint_model
        self._blank_index = blank_index
        self.frame_looping = None
        if not loop_labels and not durations and not fusion_models and not preserve_alignments:
            from .rnnt_greedy import FrameLoopingBatchedComputer

            self.frame_looping = FrameLoopingBatchedComputer(decoder_model, joint_model, blank_index, max_symbols_per_step)
        self.decoding_computer = GreedyBatchedLabelLoopingComputer(
            decoder_model, joint_model, blank_index, durations, max_symbols_per_step, preserve_alignments,
            preserve_frame_confidence, include_duration, fusion_models, fusion_models_alpha,
            allow_cuda_graphs=use_cuda_graph_decoder)

    def disable_cuda_graphs(self):
        self.decoding_computer.disable_cuda_graphs()

    def maybe_enable_cuda_graphs(self):
        self.decoding_computer.maybe_enable_cuda_graphs()

    @torch.no_grad()
    def __call__(self, encoder_output: torch.Tensor, encoded_lengths: torch.Tensor,
                 partial_hypotheses: Optional[List[Hypothesis]] = None):
        """encoder_output: [B, D, T].  ``partial_hypotheses`` carry the decoder state for streaming continuation."""
        x = encoder_output.transpose(1, 2)
        prev = None
        if self.frame_looping is not None and partial_hypotheses is None:
            hyps = self.frame_looping(x, encoded_lengths.to(x.device))
            out = batched_hyps_to_hypotheses(hyps, None, batch_size=x.shape[0])
            for h, n in zip(out, encoded_lengths.tolist()):
                h.last_frame = int(n)
            return (out,)
        if partial_hypotheses is not None and any(h is not None and h.dec_state is not None for h in partial_hypotheses):
            # streams that join a running batch start from the prediction net's start-symbol state
            fresh = None
            states = []
            for h in partial_hypotheses:
                if h is not None and h.dec_state is not None:
                    states.append(h.dec_state)
                else:
                    if fresh is None:
                        fresh = self.decoding_computer.initial_state(1, x.device)
                    states.append(fresh)
            prev = merge_states(states)
        hyps, _, state = self.decoding_computer(x, encoded_lengths.to(x.device), prev)
        out = batched_hyps_to_hypotheses(hyps, None, batch_size=x.shape[0])
        states = split_state(state, x.shape[0])
        enc_lens = encoded_lengths.tolist()           # one device read for the whole batch
        for i, h in enumerate(out):
            h.dec_state = states[i]
            if partial_hypotheses is not None and partial_hypotheses[i] is not None:
                ph = partial_hypotheses[i]
                off = int(ph.last_frame or 0)
                h.y_sequence = torch.cat([torch.as_tensor(ph.y_sequence, dtype=torch.long), h.y_sequence])
                h.timestamp = torch.cat([torch.as_tensor(ph.timestamp, dtype=torch.long), h.timestamp + off])
                h.score = h.score + ph.score
                h.last_frame = off + int(enc_lens[i])
            else:
                h.last_frame = int(enc_lens[i])
        return (out,)


class BeamBatchedRNNTInfer:
    """``malsd_batch`` / ``maes_batch`` strategies: the GPU-resident beam search of ``batched_beam`` behind the decoder
    interface (reference: ``rnnt_beam_decoding.py`` ``BeamBatchedRNNTInfer`` / ``tdt_beam_decoding.py`` ``BeamBatchedTDTInfer``)."""

    def __init__(self, decoder_model, joint_model, blank_index: int, beam_size: int = 4, durations=None,
                 max_symbols_per_step=10, score_norm: bool = True, return_best_hypothesis: bool = True,
                 fusion_models=None, fusion_models_alpha=None, search_type: str = "malsd_batch", maes_num_steps: int = 2,
                 maes_expansion_beta: int = 2, maes_expansion_gamma: float = 2.3, **_):
        from .batched_beam import ModifiedAESBatchedComputer, ModifiedALSDBatchedComputer

        self.return_best_hypothesis = return_best_hypothesis
        self.score_norm = score_norm
        if search_type == "maes_batch":
            self.decoding_computer = ModifiedAESBatchedComputer(
                decoder_model, joint_model, blank_index, beam_size, maes_num_steps, maes_expansion_beta, maes_expansion_gamma,
                fusion_models, fusion_models_alpha, score_norm=score_norm, durations=durations)
        else:
            self.decoding_computer = ModifiedALSDBatchedComputer(
                decoder_model, joint_model, blank_index, beam_size, durations, max_symbols_per_step, fusion_models,
                fusion_models_alpha, score_norm=score_norm)

    @torch.no_grad()
    def __call__(self, encoder_output: torch.Tensor, encoded_lengths: torch.Tensor, partial_hypotheses=None):
        x = encoder_output.transpose(1, 2)
        with torch.autocast(x.device.type, enabled=False), ops.compute_dtype(None):
            beams = self.decoding_computer(x, encoded_lengths)
        out = []
        for nbest in beams.to_hyps_list(score_norm=self.score_norm):
            hs = [Hypothesis(score=s, y_sequence=torch.tensor(tok, dtype=torch.long), timestamp=torch.tensor(frm, dtype=torch.long))
                  for tok, frm, s in nbest] or [Hypothesis(score=0.0, y_sequence=torch.zeros(0, dtype=torch.long))]
            out.append(hs[0] if self.return_best_hypothesis else NBestHypotheses(hs))
        return (out,)


def split_state(state: LabelLoopingState, B: int) -> List[LabelLoopingState]:
    """Per-stream states as VIEWS of the batched tensors (no copies, no kernel launches); each remembers its parent and row so
    that ``merge_states`` can hand the parent back untouched when the same streams meet again in the same order."""
    out = []
    for i in range(B):
        ps = tuple(s[:, i:i + 1] for s in state.predictor_state) if state.predictor_state is not None else None
        st = LabelLoopingState(predictor_state=ps, predictor_output=state.predictor_output[i:i + 1], labels=state.labels[i:i + 1],
                               decoded_lengths=state.decoded_lengths[i:i + 1], time_jumps=state.time_jumps[i:i + 1],
                               fusion_states=[f[i:i + 1] for f in state.fusion_states] if state.fusion_states else None)
        st._batch_ref = (state, i, B)
        out.append(st)
    return out


def merge_states(states: List[LabelLoopingState]) -> LabelLoopingState:
    ref = getattr(states[0], "_batch_ref", None)
    if ref is not None and ref[2] == len(states) and all(getattr(s, "_batch_ref", (None, -1, 0))[0] is ref[0] and s._batch_ref[1] == i
                                                         for i, s in enumerate(states)):
        return ref[0]                       # the very batch these states were split from, in the same order
    ps = None
    if states[0].predictor_state is not None:
        ps = tuple(torch.cat([s.predictor_state[k] for s in states], dim=1) for k in range(len(states[0].predictor_state)))
    return LabelLoopingState(
        predictor_state=ps, predictor_output=torch.cat([s.predictor_output for s in states], dim=0),
        labels=torch.cat([s.labels for s in states]), decoded_lengths=torch.cat([s.decoded_lengths for s in states]),
        time_jumps=torch.cat([s.time_jumps for s in states]),
        fusion_states=[torch.cat([s.fusion_states[k] for s in states]) for k in range(len(states[0].fusion_states))]
        if states[0].fusion_states else None)


class AbstractRNNTDecoding:
    def __init__(self, decoding_cfg, decoder, joint, blank_id: int, supported_punctuation=None):
        if decoding_cfg is None:
            decoding_cfg = OmegaConf.structured(RNNTDecodingConfig)
        elif not isinstance(decoding_cfg, DictConfig):
            decoding_cfg = OmegaConf.create(decoding_cfg)
        self.cfg = decoding_cfg
        self.blank_id = blank_id
        self.supported_punctuation = supported_punctuation
        self.num_extra_outputs = joint.num_extra_outputs
        self.big_blank_durations = list(cfg_get(self.cfg, "big_blank_durations", None) or [])
        self.durations = list(cfg_get(self.cfg, "durations", None) or [])
        self.compute_hypothesis_token_set = cfg_get(self.cfg, "compute_hypothesis_token_set", False)
        self.compute_langs = cfg_get(self.cfg, "compute_langs", False)
        self.preserve_alignments = cfg_get(self.cfg, "preserve_alignments", None)
        self.compute_timestamps = cfg_get(self.cfg, "compute_timestamps", None)
        self.tdt_include_token_duration = cfg_get(self.cfg, "tdt_include_token_duration", False)
        self.word_seperator = cfg_get(self.cfg, "word_seperator", " ")
        self.segment_seperators = list(cfg_get(self.cfg, "segment_seperators", [".", "?", "!"]) or [])
        self.segment_gap_threshold = cfg_get(self.cfg, "segment_gap_threshold", None)
        self._is_tdt = len(self.durations) > 0
        if self._is_tdt and self.num_extra_outputs != len(self.durations):
            raise ValueError("the joint's num_extra_outputs must equal len(durations) for TDT decoding")
        strategy = cfg_get(self.cfg, "strategy", "greedy_batch")
        possible = ["greedy", "greedy_batch", "beam", "tsd", "alsd", "maes", "malsd_batch", "maes_batch"]
        if strategy not in possible:
            raise ValueError(f"Decoding strategy must be one of {possible}")
        self.strategy = strategy
        g = cfg_get(self.cfg, "greedy", None) or {}
        bm = cfg_get(self.cfg, "beam", None) or {}
        if strategy == "greedy" and not cfg_get(g, "ngram_lm_model", None) and not cfg_get(g, "boosting_tree", None):
            from .rnnt_greedy import GreedyRNNTInfer

            self.decoding = GreedyRNNTInfer(
                decoder, joint, blank_id, durations=self.durations,
                max_symbols_per_step=cfg_get(g, "max_symbols", None) or cfg_get(g, "max_symbols_per_step", 10),
                preserve_alignments=bool(self.preserve_alignments),
                preserve_frame_confidence=bool(cfg_get(self.cfg, "preserve_frame_confidence", False)),
                include_duration=bool(self.tdt_include_token_duration))
        elif strategy in ("greedy", "greedy_batch"):
            fusion_models, alphas = [], []
            if cfg_get(g, "ngram_lm_model", None):
                from .ngram_lm import NGramGPULanguageModel

                fusion_models.append(NGramGPULanguageModel.from_file(g["ngram_lm_model"], vocab_size=blank_id))
                alphas.append(cfg_get(g, "ngram_lm_alpha", 0.0))
            if cfg_get(g, "boosting_tree", None) and cfg_get(g, "boosting_tree_alpha", 0.0):
                from .context_biasing import GPUBoostingTreeModel

                bt = g["boosting_tree"]
                fusion_models.append(bt if hasattr(bt, "advance") else GPUBoostingTreeModel.from_config(bt))
                alphas.append(cfg_get(g, "boosting_tree_alpha", 0.0))
            self.decoding = GreedyBatchedRNNTInfer(
                decoder, joint, blank_id, durations=self.durations,
                max_symbols_per_step=cfg_get(g, "max_symbols", None) or cfg_get(g, "max_symbols_per_step", 10),
                preserve_alignments=bool(self.preserve_alignments), loop_labels=cfg_get(g, "loop_labels", True),
                use_cuda_graph_decoder=cfg_get(g, "use_cuda_graph_decoder", True),
                include_duration=bool(self.tdt_include_token_duration), fusion_models=fusion_models,
                fusion_models_alpha=alphas)
        elif strategy in ("malsd_batch", "maes_batch"):
            fusion_models, alphas = [], []
            if cfg_get(bm, "ngram_lm_model", None):
                from .ngram_lm import NGramGPULanguageModel

                fusion_models.append(NGramGPULanguageModel.from_file(bm["ngram_lm_model"], vocab_size=blank_id))
                alphas.append(cfg_get(bm, "ngram_lm_alpha", 0.0))
            if cfg_get(bm, "boosting_tree", None) is not None and cfg_get(bm, "boosting_tree_alpha", 0.0):
                bt = bm["boosting_tree"]
                if hasattr(bt, "advance"):
                    fusion_models.append(bt)
                    alphas.append(cfg_get(bm, "boosting_tree_alpha", 0.0))
            self.decoding = BeamBatchedRNNTInfer(
                decoder, joint, blank_id, beam_size=cfg_get(bm, "beam_size", 4), durations=self.durations,
                max_symbols_per_step=cfg_get(bm, "max_symbols_per_step", None) or cfg_get(bm, "max_symbols", 10),
                score_norm=cfg_get(bm, "score_norm", True), return_best_hypothesis=cfg_get(bm, "return_best_hypothesis", True),
                fusion_models=fusion_models, fusion_models_alpha=alphas, search_type=strategy,
                maes_num_steps=cfg_get(bm, "maes_num_steps", 2), maes_expansion_beta=cfg_get(bm, "maes_expansion_beta", 2),
                maes_expansion_gamma=cfg_get(bm, "maes_expansion_gamma", 2.3))
        else:
            st = {"beam": "default"}.get(strategy, strategy)
            self.decoding = BeamRNNTInfer(
                decoder, joint, blank_id, beam_size=cfg_get(bm, "beam_size", 4), search_type=st,
                score_norm=cfg_get(bm, "score_norm", True), return_best_hypothesis=cfg_get(bm, "return_best_hypothesis", True),
                durations=self.durations, alsd_max_target_len=cfg_get(bm, "alsd_max_target_len", 1.0),
                max_symbols_per_step=cfg_get(bm, "max_symbols_per_step", 10),
                softmax_temperature=cfg_get(bm, "softmax_temperature", 1.0))

    def rnnt_decoder_predictions_tensor(self, encoder_output: torch.Tensor, encoded_lengths: torch.Tensor,
                                        return_hypotheses: bool = False,
                                        partial_hypotheses: Optional[List[Hypothesis]] = None) -> List[Hypothesis]:
        with torch.inference_mode(False), torch.no_grad():
            if isinstance(self.decoding, GreedyBatchedRNNTInfer):
                (hyps,) = self.decoding(encoder_output, encoded_lengths, partial_hypotheses=partial_hypotheses)
            else:
                (hyps,) = self.decoding(encoder_output, encoded_lengths)
        if hyps and isinstance(hyps[0], NBestHypotheses):
            all_h = []
            for nb in hyps:
                dec = self.decode_hypothesis(nb.n_best_hypotheses)
                all_h.append(dec)
            return all_h if return_hypotheses else [h[0] for h in all_h]
        hyps = self.decode_hypothesis(hyps)
        if self.compute_timestamps:
            ts_type = cfg_get(self.cfg, "rnnt_timestamp_type", "all")
            for i in range(len(hyps)):
                hyps[i] = self.compute_rnnt_timestamps(hyps[i], ts_type)
        return hyps

    __call__ = rnnt_decoder_predictions_tensor

    def decode_hypothesis(self, hyps: List[Hypothesis]) -> List[Hypothesis]:
        for h in hyps:
            pred = h.y_sequence.tolist() if torch.is_tensor(h.y_sequence) else list(h.y_sequence)
            if self.big_blank_durations:
                nb = len(self.big_blank_durations)
                pred = [p for p in pred if p < self.blank_id - nb]
            else:
                pred = [p for p in pred if p != self.blank_id]
            h.text = self.decode_tokens_to_str(pred)
            if self.compute_hypothesis_token_set:
                h.tokens = self.decode_ids_to_tokens(pred)
        return hyps

    def compute_rnnt_timestamps(self, hyp: Hypothesis, timestamp_type: str = "all") -> Hypothesis:
        ids = hyp.y_sequence.tolist() if torch.is_tensor(hyp.y_sequence) else list(hyp.y_sequence)
        ts = hyp.timestamp.tolist() if torch.is_tensor(hyp.timestamp) else list(hyp.timestamp)
        durs = hyp.token_duration.tolist() if torch.is_tensor(hyp.token_duration) else None
        toks = self.decode_ids_to_tokens(ids)
        chars = []
        for i, (tok, t) in enumerate(zip(toks, ts)):
            end = t + (durs[i] if durs is not None and durs[i] > 0 else 1)
            chars.append({"char": [tok], "start_offset": t, "end_offset": end})
        result: Dict[str, Any] = {"timestep": ts}
        if timestamp_type in ("char", "all"):
            result["char"] = chars
        if timestamp_type in ("word", "all", "segment"):
            words = self._get_word_offsets(chars, ids)
            result["word"] = words
            if timestamp_type in ("segment", "all"):
                result["segment"] = self._get_segment_offsets(words)
        hyp.timestamp = result
        return hyp

    def _get_word_offsets(self, chars, ids) -> List[Dict[str, Any]]:
        words, cur, start, end = [], "", None, None
        for c in chars:
            tok = c["char"][0]
            new_word = tok.startswith("▁") or tok.startswith(" ") or (len(tok) == 1 and tok == self.word_seperator)
            piece = tok.replace("▁", "").strip() if tok not in (self.word_seperator,) else ""
            if new_word and cur:
                words.append({"word": cur, "start_offset": start, "end_offset": end})
                cur, start = "", None
            if piece:
                if not cur:
                    start = c["start_offset"]
                cur += piece if (tok.startswith("▁") or self._is_bpe()) else piece
                end = c["end_offset"]
        if cur:
            words.append({"word": cur, "start_offset": start, "end_offset": end})
        return words

    def _is_bpe(self) -> bool:
        return False

    def _get_segment_offsets(self, words) -> List[Dict[str, Any]]:
        segs, cur, start = [], [], None
        prev_end = None
        for w in words:
            gap_break = self.segment_gap_threshold is not None and prev_end is not None and \
                w["start_offset"] - prev_end >= self.segment_gap_threshold
            if gap_break and cur:
                segs.append({"segment": " ".join(cur), "start_offset": start, "end_offset": prev_end})
                cur, start = [], None
            if not cur:
                start = w["start_offset"]
            cur.append(w["word"])
            prev_end = w["end_offset"]
            if w["word"] and w["word"][-1] in self.segment_seperators:
                segs.append({"segment": " ".join(cur), "start_offset": start, "end_offset": prev_end})
                cur, start = [], None
        if cur:
            segs.append({"segment": " ".join(cur), "start_offset": start, "end_offset": prev_end})
        return segs

    def decode_tokens_to_str(self, tokens: List[int]) -> str:
        raise NotImplementedError

    def decode_ids_to_tokens(self, tokens: List[int]) -> List[str]:
        raise NotImplementedError


class RNNTDecoding(AbstractRNNTDecoding):
    def __init__(self, decoding_cfg, decoder, joint, vocabulary):
        blank_id = len(vocabulary) + joint.num_extra_outputs
        if cfg_get(decoding_cfg, "model_type", "rnnt") == "tdt" or (cfg_get(decoding_cfg, "durations", None)):
            blank_id = len(vocabulary)
        if cfg_get(decoding_cfg, "big_blank_durations", None):
            blank_id = len(vocabulary) + joint.num_extra_outputs
        self.labels_map = {i: vocabulary[i] for i in range(len(vocabulary))}
        super().__init__(decoding_cfg, decoder, joint, blank_id)

    def decode_tokens_to_str(self, tokens):
        return "".join(self.labels_map[t] for t in tokens if t in self.labels_map)

    def decode_ids_to_tokens(self, tokens):
        return [self.labels_map[t] for t in tokens if t in self.labels_map]


class RNNTBPEDecoding(AbstractRNNTDecoding):
    def __init__(self, decoding_cfg, decoder, joint, tokenizer):
        blank_id = tokenizer.vocab_size
        if cfg_get(decoding_cfg, "big_blank_durations", None):
            blank_id = tokenizer.vocab_size + joint.num_extra_outputs
        self.tokenizer = tokenizer
        super().__init__(decoding_cfg, decoder, joint, blank_id)

    def _is_bpe(self):
        return True

    def decode_tokens_to_str(self, tokens):
        return self.tokenizer.ids_to_text(tokens)

    def decode_ids_to_tokens(self, tokens):
        return self.tokenizer.ids_to_tokens(tokens)

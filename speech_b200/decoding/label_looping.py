"""Batched greedy label-looping decoding for RNNT and TDT.

The algorithm loops over *labels* (outer loop) and, inside, advances every utterance over blank
frames until it finds its next non-blank symbol (inner loop) — the scheme of
``nemo/collections/asr/parts/submodules/transducer_decoding/{rnnt,tdt}_label_looping.py``
(``torch_impl``: ``rnnt_label_looping.py:288-592``, ``tdt_label_looping.py:323-656``):

* the encoder output is projected once; the prediction-net output is projected after every label,
* TDT: ``t += durations[argmax(duration_logits)]``; a blank with duration 0 is forced to 1; labels may
  carry duration 0,
* ``max_symbols`` bounds the labels emitted on one frame (then the frame index is forced forward),
* an optional fusion model (n-gram LM / boosting tree) adds ``alpha * scores[B,V]`` to the non-blank
  logits but may not flip a blank into a label or back,
* the decoder state (LSTM state, last label, current frame) is returned so decoding continues across
  streaming chunks.

Two execution modes share the same step function: a host-driven loop (CPU, debugging) and, on GPUs, a
CUDA graph with device-side loop conditions built by the native graph builder
(``speech_b200.ops.native.LabelLoopingGraph``), which has zero host synchronisation per utterance batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

import torch

from .. import ops


class BatchedHyps:
    """Growing per-utterance token / timestamp / score arrays kept on the device
    (reference: ``parts/utils/rnnt_utils.py`` ``BatchedHyps``, ``batched_hyps.py:18-351``)."""

    def __init__(self, batch_size: int, init_length: int, device=None, float_dtype=torch.float32,
                 store_durations: bool = False):
        self._max_length = max(1, init_length)
        self.device = device
        self.current_lengths = torch.zeros(batch_size, device=device, dtype=torch.long)
        self.transcript = torch.zeros((batch_size, self._max_length), device=device, dtype=torch.long)
        self.timestamps = torch.zeros((batch_size, self._max_length), device=device, dtype=torch.long)
        self.token_durations = torch.zeros((batch_size, self._max_length), device=device, dtype=torch.long) \
            if store_durations else None
        self.scores = torch.zeros(batch_size, device=device, dtype=float_dtype)
        self.last_timestamp = torch.full((batch_size,), -1, device=device, dtype=torch.long)
        self.last_timestamp_lasts = torch.zeros(batch_size, device=device, dtype=torch.long)
        self._batch_indices = torch.arange(batch_size, device=device)

    def _grow(self):
        def g(t):
            return torch.cat([t, torch.zeros_like(t)], dim=-1)

        self.transcript, self.timestamps = g(self.transcript), g(self.timestamps)
        if self.token_durations is not None:
            self.token_durations = g(self.token_durations)
        self._max_length *= 2

    def add_results_masked_(self, active_mask, labels, time_indices, scores, token_durations=None):
        """In-place append for rows where ``active_mask``; no host sync unless storage must grow."""
        if int(self.current_lengths.max()) >= self._max_length:
            self._grow()
        self.add_results_masked_no_checks_(active_mask, labels, time_indices, scores, token_durations)

    def add_results_masked_no_checks_(self, active_mask, labels, time_indices, scores, token_durations=None):
        self.scores = torch.where(active_mask, self.scores + scores.to(self.scores.dtype), self.scores)
        idx = self.current_lengths.clamp(max=self._max_length - 1)
        cur_lab = self.transcript[self._batch_indices, idx]
        cur_ts = self.timestamps[self._batch_indices, idx]
        self.transcript[self._batch_indices, idx] = torch.where(active_mask, labels, cur_lab)
        self.timestamps[self._batch_indices, idx] = torch.where(active_mask, time_indices, cur_ts)
        if self.token_durations is not None and token_durations is not None:
            cur_d = self.token_durations[self._batch_indices, idx]
            self.token_durations[self._batch_indices, idx] = torch.where(active_mask, token_durations, cur_d)
        same = self.last_timestamp == time_indices
        self.last_timestamp_lasts = torch.where(active_mask & same, self.last_timestamp_lasts + 1,
                                                torch.where(active_mask, torch.ones_like(self.last_timestamp_lasts),
                                                            self.last_timestamp_lasts))
        self.last_timestamp = torch.where(active_mask, time_indices, self.last_timestamp)
        self.current_lengths = self.current_lengths + active_mask.long()


@dataclass
class LabelLoopingState:
    """Decoder state carried between calls (chunks): prediction-net state, its last projected output, last
    emitted label and per-utterance frame offset into the *next* chunk."""

    predictor_state: Any = None
    predictor_output: Optional[torch.Tensor] = None
    labels: Optional[torch.Tensor] = None
    decoded_lengths: Optional[torch.Tensor] = None
    time_jumps: Optional[torch.Tensor] = None
    fusion_states: Optional[list] = None


class GreedyBatchedLabelLoopingComputer:
    """RNNT when ``durations`` is empty, TDT otherwise."""

    def __init__(self, decoder, joint, blank_index: int, durations: Optional[List[int]] = None,
                 max_symbols_per_step: Optional[int] = 10, preserve_alignments: bool = False,
                 preserve_frame_confidence: bool = False, include_duration: bool = False, fusion_models=None,
                 fusion_models_alpha=None, allow_cuda_graphs: bool = True):
        self.decoder, self.joint = decoder, joint
        self._blank_index = blank_index
        self.durations = list(durations) if durations else []
        self.max_symbols = max_symbols_per_step
        self.include_duration = include_duration
        self.fusion_models = list(fusion_models or [])
        self.fusion_models_alpha = list(fusion_models_alpha or [])
        self.allow_cuda_graphs = allow_cuda_graphs
        self.cuda_graphs_mode: Optional[str] = None
        self._graph = None

    # ------------------------------------------------------------------ configuration toggles
    def force_cuda_graphs_mode(self, mode: Optional[str]):
        """``full_graph`` | ``no_while_loops`` | ``no_graphs`` | ``None`` (auto)."""
        if mode not in (None, "full_graph", "no_while_loops", "no_graphs"):
            raise ValueError(f"unknown cuda graphs mode {mode}")
        self.cuda_graphs_mode = mode
        self._graph = None

    def maybe_enable_cuda_graphs(self):
        self.allow_cuda_graphs = True

    def disable_cuda_graphs(self):
        self.allow_cuda_graphs = False
        self._graph = None

    # ------------------------------------------------------------------ entry point
    @torch.no_grad()
    def __call__(self, x: torch.Tensor, out_len: torch.Tensor, prev_batched_state: Optional[LabelLoopingState] = None
                 ) -> Tuple[BatchedHyps, None, LabelLoopingState]:
        """x: [B, T, D_enc] encoder output; out_len: [B].  Returns (hyps, alignments, state)."""
        use_graph = (x.is_cuda and self.allow_cuda_graphs and self.cuda_graphs_mode != "no_graphs"
                     and not self.fusion_models and not ops.eager_allowed() and ops.native_available()
                     and self._graph_supported())
        with torch.autocast(x.device.type, enabled=False), ops.compute_dtype(None):
            if use_graph:
                return self._graph_impl(x, out_len, prev_batched_state)
            return self.torch_impl(x, out_len, prev_batched_state)

    @torch.no_grad()
    def initial_state(self, batch_size: int, device) -> LabelLoopingState:
        """Decoder state of streams that have not emitted anything yet (prediction net fed with the start symbol)."""
        dt = torch.float32
        with torch.autocast(torch.device(device).type, enabled=False), ops.compute_dtype(None):
            dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=batch_size)
            dec_proj = self.joint.project_prednet(dec_out.to(dt))
        return LabelLoopingState(
            predictor_state=tuple(state) if state is not None else None, predictor_output=dec_proj,
            labels=torch.full((batch_size,), self._blank_index, device=device, dtype=torch.long),
            decoded_lengths=torch.zeros(batch_size, device=device, dtype=torch.long),
            time_jumps=torch.zeros(batch_size, device=device, dtype=torch.long), fusion_states=None)

    def _graph_supported(self) -> bool:
        from ..ops import native

        return hasattr(native, "LabelLoopingGraph") and native.LabelLoopingGraph.supports(self)

    def _graph_impl(self, x, out_len, prev):
        from ..ops import native

        if self._graph is None:
            self._graph = native.LabelLoopingGraph(self)
        return self._graph(x, out_len, prev)

    # ------------------------------------------------------------------ host-driven implementation
    def torch_impl(self, x, out_len, prev: Optional[LabelLoopingState] = None):
        B, T, _ = x.shape
        dev = x.device
        dt = torch.float32
        enc = self.joint.project_encoder(x.to(dt))  # [B,T,H]
        lin = self.joint.joint_net[-1]
        act = self.joint.joint_net[0]
        nd = len(self.durations)
        dur_t = torch.tensor(self.durations, device=dev, dtype=torch.long) if nd else None
        hyps = BatchedHyps(B, init_length=max(8, T * 2 if self.max_symbols is None else T), device=dev,
                           store_durations=self.include_duration and nd > 0)
        bidx = torch.arange(B, device=dev)
        if prev is None or prev.predictor_state is None:
            state = self.decoder.initialize_state(torch.zeros(B, 1, device=dev, dtype=dt))
            dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=B)
            state = tuple(state) if state is not None else None
            dec_proj = self.joint.project_prednet(dec_out.to(dt))  # [B,1,H]
            time_idx = torch.zeros(B, device=dev, dtype=torch.long)
            labels = torch.full((B,), self._blank_index, device=dev, dtype=torch.long)
        else:
            state, dec_proj = prev.predictor_state, prev.predictor_output
            time_idx = prev.time_jumps.clone() if prev.time_jumps is not None else torch.zeros(B, device=dev, dtype=torch.long)
            labels = prev.labels.clone()
        fusion_states = None
        if self.fusion_models:
            fusion_states = prev.fusion_states if (prev is not None and prev.fusion_states is not None) else \
                [m.get_init_states(batch_size=B, bos=True) for m in self.fusion_models]
        last_t = (out_len - 1).clamp(min=0)
        active = time_idx < out_len
        V1 = lin.out_features - nd

        def joint_step(tidx):
            f = enc[bidx, torch.minimum(tidx, last_t)]
            h = act(f + dec_proj[:, 0])
            return torch.nn.functional.linear(h, lin.weight.to(dt), lin.bias.to(dt))

        while bool(active.any()):
            logits = joint_step(time_idx)
            tok = logits[:, :V1]
            scores, lab = tok.max(dim=-1)
            if self.fusion_models:
                fused = tok.clone()
                fscores = []
                for m, a, st in zip(self.fusion_models, self.fusion_models_alpha, fusion_states):
                    sc, nxt = m.advance(st)
                    fscores.append((sc, nxt))
                    fused[:, : self._blank_index] += a * sc.to(dt)
                nb_scores, nb_lab = fused[:, : self._blank_index].max(dim=-1)
                lab = torch.where(lab == self._blank_index, lab, nb_lab)
            if nd:
                jump = dur_t[logits[:, V1:].argmax(dim=-1)]
            else:
                jump = (lab == self._blank_index).long()
            is_blank = lab == self._blank_index
            if nd:
                jump = torch.where(is_blank & (jump == 0), torch.ones_like(jump), jump)
            time_start = time_idx.clone()
            time_idx = time_idx + torch.where(active, jump, torch.zeros_like(jump))
            active = time_idx < out_len
            advance = active & is_blank
            # inner loop: rows that are on a blank keep moving until they find a label or run out of frames
            while bool(advance.any()):
                time_start = torch.where(advance, time_idx, time_start)
                logits2 = joint_step(time_idx)
                tok2 = logits2[:, :V1]
                s2, l2 = tok2.max(dim=-1)
                if self.fusion_models:
                    fused2 = tok2.clone()
                    for (sc, _), a in zip(fscores, self.fusion_models_alpha):
                        fused2[:, : self._blank_index] += a * sc.to(dt)
                    _, nbl2 = fused2[:, : self._blank_index].max(dim=-1)
                    l2 = torch.where(l2 == self._blank_index, l2, nbl2)
                if nd:
                    j2 = dur_t[logits2[:, V1:].argmax(dim=-1)]
                    j2 = torch.where((l2 == self._blank_index) & (j2 == 0), torch.ones_like(j2), j2)
                else:
                    j2 = (l2 == self._blank_index).long()
                lab = torch.where(advance, l2, lab)
                scores = torch.where(advance, s2, scores)
                jump = torch.where(advance, j2, jump)
                time_idx = time_idx + torch.where(advance, j2, torch.zeros_like(j2))
                is_blank = lab == self._blank_index
                active = time_idx < out_len
                advance = active & is_blank
            found = (lab != self._blank_index) & (time_start < out_len)
            hyps.add_results_masked_(found, lab, time_start, scores, jump if nd else None)
            # prediction network step for rows that found a label
            emb_in = torch.where(found, lab, torch.full_like(lab, self._blank_index)).unsqueeze(1)
            new_out, new_state = self.decoder.predict(emb_in, state=state, add_sos=False, batch_size=B)
            new_proj = self.joint.project_prednet(new_out.to(dt))
            dec_proj = torch.where(found[:, None, None], new_proj, dec_proj)
            if state is None:
                state = tuple(new_state)
            else:
                self.decoder.batch_replace_states_mask(list(new_state), list(state), found)
            labels = torch.where(found, lab, labels)
            if self.fusion_models:
                for i, (sc, nxt) in enumerate(fscores):
                    picked = nxt[bidx, lab.clamp(max=self._blank_index - 1)]
                    fusion_states[i] = torch.where(found, picked, fusion_states[i])
            if self.max_symbols is not None:
                force = active & found & (hyps.last_timestamp_lasts >= self.max_symbols) & (hyps.last_timestamp == time_idx)
                time_idx = time_idx + force.long()
                active = time_idx < out_len
        out_state = LabelLoopingState(predictor_state=state, predictor_output=dec_proj, labels=labels,
                                      decoded_lengths=out_len.clone(), time_jumps=(time_idx - out_len).clamp(min=0),
                                      fusion_states=fusion_states)
        return hyps, None, out_state

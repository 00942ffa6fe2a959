"""Greedy transducer decoders other than the label-looping one.

* :class:`GreedyRNNTInfer` (``strategy: greedy``) decodes one utterance at a time, frame by frame, the way the textbook
  algorithm is written (reference ``rnnt_greedy_decoding.py`` ``GreedyRNNTInfer`` / ``GreedyTDTInfer``).  It is the
  reference point for the batched decoders and keeps per-frame alignments and confidences cheaply.
* :class:`FrameLoopingBatchedComputer` (``greedy_batch`` with ``loop_labels: false``) walks the *frames* of the whole batch
  in lockstep and, inside a frame, emits labels for the rows that are not on blank yet (reference
  ``GreedyBatchedRNNTInfer._greedy_decode_blank_as_pad_loop_frames``).  Plain RNNT only: with TDT durations rows jump by
  different amounts and label looping is the batched algorithm.

Both return the same :class:`BatchedHyps` / :class:`Hypothesis` records as the label-looping decoder and give the same
transcripts; which one is fastest depends on how many labels per frame the model emits.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .label_looping import BatchedHyps


class _JointStep:
    """Projected encoder frames + one prediction-net vector -> logits, without materialising the joint lattice."""

    def __init__(self, joint, x: torch.Tensor):
        self.joint = joint
        self.enc = joint.project_encoder(x.float())          # [B, T, H]
        self.lin, self.act = joint.joint_net[-1], joint.joint_net[0]

    def __call__(self, f: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(self.act(f + g), self.lin.weight.float(), self.lin.bias.float())


class GreedyRNNTInfer:
    def __init__(self, decoder_model, joint_model, blank_index: int, durations=None, max_symbols_per_step: Optional[int] = 10,
                 preserve_alignments: bool = False, preserve_frame_confidence: bool = False, include_duration: bool = False, **_):
        self.decoder, self.joint, self.blank = decoder_model, joint_model, blank_index
        self.durations = list(durations or [])
        self.max_symbols = max_symbols_per_step
        self.preserve_alignments, self.preserve_frame_confidence = preserve_alignments, preserve_frame_confidence
        self.include_duration = include_duration

    @torch.no_grad()
    def __call__(self, encoder_output: torch.Tensor, encoded_lengths: torch.Tensor, partial_hypotheses=None):
        """encoder_output: [B, D, T]."""
        from .rnnt_decoding import Hypothesis

        x = encoder_output.transpose(1, 2)
        lens = encoded_lengths.tolist()
        out: List[Hypothesis] = []
        for b in range(x.shape[0]):
            prev = partial_hypotheses[b] if partial_hypotheses is not None else None
            out.append(self._decode_one(x[b:b + 1, : int(lens[b])], prev))
        return (out,)

    def _decode_one(self, x: torch.Tensor, prev=None):
        from .rnnt_decoding import Hypothesis

        step = _JointStep(self.joint, x)
        T = x.shape[1]
        nd = len(self.durations)
        V1 = step.lin.out_features - nd
        if prev is not None and prev.dec_state is not None and isinstance(prev.dec_state, tuple) and len(prev.dec_state) == 2 \
                and torch.is_tensor(prev.dec_state[1]):
            state, g = prev.dec_state
        else:
            dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=1)
            g = self.joint.project_prednet(dec_out.float())[:, 0]
        toks, frames, durs, score = [], [], [], 0.0
        alignments, confidences = [], []
        t = 0
        emitted_here = 0
        while t < T:
            logits = step(step.enc[:, t], g)[0]
            logp = torch.log_softmax(logits[:V1], dim=-1)
            k = int(logp.argmax())
            d = self.durations[int(logits[V1:].argmax())] if nd else (1 if k == self.blank else 0)
            if self.preserve_alignments:
                while len(alignments) <= t:
                    alignments.append([])
                alignments[t].append((logp.cpu(), k))
            if self.preserve_frame_confidence:
                while len(confidences) <= t:
                    confidences.append([])
                confidences[t].append(float(logp[k].exp()))
            if k == self.blank:
                t += max(1, d)
                emitted_here = 0
                continue
            toks.append(k)
            frames.append(t)
            durs.append(d)
            score += float(logp[k])
            dec_out, state = self.decoder.predict(torch.tensor([[k]], device=x.device), state=state, add_sos=False, batch_size=1)
            g = self.joint.project_prednet(dec_out.float())[:, 0]
            emitted_here = emitted_here + 1 if d == 0 else 0
            t += d
            if self.max_symbols is not None and emitted_here >= self.max_symbols:
                t += 1
                emitted_here = 0
        off = int(prev.last_frame or 0) if prev is not None else 0
        y = torch.tensor(toks, dtype=torch.long)
        ts = torch.tensor(frames, dtype=torch.long) + off
        if prev is not None:
            y = torch.cat([torch.as_tensor(prev.y_sequence, dtype=torch.long), y])
            ts = torch.cat([torch.as_tensor(prev.timestamp, dtype=torch.long), ts])
            score += float(prev.score)
        h = Hypothesis(score=score, y_sequence=y, timestamp=ts, dec_state=(state, g), last_frame=off + T)
        if self.include_duration and nd:
            h.token_duration = torch.tensor(durs, dtype=torch.long)
        if self.preserve_alignments:
            h.alignments = alignments
        if self.preserve_frame_confidence:
            h.frame_confidence = confidences
        return h


class FrameLoopingBatchedComputer:
    """Batched greedy RNNT with the outer loop over frames.  ``__call__(x [B, T, D], out_len [B]) -> BatchedHyps``."""

    def __init__(self, decoder, joint, blank_index: int, max_symbols_per_step: Optional[int] = 10):
        self.decoder, self.joint, self.blank = decoder, joint, blank_index
        self.max_symbols = max_symbols_per_step

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, out_len: torch.Tensor):
        B, T, _ = x.shape
        dev = x.device
        step = _JointStep(self.joint, x)
        hyps = BatchedHyps(B, init_length=max(8, T), device=dev)
        dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=B)
        state = list(state) if state is not None else None
        g = self.joint.project_prednet(dec_out.float())[:, 0]                 # [B, H]
        out_len = out_len.to(dev)
        for t in range(int(T)):
            in_range = out_len > t
            not_blank = in_range.clone()
            f = step.enc[:, t]
            tvec = torch.full((B,), t, device=dev, dtype=torch.long)
            n = 0
            while bool(not_blank.any()) and (self.max_symbols is None or n < self.max_symbols):
                logits = step(f, g)
                sc, lab = logits.max(dim=-1)
                found = not_blank & (lab != self.blank)
                not_blank = found
                if not bool(found.any()):
                    break
                hyps.add_results_masked_(found, lab, tvec, sc)
                emb = torch.where(found, lab, torch.full_like(lab, self.blank)).unsqueeze(1)
                new_out, new_state = self.decoder.predict(emb, state=state, add_sos=False, batch_size=B)
                new_g = self.joint.project_prednet(new_out.float())[:, 0]
                g = torch.where(found.unsqueeze(-1), new_g, g)
                if state is None:
                    state = list(new_state) if new_state is not None else None
                elif new_state is not None:
                    self.decoder.batch_replace_states_mask(list(new_state), state, found)
                n += 1
        self.final_state, self.final_output = state, g
        return hyps

"""CUDA-graph greedy transducer decoding (RNNT / TDT) with no host synchronisation inside the loop.

The reference captures its label-looping algorithm as one CUDA graph with nested WHILE conditional nodes
(``tdt_label_looping.py:1158-1433``, ``rnnt_label_looping.py``).  Here the two nested loops are merged into ONE
fixed-shape step — every live stream evaluates the joint at its current frame; a blank advances the frame (by the predicted
duration for TDT), a label is appended and advances the prediction network of that stream only — so the whole decode is
``n`` replays of a single captured graph:

* the step is captured once per ``(batch, frames, capacity)`` shape with ``torch.cuda.CUDAGraph``; all state lives in
  static buffers (prediction-net state, projected prediction-net output, frame index, symbols-on-frame counter, hypotheses),
* the host replays the graph in bursts of ``check_every`` steps and looks at a single device flag between bursts (one
  4-byte read), so the GPU queue never drains,
* greedy decisions depend only on (frame, prediction-net state), therefore the result equals the nested-loop algorithm
  (``label_looping.GreedyBatchedLabelLoopingComputer.torch_impl``) token for token, including ``max_symbols`` handling,
  TDT durations (blank with duration 0 forced to 1) and continuation across streaming chunks.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from .label_looping import BatchedHyps, LabelLoopingState


class LabelLoopingGraph:
    def __init__(self, computer, check_every: int = 16):
        self.c = computer
        self.check_every = check_every
        self._graphs: Dict[Tuple[int, int, int], dict] = {}

    @staticmethod
    def supports(computer) -> bool:
        from ..modules.rnnt import RNNTDecoder

        return not computer.fusion_models and isinstance(computer.decoder, RNNTDecoder)

    # ------------------------------------------------------------------ one fixed-shape step on static buffers
    def _build(self, B: int, T: int, cap: int, dev, H: int):
        c = self.c
        dt = torch.float32
        nd = len(c.durations)
        lin = c.joint.joint_net[-1]
        act = c.joint.joint_net[0]
        V1 = lin.out_features - nd
        blank = c._blank_index
        max_sym = c.max_symbols if c.max_symbols is not None else 1 << 30
        s = {
            "enc": torch.zeros((B, T, H), device=dev, dtype=dt), "out_len": torch.zeros(B, device=dev, dtype=torch.long),
            "dec_proj": torch.zeros((B, 1, H), device=dev, dtype=dt), "time": torch.zeros(B, device=dev, dtype=torch.long),
            "sym": torch.zeros(B, device=dev, dtype=torch.long), "labels": torch.full((B,), blank, device=dev, dtype=torch.long),
            "any_active": torch.ones(1, device=dev, dtype=torch.int32),
            "transcript": torch.zeros((B, cap), device=dev, dtype=torch.long), "stamps": torch.zeros((B, cap), device=dev, dtype=torch.long),
            "durs": torch.zeros((B, cap), device=dev, dtype=torch.long), "length": torch.zeros(B, device=dev, dtype=torch.long),
            "score": torch.zeros(B, device=dev, dtype=dt),
            "w": lin.weight.detach().to(dt), "b": lin.bias.detach().to(dt),
            "dur_t": torch.tensor(c.durations or [0], device=dev, dtype=torch.long),
        }
        init = c.decoder.initialize_state(torch.zeros(B, 1, device=dev, dtype=dt))
        s["state"] = [torch.zeros_like(t) for t in init]
        bidx = torch.arange(B, device=dev)

        def step():
            t, out_len = s["time"], s["out_len"]
            active = t < out_len
            f = s["enc"][bidx, torch.minimum(t, (out_len - 1).clamp(min=0))]
            logits = torch.nn.functional.linear(act(f + s["dec_proj"][:, 0]), s["w"], s["b"])
            score, lab = logits[:, :V1].max(dim=-1)
            is_blank = lab == blank
            if nd:
                jump = s["dur_t"][logits[:, V1:].argmax(dim=-1)]
                jump = torch.where(is_blank & (jump == 0), torch.ones_like(jump), jump)
            else:
                jump = is_blank.long()
            found = active & ~is_blank
            # append the label (rows that found one)
            pos = s["length"].clamp(max=cap - 1).unsqueeze(1)
            s["transcript"].scatter_(1, pos, torch.where(found, lab, s["transcript"].gather(1, pos).squeeze(1)).unsqueeze(1))
            s["stamps"].scatter_(1, pos, torch.where(found, t, s["stamps"].gather(1, pos).squeeze(1)).unsqueeze(1))
            s["durs"].scatter_(1, pos, torch.where(found, jump, s["durs"].gather(1, pos).squeeze(1)).unsqueeze(1))
            s["length"].add_(found.long())
            s["score"].add_(torch.where(found, score, torch.zeros_like(score)))
            s["labels"].copy_(torch.where(found, lab, s["labels"]))
            # frame bookkeeping: a label that stays on its frame counts towards max_symbols, which forces the frame forward
            sym = torch.where(found & (jump == 0), s["sym"] + 1, torch.zeros_like(s["sym"]))
            forced = found & (jump == 0) & (sym >= max_sym)
            s["sym"].copy_(torch.where(forced, torch.zeros_like(sym), sym))
            s["time"].add_(torch.where(active, jump + forced.long(), torch.zeros_like(jump)))
            # prediction network for the rows that emitted (fixed shape: all rows run, the others keep their state)
            emb_in = torch.where(found, lab, torch.full_like(lab, blank)).unsqueeze(1)
            new_out, new_state = c.decoder.predict(emb_in, state=tuple(s["state"]), add_sos=False, batch_size=B)
            new_proj = c.joint.project_prednet(new_out.to(dt))
            s["dec_proj"].copy_(torch.where(found[:, None, None], new_proj, s["dec_proj"]))
            for old, new in zip(s["state"], new_state):
                old.copy_(torch.where(found.view(1, B, 1), new.to(old.dtype), old))
            s["any_active"].copy_((s["time"] < out_len).any().to(torch.int32).view(1))

        s["step"] = step
        return s

    def _get(self, B, T, cap, dev, H):
        key = (B, T, cap)
        g = self._graphs.get(key)
        if g is None:
            g = self._build(B, T, cap, dev, H)
            self._graphs[key] = g
        return g

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, out_len: torch.Tensor, prev: Optional[LabelLoopingState] = None):
        c = self.c
        B, T, _ = x.shape
        dev = x.device
        dt = torch.float32
        enc = c.joint.project_encoder(x.to(dt))
        H = enc.shape[-1]
        Tp = -(-T // 16) * 16                                   # few distinct graph shapes: frames rounded up to 16
        per_frame = c.max_symbols if c.max_symbols is not None else 4
        cap = Tp * min(per_frame, 4) + 16
        s = self._get(B, Tp, cap, dev, H)
        s["enc"].zero_()
        s["enc"][:, :T].copy_(enc)
        s["out_len"].copy_(out_len.to(dev))
        s["transcript"].zero_(); s["stamps"].zero_(); s["durs"].zero_(); s["length"].zero_(); s["score"].zero_(); s["sym"].zero_()
        if prev is None or prev.predictor_state is None:
            init = c.initial_state(B, dev)
        else:
            init = prev
        for old, new in zip(s["state"], init.predictor_state):
            old.copy_(new.to(old.dtype))
        s["dec_proj"].copy_(init.predictor_output.to(dt))
        s["labels"].copy_(init.labels)
        s["time"].copy_(init.time_jumps if init.time_jumps is not None else torch.zeros_like(s["time"]))
        s["any_active"].fill_(1)
        if "graph" not in s:
            # warm-up on a side stream (lazy initialisation, allocator), then capture one step
            snap = {k: v.clone() for k, v in s.items() if torch.is_tensor(v)}
            st_snap = [t.clone() for t in s["state"]]
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                s["step"]()
            torch.cuda.current_stream(dev).wait_stream(side)
            for k, v in snap.items():
                s[k].copy_(v)
            for t, v in zip(s["state"], st_snap):
                t.copy_(v)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                s["step"]()
            for k, v in snap.items():
                s[k].copy_(v)
            for t, v in zip(s["state"], st_snap):
                t.copy_(v)
            s["graph"] = g
        max_iters = int(Tp) * (1 + min(per_frame, 4)) + 8
        if "flag" not in s:
            s["flag"] = torch.zeros(2, dtype=torch.int32).pin_memory()
        flag = s["flag"]
        it, burst, pending = 0, 0, None
        while it < max_iters:
            for _ in range(self.check_every):
                s["graph"].replay()
            it += self.check_every
            # the flag of burst k is read while burst k+1 is already queued, so the device never waits for the host
            slot = burst & 1
            flag[slot:slot + 1].copy_(s["any_active"], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            if pending is not None:
                pending[1].synchronize()
                if int(flag[pending[0]]) == 0:
                    break
            pending = (slot, ev)
            burst += 1
        torch.cuda.current_stream(dev).synchronize()
        n = s["length"].clone()
        hyps = BatchedHyps(B, init_length=max(1, int(n.max())), device=dev, store_durations=c.include_duration and len(c.durations) > 0)
        L = min(hyps.transcript.shape[1], s["transcript"].shape[1])      # the two buffers round their capacities differently
        hyps.transcript[:, :L].copy_(s["transcript"][:, :L])
        hyps.timestamps[:, :L].copy_(s["stamps"][:, :L])
        if hyps.token_durations is not None:
            hyps.token_durations[:, :L].copy_(s["durs"][:, :L])
        hyps.current_lengths.copy_(n)
        hyps.scores.copy_(s["score"])
        state = LabelLoopingState(predictor_state=tuple(t.clone() for t in s["state"]), predictor_output=s["dec_proj"].clone(),
                                  labels=s["labels"].clone(), decoded_lengths=s["out_len"].clone(),
                                  time_jumps=(s["time"] - s["out_len"]).clamp(min=0), fusion_states=None)
        return hyps, None, state

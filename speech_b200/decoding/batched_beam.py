"""GPU-resident batched beam search: modified alignment-length synchronous decoding (MALSD) for RNNT / TDT and prefix beam
search for CTC.  Every tensor carries a ``[batch, beam]`` leading shape, all per-step work is vectorised torch ops (plus the
framework's LSTM / joint kernels), and the loop condition is the only host read per step.

Reference behaviour: ``rnnt_malsd_batched_computer.py:233`` / ``tdt_malsd_batched_computer.py:227`` (expand every beam entry
by blank and by its best labels, keep the ``beam_size`` best per utterance, recombine entries with equal transcripts,
optional n-gram LM / boosting-tree fusion with ``blank_lm_score_mode`` "no_score" semantics), ``BatchedBeamHyps``
(``parts/utils/batched_beam_decoding_utils.py``) and ``ctc_batched_beam_decoding.py:154``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

NEG = -1e30
_HASH_MUL = 1000003


class BatchedBeamHyps:
    """Beam storage: token arrays ``[B, K, L]`` with lengths, scores, per-token frame indices and a rolling hash that
    identifies equal transcripts."""

    def __init__(self, batch_size: int, beam_size: int, init_length: int, device, blank: int):
        B, K = batch_size, beam_size
        self.B, self.K, self.blank = B, K, blank
        self.max_len = max(4, init_length)
        self.tokens = torch.zeros((B, K, self.max_len), dtype=torch.long, device=device)
        self.frames = torch.zeros((B, K, self.max_len), dtype=torch.long, device=device)
        self.lengths = torch.zeros((B, K), dtype=torch.long, device=device)
        self.scores = torch.full((B, K), NEG, dtype=torch.float32, device=device)
        self.scores[:, 0] = 0.0
        self.hash = torch.zeros((B, K), dtype=torch.long, device=device)
        self.prev_hash = torch.full((B, K), -1, dtype=torch.long, device=device)   # hash of the transcript without its last token
        self.last_label = torch.full((B, K), blank, dtype=torch.long, device=device)

    def _grow(self):
        z = torch.zeros_like(self.tokens)
        self.tokens = torch.cat([self.tokens, z], dim=-1)
        self.frames = torch.cat([self.frames, torch.zeros_like(z)], dim=-1)
        self.max_len *= 2

    def reorder_and_extend(self, src: torch.Tensor, labels: torch.Tensor, frames: torch.Tensor, scores: torch.Tensor):
        """New beam entry k continues old entry ``src[b,k]``; ``labels`` < 0 (or blank) means no token is appended."""
        if int(self.lengths.max()) + 1 >= self.max_len:
            self._grow()
        idx = src.unsqueeze(-1).expand(-1, -1, self.max_len)
        self.tokens = self.tokens.gather(1, idx)
        self.frames = self.frames.gather(1, idx)
        self.lengths = self.lengths.gather(1, src)
        self.hash = self.hash.gather(1, src)
        self.prev_hash = self.prev_hash.gather(1, src)
        self.last_label = self.last_label.gather(1, src)
        add = (labels >= 0) & (labels != self.blank)
        pos = self.lengths.clamp(max=self.max_len - 1).unsqueeze(-1)
        self.tokens.scatter_(2, pos, torch.where(add, labels, self.tokens.gather(2, pos).squeeze(-1)).unsqueeze(-1))
        self.frames.scatter_(2, pos, torch.where(add, frames, self.frames.gather(2, pos).squeeze(-1)).unsqueeze(-1))
        self.lengths = self.lengths + add.long()
        self.prev_hash = torch.where(add, self.hash, self.prev_hash)
        self.hash = torch.where(add, (self.hash * _HASH_MUL + labels + 1) % 2305843009213693951, self.hash)
        self.last_label = torch.where(add, labels, self.last_label)
        self.scores = scores

    def recombine(self, extra_key: Optional[torch.Tensor] = None, mode: str = "max"):
        """Entries of one utterance with equal transcripts (and equal ``extra_key``): keep the first, fold the others' score
        into it (``max`` or log-sum-exp) and deactivate them."""
        same = (self.hash.unsqueeze(2) == self.hash.unsqueeze(1)) & (self.lengths.unsqueeze(2) == self.lengths.unsqueeze(1))
        if extra_key is not None:
            same = same & (extra_key.unsqueeze(2) == extra_key.unsqueeze(1))
        valid = self.scores > NEG / 2
        same = same & valid.unsqueeze(1) & valid.unsqueeze(2)
        K = self.K
        order = torch.arange(K, device=self.scores.device)
        earlier = same & (order.view(1, 1, K) < order.view(1, K, 1))      # [b, i, j]: j < i duplicates i
        is_dup = earlier.any(dim=2)
        grp = same & ~is_dup.unsqueeze(1)                                   # rows of survivors gather their group
        sc = self.scores.unsqueeze(1).expand(-1, K, -1).masked_fill(~same, NEG)
        merged = sc.max(dim=2).values if mode == "max" else torch.logsumexp(sc, dim=2)
        self.scores = torch.where(is_dup, torch.full_like(self.scores, NEG), torch.where(valid, merged, self.scores))

    def to_hyps_list(self, score_norm: bool = True) -> List[List[Tuple[List[int], List[int], float]]]:
        out = []
        sc = self.scores / self.lengths.clamp(min=1).float() if score_norm else self.scores
        sc = torch.where(self.scores > NEG / 2, sc, torch.full_like(sc, NEG))
        order = sc.argsort(dim=1, descending=True)
        tok, frm, ln, s = self.tokens.cpu(), self.frames.cpu(), self.lengths.cpu(), self.scores.cpu()
        for b in range(self.B):
            cur = []
            for k in order[b].tolist():
                if float(s[b, k]) <= NEG / 2:
                    continue
                n = int(ln[b, k])
                cur.append((tok[b, k, :n].tolist(), frm[b, k, :n].tolist(), float(s[b, k])))
            out.append(cur)
        return out


class MALSDCarry:
    """What MALSD keeps between two chunks of a stream: the beam, the prediction-network state and output of every entry, how far
    an entry's time index ran past the end of the chunk (TDT durations may jump over it), language-model states, and the number of
    encoder frames consumed so far (so that token frame indices stay global).  ``merge`` stacks the carries of several streams into
    one batch and ``split`` undoes it, which lets a server batch whichever streams have a chunk ready."""

    def __init__(self, hyps: BatchedBeamHyps, state, dec_proj: torch.Tensor, t_over: torch.Tensor, fstates: list, frame_offset: torch.Tensor):
        self.hyps, self.state, self.dec_proj, self.t_over, self.fstates, self.frame_offset = hyps, state, dec_proj, t_over, fstates, frame_offset

    @staticmethod
    def merge(carries: "List[MALSDCarry]") -> "MALSDCarry":
        h0 = carries[0].hyps
        L = max(c.hyps.max_len for c in carries)
        B = sum(c.hyps.B for c in carries)
        hy = BatchedBeamHyps(B, h0.K, L, h0.tokens.device, h0.blank)
        hy.max_len = L
        pad = lambda t: torch.nn.functional.pad(t, (0, L - t.shape[-1]))  # noqa: E731
        hy.tokens = torch.cat([pad(c.hyps.tokens) for c in carries], 0)
        hy.frames = torch.cat([pad(c.hyps.frames) for c in carries], 0)
        for name in ("lengths", "scores", "hash", "prev_hash", "last_label"):
            setattr(hy, name, torch.cat([getattr(c.hyps, name) for c in carries], 0))
        state = None
        if carries[0].state is not None:
            state = [torch.cat([c.state[i] for c in carries], dim=1) for i in range(len(carries[0].state))]
        fst = [torch.cat([c.fstates[i] for c in carries], 0) for i in range(len(carries[0].fstates))]
        return MALSDCarry(hy, state, torch.cat([c.dec_proj for c in carries], 0), torch.cat([c.t_over for c in carries], 0), fst,
                          torch.cat([c.frame_offset for c in carries], 0))

    def split(self) -> "List[MALSDCarry]":
        out, K = [], self.hyps.K
        for b in range(self.hyps.B):
            hy = BatchedBeamHyps(1, K, self.hyps.max_len, self.hyps.tokens.device, self.hyps.blank)
            hy.max_len = self.hyps.max_len
            for name in ("tokens", "frames", "lengths", "scores", "hash", "prev_hash", "last_label"):
                setattr(hy, name, getattr(self.hyps, name)[b:b + 1].clone())
            state = None if self.state is None else [s[:, b * K:(b + 1) * K].clone() for s in self.state]
            out.append(MALSDCarry(hy, state, self.dec_proj[b * K:(b + 1) * K].clone(), self.t_over[b:b + 1].clone(),
                                  [f[b:b + 1].clone() for f in self.fstates], self.frame_offset[b:b + 1].clone()))
        return out


class ModifiedALSDBatchedComputer:
    """MALSD beam search for RNNT (``durations`` empty) and TDT.  Called with ``carry`` it continues a stream on its next chunk of
    encoder frames and leaves the new carry in ``self.carry`` (``rnnt_malsd_batched_computer.py`` ``ModifiedALSDBatchedRNNTComputer``
    called with a ``prev_batched_state``)."""

    def __init__(self, decoder, joint, blank_index: int, beam_size: int = 4, durations: Optional[List[int]] = None,
                 max_symbols_per_step: Optional[int] = 10, fusion_models=None, fusion_models_alpha=None,
                 blank_lm_score_mode: str = "no_score", pruning_mode: str = "late", score_norm: bool = True,
                 allow_cuda_graphs: bool = False, max_expansions: Optional[int] = None):
        self.decoder, self.joint = decoder, joint
        self.blank, self.K = blank_index, beam_size
        self.durations = list(durations or [])
        self.max_symbols = max_symbols_per_step or 10
        self.fusion_models = list(fusion_models or [])
        self.fusion_alphas = list(fusion_models_alpha or [])
        self.score_norm = score_norm
        self.max_exp = max_expansions or beam_size

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, out_len: torch.Tensor, carry: Optional[MALSDCarry] = None) -> BatchedBeamHyps:
        """x: [B, T, D_enc]; returns the final beam (of the whole stream so far when ``carry`` is given)."""
        B, T, _ = x.shape
        K, dev, dt = self.K, x.device, torch.float32
        enc = self.joint.project_encoder(x.to(dt))
        lin, act = self.joint.joint_net[-1], self.joint.joint_net[0]
        nd = len(self.durations)
        dur_t = torch.tensor(self.durations, device=dev, dtype=torch.long) if nd else None
        V1 = lin.out_features - nd
        out_len = out_len.to(dev)
        if carry is None:
            hyps = BatchedBeamHyps(B, K, init_length=T, device=dev, blank=self.blank)
            dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=B * K)
            state = [s for s in state] if state is not None else None
            dec_proj = self.joint.project_prednet(dec_out.to(dt))[:, 0]          # [B*K, H]
            t_idx = torch.zeros((B, K), dtype=torch.long, device=dev)
            fstates = [m.get_init_states(B * K, bos=True).view(B, K) for m in self.fusion_models]
            frame_offset = torch.zeros(B, dtype=torch.long, device=dev)
        else:
            hyps, state, dec_proj, t_idx = carry.hyps, carry.state, carry.dec_proj, carry.t_over.clone()
            fstates, frame_offset = list(carry.fstates), carry.frame_offset
        sym = torch.zeros((B, K), dtype=torch.long, device=dev)              # labels emitted on the current frame
        last_t = (out_len - 1).clamp(min=0).view(B, 1)
        bidx = torch.arange(B, device=dev).view(B, 1).expand(B, K)
        E = min(self.max_exp, V1 - 1)
        for _ in range(int(T) * (self.max_symbols + 1) + 1):
            active = (t_idx < out_len.view(B, 1)) & (hyps.scores > NEG / 2)
            if not bool(active.any()):
                break
            f = enc[bidx, torch.minimum(t_idx, last_t)]                        # [B,K,H]
            logits = torch.nn.functional.linear(act(f + dec_proj.view(B, K, -1)), lin.weight.to(dt), lin.bias.to(dt))
            lp_tok = torch.log_softmax(logits[..., :V1], dim=-1)
            lab_scores = lp_tok.clone()
            lab_scores[..., self.blank] = NEG
            fnext = []
            for m, a, st in zip(self.fusion_models, self.fusion_alphas, fstates):
                sc, nx = m.advance(st.reshape(-1))
                lab_scores[..., : self.blank] += a * sc.view(B, K, -1).to(dt)
                fnext.append(nx.view(B, K, -1))
            lab_scores = torch.where((sym >= self.max_symbols).unsqueeze(-1), torch.full_like(lab_scores, NEG), lab_scores)
            top_s, top_v = lab_scores.topk(E, dim=-1)                           # [B,K,E]
            blank_s = lp_tok[..., self.blank]
            if nd:
                lp_dur = torch.log_softmax(logits[..., V1:], dim=-1)           # [B,K,nd]
                # candidates: (label e, duration d) and (blank, duration d with 0 -> 1)
                cand_lab = (top_s.unsqueeze(-1) + lp_dur.unsqueeze(2)).reshape(B, K, E * nd)
                cand_lab_v = top_v.unsqueeze(-1).expand(-1, -1, -1, nd).reshape(B, K, E * nd)
                cand_lab_d = dur_t.view(1, 1, 1, nd).expand(B, K, E, nd).reshape(B, K, E * nd)
                bd = torch.where(dur_t == 0, torch.ones_like(dur_t), dur_t)
                cand_blk = blank_s.unsqueeze(-1) + lp_dur
                if (dur_t == 0).any() and (dur_t == 1).any():                  # duration 0 and 1 both mean "one frame" for blank
                    i0, i1 = int((dur_t == 0).nonzero()[0]), int((dur_t == 1).nonzero()[0])
                    merged = torch.logsumexp(torch.stack([cand_blk[..., i0], cand_blk[..., i1]]), dim=0)
                    cand_blk = cand_blk.clone()
                    cand_blk[..., i1] = merged
                    cand_blk[..., i0] = NEG
                cand_s = torch.cat([cand_lab, cand_blk], dim=-1)
                cand_v = torch.cat([cand_lab_v, torch.full((B, K, nd), self.blank, device=dev, dtype=torch.long)], dim=-1)
                cand_d = torch.cat([cand_lab_d, bd.view(1, 1, nd).expand(B, K, nd)], dim=-1)
            else:
                cand_s = torch.cat([top_s, blank_s.unsqueeze(-1)], dim=-1)
                cand_v = torch.cat([top_v, torch.full((B, K, 1), self.blank, device=dev, dtype=torch.long)], dim=-1)
                cand_d = (cand_v == self.blank).long()
            C = cand_s.shape[-1]
            total = hyps.scores.unsqueeze(-1) + cand_s
            total = torch.where(active.unsqueeze(-1), total, torch.full_like(total, NEG))
            # finished entries compete with their own score through one "stay" candidate
            stay = torch.where(active, torch.full_like(hyps.scores, NEG), hyps.scores)
            flat = torch.cat([total.reshape(B, K * C), stay], dim=1)
            best_s, best_i = flat.topk(K, dim=1)
            is_stay = best_i >= K * C
            src = torch.where(is_stay, best_i - K * C, best_i // C)
            ci = torch.where(is_stay, torch.zeros_like(best_i), best_i % C)
            pick = lambda a: a.gather(1, (src * C + ci).clamp(max=K * C - 1))  # noqa: E731
            lab = torch.where(is_stay, torch.full_like(src, -1), pick(cand_v.reshape(B, K * C)))
            dur = torch.where(is_stay, torch.zeros_like(src), pick(cand_d.reshape(B, K * C)))
            emitted = (lab >= 0) & (lab != self.blank)
            old_t = t_idx.gather(1, src)
            hyps.reorder_and_extend(src, lab, old_t + frame_offset.view(B, 1), best_s)
            t_idx = old_t + dur
            sym = torch.where(dur > 0, torch.zeros_like(sym), sym.gather(1, src) + emitted.long())
            # prediction network: entries that emitted a label advance, the others keep the state of their source
            flat_src = (torch.arange(B, device=dev).view(B, 1) * K + src).reshape(-1)
            if state is not None:
                state = [s.index_select(1, flat_src) for s in state]
            dec_proj = dec_proj.index_select(0, flat_src)
            emb_in = torch.where(emitted, lab, torch.full_like(lab, self.blank)).reshape(-1, 1)
            new_out, new_state = self.decoder.predict(emb_in, state=state, add_sos=False, batch_size=B * K)
            new_proj = self.joint.project_prednet(new_out.to(dt))[:, 0]
            em = emitted.reshape(-1)
            dec_proj = torch.where(em.unsqueeze(-1), new_proj, dec_proj)
            if state is not None:
                state = [torch.where(em.view(1, -1, 1), ns, s) for ns, s in zip(new_state, state)]
            for i in range(len(fstates)):
                st_src = fstates[i].gather(1, src)
                nx = fnext[i].gather(1, src.unsqueeze(-1).expand(-1, -1, fnext[i].shape[-1]))
                adv = nx.gather(2, lab.clamp(min=0, max=self.blank - 1).unsqueeze(-1)).squeeze(-1)
                fstates[i] = torch.where(emitted, adv, st_src)
            hyps.recombine(extra_key=t_idx)
        self.final_t = t_idx
        self.carry = MALSDCarry(hyps, state, dec_proj, (t_idx - out_len.view(B, 1)).clamp(min=0), fstates, frame_offset + out_len)
        return hyps


class ModifiedAESBatchedComputer:
    """Batched modified adaptive expansion search (mAES) for plain RNNT (reference ``rnnt_maes_batched_computer.py:30-370``,
    after Kim et al., "Accelerating RNN transducer inference via adaptive expansion search").

    The search is time synchronous: every beam entry of an utterance sits on the same frame.  On each frame the beam is
    expanded ``maes_num_steps`` times.  One expansion takes the ``beam_size + maes_expansion_beta`` best tokens (blank
    included) of every entry that has not taken blank on this frame yet, drops the candidates more than
    ``maes_expansion_gamma`` below that entry's best candidate, removes candidates that spell the same transcript, and
    keeps the best ``beam_size`` of the candidates and of the entries already closed on this frame.  Entries still open
    after the last expansion are closed with a forced blank.  Before the expansions a *prefix search* adds to an entry
    the probability of reaching it from another beam entry that is its prefix by one token.
    """

    def __init__(self, decoder, joint, blank_index: int, beam_size: int = 4, maes_num_steps: int = 2, maes_expansion_beta: int = 2,
                 maes_expansion_gamma: float = 2.3, fusion_models=None, fusion_models_alpha=None, score_norm: bool = True,
                 durations=None, **_):
        if durations:
            raise ValueError("maes_batch decodes plain RNNT only; use malsd_batch for TDT models")
        if maes_num_steps < 1:
            raise ValueError("maes_num_steps must be at least 1")
        self.decoder, self.joint = decoder, joint
        self.blank, self.K = blank_index, beam_size
        self.steps, self.gamma = int(maes_num_steps), float(maes_expansion_gamma)
        self.E = beam_size + int(maes_expansion_beta)
        self.fusion_models = list(fusion_models or [])
        self.fusion_alphas = list(fusion_models_alpha or [])
        self.score_norm = score_norm

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, out_len: torch.Tensor) -> BatchedBeamHyps:
        B, T, _ = x.shape
        K, dev, dt = self.K, x.device, torch.float32
        enc = self.joint.project_encoder(x.to(dt))
        lin, act = self.joint.joint_net[-1], self.joint.joint_net[0]
        V1 = lin.out_features
        E = min(self.E, V1)
        hyps = BatchedBeamHyps(B, K, init_length=T, device=dev, blank=self.blank)
        dec_out, state = self.decoder.predict(None, state=None, add_sos=False, batch_size=B * K)
        state = [s for s in state] if state is not None else None
        dec_proj = self.joint.project_prednet(dec_out.to(dt))[:, 0]              # [B*K, H]
        out_len = out_len.to(dev)
        fstates = [m.get_init_states(B * K, bos=True).view(B, K) for m in self.fusion_models]
        brange = torch.arange(B, device=dev).view(B, 1)

        def logps_at(t):
            f = enc[:, min(t, T - 1)].unsqueeze(1)                                 # [B,1,H]
            logits = torch.nn.functional.linear(act(f + dec_proj.view(B, K, -1)), lin.weight.to(dt), lin.bias.to(dt))
            lp = torch.log_softmax(logits, dim=-1)
            nxt = []
            for m, a, st in zip(self.fusion_models, self.fusion_alphas, fstates):
                sc, nx = m.advance(st.reshape(-1))
                lp[..., : self.blank] += a * sc.view(B, K, -1).to(dt)
                nxt.append(nx.view(B, K, -1))
            return lp, nxt

        for t in range(int(T)):
            frame_on = (out_len > t).view(B, 1)
            alive = hyps.scores > NEG / 2
            open_ = frame_on & alive                                                # entries that may still emit on this frame
            if not bool(open_.any()):
                break
            lp, fnext = logps_at(t)
            # prefix search: entry j = entry i + [v]  =>  score_j (+)= score_i + log p_i(v)
            ext = (hyps.prev_hash.unsqueeze(1) == hyps.hash.unsqueeze(2)) & (hyps.lengths.unsqueeze(1) == hyps.lengths.unsqueeze(2) + 1)
            ext = ext & open_.unsqueeze(2) & open_.unsqueeze(1)                     # [b, i, j]
            via = hyps.scores.unsqueeze(2) + lp.gather(2, hyps.last_label.clamp(max=V1 - 1).unsqueeze(1).expand(B, K, K))
            via = via.masked_fill(~ext, NEG)
            hyps.scores = torch.where(open_, torch.logsumexp(torch.cat([hyps.scores.unsqueeze(1), via], dim=1), dim=1), hyps.scores)
            tvec = torch.full((B, K), t, device=dev, dtype=torch.long)
            for _ in range(self.steps):
                if not bool(open_.any()):
                    break
                top_s, top_v = lp.topk(E, dim=-1)                                   # [B,K,E]
                cand = hyps.scores.unsqueeze(-1) + top_s
                cand = cand.masked_fill(cand <= cand.max(dim=-1, keepdim=True).values - self.gamma, NEG)
                cand = cand.masked_fill(~open_.unsqueeze(-1), NEG)
                cand_lab = top_v
                # a closed entry competes unchanged through the last slot of its row
                closed = alive & ~open_
                cand[..., -1] = torch.where(closed, hyps.scores, cand[..., -1])
                cand_lab = cand_lab.clone()
                cand_lab[..., -1] = torch.where(closed, torch.full_like(top_v[..., -1], -1), cand_lab[..., -1])
                # duplicates: same transcript after the step and same open / closed status
                is_tok = (cand_lab >= 0) & (cand_lab != self.blank)
                new_hash = torch.where(is_tok, (hyps.hash.unsqueeze(-1) * _HASH_MUL + cand_lab + 1) % 2305843009213693951,
                                       hyps.hash.unsqueeze(-1).expand(B, K, E))
                key_h, key_o, sc = new_hash.reshape(B, K * E), is_tok.reshape(B, K * E), cand.reshape(B, K * E)
                same = (key_h.unsqueeze(2) == key_h.unsqueeze(1)) & (key_o.unsqueeze(2) == key_o.unsqueeze(1))
                live = sc > NEG / 2
                same = same & live.unsqueeze(1) & live.unsqueeze(2)
                better = same & ((sc.unsqueeze(1) > sc.unsqueeze(2)) |
                                 ((sc.unsqueeze(1) == sc.unsqueeze(2)) &
                                  (torch.arange(K * E, device=dev).view(1, 1, -1) < torch.arange(K * E, device=dev).view(1, -1, 1))))
                sc = sc.masked_fill(better.any(dim=2), NEG)                          # someone equal and better exists
                best_s, best_i = sc.topk(K, dim=1)
                src = best_i // E
                lab = cand_lab.reshape(B, K * E).gather(1, best_i)
                lab = torch.where(best_s > NEG / 2, lab, torch.full_like(lab, -1))
                emitted = (lab >= 0) & (lab != self.blank)
                was_open = open_.gather(1, src)
                hyps.reorder_and_extend(src, lab, tvec, best_s)
                flat_src = (brange * K + src).reshape(-1)
                if state is not None:
                    state = [s.index_select(1, flat_src) for s in state]
                dec_proj = dec_proj.index_select(0, flat_src)
                emb_in = torch.where(emitted, lab, torch.full_like(lab, self.blank)).reshape(-1, 1)
                new_out, new_state = self.decoder.predict(emb_in, state=state, add_sos=False, batch_size=B * K)
                new_proj = self.joint.project_prednet(new_out.to(dt))[:, 0]
                em = emitted.reshape(-1)
                dec_proj = torch.where(em.unsqueeze(-1), new_proj, dec_proj)
                if state is not None:
                    state = [torch.where(em.view(1, -1, 1), ns, s) for ns, s in zip(new_state, state)]
                for i in range(len(fstates)):
                    st_src = fstates[i].gather(1, src)
                    nx = fnext[i].gather(1, src.unsqueeze(-1).expand(-1, -1, fnext[i].shape[-1]))
                    adv = nx.gather(2, lab.clamp(min=0, max=self.blank - 1).unsqueeze(-1)).squeeze(-1)
                    fstates[i] = torch.where(emitted, adv, st_src)
                alive = hyps.scores > NEG / 2
                open_ = was_open & emitted & alive
                lp, fnext = logps_at(t)
            if bool(open_.any()):
                hyps.scores = torch.where(open_, hyps.scores + lp[..., self.blank], hyps.scores)
            hyps.recombine()
        return hyps


class BatchedBeamCTCComputer:
    """Prefix beam search over CTC log-probabilities for a whole batch at once."""

    def __init__(self, blank_index: int, beam_size: int = 4, beam_beta: float = 0.0, beam_threshold: float = 20.0,
                 fusion_models=None, fusion_models_alpha=None, allow_cuda_graphs: bool = False):
        self.blank, self.K = blank_index, beam_size
        self.beta, self.threshold = beam_beta, beam_threshold
        self.fusion_models = list(fusion_models or [])
        self.fusion_alphas = list(fusion_models_alpha or [])

    @torch.no_grad()
    def __call__(self, log_probs: torch.Tensor, lengths: torch.Tensor) -> BatchedBeamHyps:
        """log_probs: [B, T, V+1]."""
        B, T, V1 = log_probs.shape
        K, dev = self.K, log_probs.device
        lp_all = log_probs.float()
        hyps = BatchedBeamHyps(B, K, init_length=T, device=dev, blank=self.blank)
        pb = hyps.scores.clone()                                   # prefix ends in blank
        pnb = torch.full_like(pb, NEG)                             # prefix ends in its last label
        lm_acc = torch.zeros_like(pb)
        fstates = [m.get_init_states(B * K, bos=True).view(B, K) for m in self.fusion_models]
        lengths = lengths.to(dev)
        tok_ids = torch.arange(V1, device=dev)
        for t in range(T):
            live = (t < lengths).view(B, 1)
            lp = lp_all[:, t].unsqueeze(1).expand(B, K, V1)
            tot = torch.logaddexp(pb, pnb)
            last = hyps.last_label
            lm_bonus = torch.zeros((B, K, V1), device=dev)
            fnext = []
            for m, a, st in zip(self.fusion_models, self.fusion_alphas, fstates):
                sc, nx = m.advance(st.reshape(-1))
                lm_bonus[..., : self.blank] += a * sc.view(B, K, -1)
                fnext.append(nx.view(B, K, -1))
            # stay: blank, or repeat of the last label (no new token)
            stay_pb = tot + lp[..., self.blank]
            stay_pnb = torch.where(last != self.blank, pnb + lp.gather(2, last.clamp(max=V1 - 1).unsqueeze(-1)).squeeze(-1),
                                   torch.full_like(pnb, NEG))
            # extend by v: after a blank anything goes; directly after label `last` only v != last
            same = tok_ids.view(1, 1, V1) == last.unsqueeze(-1)
            ext = torch.where(same, pb.unsqueeze(-1), tot.unsqueeze(-1)) + lp
            ext[..., self.blank] = NEG
            ext_rank = ext + lm_bonus + self.beta
            valid = hyps.scores > NEG / 2
            ext_rank = torch.where(valid.unsqueeze(-1), ext_rank, torch.full_like(ext_rank, NEG))
            stay_rank = torch.where(valid, torch.logaddexp(stay_pb, stay_pnb) + lm_acc, torch.full_like(pb, NEG))
            flat = torch.cat([ext_rank.reshape(B, K * V1) + lm_acc.repeat_interleave(V1, dim=1), stay_rank], dim=1)
            best_s, best_i = flat.topk(K, dim=1)
            is_stay = best_i >= K * V1
            src = torch.where(is_stay, best_i - K * V1, best_i // V1)
            lab = torch.where(is_stay, torch.full_like(src, -1), best_i % V1)
            g = lambda a: a.gather(1, src)  # noqa: E731
            ext_sel = ext.reshape(B, K * V1).gather(1, best_i.clamp(max=K * V1 - 1))
            bonus_sel = lm_bonus.reshape(B, K * V1).gather(1, best_i.clamp(max=K * V1 - 1))
            new_pb = torch.where(is_stay, g(stay_pb), torch.full_like(pb, NEG))
            new_pnb = torch.where(is_stay, g(stay_pnb), ext_sel)
            new_lm = torch.where(is_stay, g(lm_acc), g(lm_acc) + bonus_sel + self.beta)
            # frames past the end of an utterance leave its beam untouched
            keep_src = torch.arange(K, device=dev).view(1, K).expand(B, K)
            src = torch.where(live, src, keep_src)
            lab = torch.where(live, lab, torch.full_like(lab, -1))
            new_pb = torch.where(live, new_pb, pb)
            new_pnb = torch.where(live, new_pnb, pnb)
            new_lm = torch.where(live, new_lm, lm_acc)
            score = torch.where(torch.maximum(new_pb, new_pnb) > NEG / 2, torch.logaddexp(new_pb, new_pnb) + new_lm,
                                torch.full_like(pb, NEG))
            score = torch.where(live, torch.where(best_s > NEG / 2, score, torch.full_like(score, NEG)), hyps.scores)
            hyps.reorder_and_extend(src, lab, torch.full_like(src, t), score)
            for i in range(len(fstates)):
                st_src = fstates[i].gather(1, src)
                nx = fnext[i].gather(1, src.unsqueeze(-1).expand(-1, -1, fnext[i].shape[-1]))
                adv = nx.gather(2, lab.clamp(min=0, max=self.blank - 1).unsqueeze(-1)).squeeze(-1)
                fstates[i] = torch.where(lab >= 0, adv, st_src)
            pb, pnb, lm_acc = new_pb, new_pnb, new_lm
            # equal prefixes reached along different paths: add their probabilities
            same_h = (hyps.hash.unsqueeze(2) == hyps.hash.unsqueeze(1)) & (hyps.lengths.unsqueeze(2) == hyps.lengths.unsqueeze(1))
            ok = hyps.scores > NEG / 2
            same_h = same_h & ok.unsqueeze(1) & ok.unsqueeze(2)
            order = torch.arange(K, device=dev)
            is_dup = (same_h & (order.view(1, 1, K) < order.view(1, K, 1))).any(dim=2)
            fold = lambda a: torch.logsumexp(a.unsqueeze(1).expand(-1, K, -1).masked_fill(~same_h, NEG), dim=2)  # noqa: E731
            pb = torch.where(is_dup, torch.full_like(pb, NEG), torch.where(ok, fold(pb), pb))
            pnb = torch.where(is_dup, torch.full_like(pnb, NEG), torch.where(ok, fold(pnb), pnb))
            hyps.scores = torch.where(is_dup | ~ok, torch.full_like(pb, NEG), torch.logaddexp(pb, pnb) + lm_acc)
        return hyps

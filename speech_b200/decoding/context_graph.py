"""Context graphs on the host: the phrase automaton used for shallow-fusion biasing inside beam searches that run on the CPU, the
CTC-topology graph used by word spotting, and the merge of spotted phrases into a greedy transcript.

* ``ContextGraph`` — a trie over the token sequences of the bias phrases with Aho-Corasick failure links.  ``forward_one_step(state,
  token)`` returns the score increment and the next state: matching a token of a phrase earns ``context_score`` (per phrase scores
  allowed), leaving a partly matched phrase takes back what was earned (so only completed phrases keep their boost), a completed
  phrase keeps it.  ``finalize(state)`` takes back the boost of a phrase left unfinished at the end of the utterance.
* ``CTCContextGraph`` — the same phrases with CTC topology (optional blank between tokens, self-loops), flattened into arrays
  for token-passing search.
* ``merge_alignment_with_ws_hyps`` — replaces the words of a greedy CTC alignment that overlap a spotted phrase by the phrase.

References: ``asr/parts/context_biasing/context_graph_universal.py`` (``ContextGraph``), ``context_graph_ctc.py``,
``context_biasing_utils.py`` (``merge_alignment_with_ws_hyps``).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

__all__ = ["CTCContextGraph", "ContextGraph", "ContextState", "merge_alignment_with_ws_hyps"]


@dataclass
class ContextState:
    id: int
    token: int
    token_score: float                    # score of the arc that enters this state
    node_score: float                     # sum of the arc scores from the root to here
    output_score: float                   # boost of the longest phrase that ends here or on the failure path (0 when none)
    is_end: bool
    level: int
    phrase: str = ""
    next: Dict[int, "ContextState"] = field(default_factory=dict)
    fail: Optional["ContextState"] = None
    output: Optional["ContextState"] = None


class ContextGraph:
    def __init__(self, context_score: float, depth_scaling: float = 1.0, ac_threshold: float = 1.0):
        """``depth_scaling``: the score of an arc at depth d is ``context_score * depth_scaling ** (d - 1)`` (> 1 favours long phrases);
        ``ac_threshold`` is kept with a finished phrase for acoustic re-checks by the caller."""
        self.context_score, self.depth_scaling, self.ac_threshold = context_score, depth_scaling, ac_threshold
        self.num_nodes = 0
        self.root = self._new(-1, 0.0, 0.0, False, 0)
        self.root.fail = self.root

    def _new(self, token, token_score, node_score, is_end, level, phrase="") -> ContextState:
        st = ContextState(self.num_nodes, token, token_score, node_score, node_score if is_end else 0.0, is_end, level, phrase)
        self.num_nodes += 1
        return st

    def build(self, token_ids: Sequence[Sequence[int]], phrases: Optional[Sequence[str]] = None, scores: Optional[Sequence[float]] = None,
              uniform_weights: bool = False) -> "ContextGraph":
        """``scores[i]`` replaces ``context_score`` for phrase i (0 = default).  ``uniform_weights`` spreads a phrase's total score
        evenly over its arcs instead of scaling by depth."""
        for i, toks in enumerate(token_ids):
            node = self.root
            base = scores[i] if scores is not None and scores[i] else self.context_score
            for d, t in enumerate(toks, 1):
                t = int(t)
                if t not in node.next:
                    s = base if uniform_weights else base * self.depth_scaling ** (d - 1)
                    node.next[t] = self._new(t, s, node.node_score + s, False, d)
                node = node.next[t]
            node.is_end = True
            node.output_score = node.node_score
            node.phrase = phrases[i] if phrases is not None else " ".join(map(str, toks))
        self._fill_fail_output()
        return self

    def _fill_fail_output(self):
        q = deque()
        for n in self.root.next.values():
            n.fail = self.root
            q.append(n)
        while q:
            cur = q.popleft()
            for t, nxt in cur.next.items():
                f = cur.fail
                while f is not self.root and t not in f.next:
                    f = f.fail
                nxt.fail = f.next[t] if t in f.next and f.next[t] is not nxt else self.root
                # the nearest phrase end on the failure path: reaching this state also completes that phrase
                o = nxt.fail
                while o is not self.root and not o.is_end:
                    o = o.fail
                nxt.output = o if o.is_end else None
                if not nxt.is_end and nxt.output is not None:
                    nxt.output_score = nxt.output.node_score
                q.append(nxt)

    def forward_one_step(self, state: ContextState, token: int, strict_mode: bool = True) -> Tuple[float, ContextState, Optional[ContextState]]:
        """-> ``(score increment, next state, phrase-end state matched by this step or None)``.  ``strict_mode`` False lets a
        completed phrase restart from the root without losing its boost (phrases that may repeat back to back)."""
        token = int(token)
        if token in state.next:
            nxt = state.next[token]
            score = nxt.token_score
        else:
            f = state.fail
            while f is not self.root and token not in f.next:
                f = f.fail
            nxt = f.next[token] if token in f.next else self.root
            kept = state.node_score if (state.is_end and not strict_mode) else (state.output_score if not state.is_end else state.node_score)
            # what was earned on the abandoned path is returned, except the part that belongs to a completed phrase
            score = nxt.node_score - state.node_score + (kept if state.is_end or state.output_score else 0.0)
        matched = nxt if nxt.is_end else nxt.output
        return score, nxt, matched

    def finalize(self, state: ContextState) -> Tuple[float, ContextState]:
        """End of the utterance: an unfinished phrase gives its boost back."""
        if state.is_end:
            return 0.0, self.root
        return -(state.node_score - state.output_score), self.root

    def score_sequence(self, tokens: Sequence[int]) -> Tuple[float, List[str]]:
        """Total boost of a finished token sequence and the phrases found in it."""
        st, total, found = self.root, 0.0, []
        for t in tokens:
            s, st, m = self.forward_one_step(st, t)
            total += s
            if m is not None:
                found.append(m.phrase)
        s, _ = self.finalize(st)
        return total + s, found


class CTCContextGraph:
    """Phrases with CTC topology as flat arrays: state 2k is "before token k" (blank self-loop), state 2k+1 is "in token k"
    (token self-loop); arcs 2k -> 2k+1, 2k+1 -> 2k+2 (blank) and 2k+1 -> 2k+3 when the next token differs.  ``search`` runs
    token passing over log-probabilities and returns, per phrase, the best ``(score per frame, start, end)`` ending at each frame
    above the threshold."""

    def __init__(self, phrases: Dict[str, Sequence[int]], blank: int):
        self.blank, self.names = blank, list(phrases)
        self.tokens = [list(map(int, phrases[n])) for n in self.names]

    def search(self, log_probs: np.ndarray, threshold: float = -3.0, blank_weight: float = 0.5) -> List[Tuple[str, float, int, int]]:
        lp = np.asarray(log_probs, dtype=np.float64)
        T = lp.shape[0]
        out: List[Tuple[str, float, int, int]] = []
        NEG = -1e30
        for name, toks in zip(self.names, self.tokens):
            n = len(toks)
            if not n:
                continue
            sc = np.full(n, NEG)
            st = np.zeros(n, dtype=np.int64)
            tok = np.asarray(toks)
            for t in range(T):
                emit = lp[t, tok]
                stay = np.where(sc > NEG, sc + np.maximum(emit, lp[t, self.blank] * blank_weight), NEG)
                adv = np.full(n, NEG)
                adv_st = np.zeros(n, dtype=np.int64)
                adv[0], adv_st[0] = emit[0], t
                if n > 1:
                    ok = sc[:-1] > NEG
                    adv[1:] = np.where(ok, sc[:-1] + emit[1:], NEG)
                    adv_st[1:] = st[:-1]
                take = adv > stay
                # a hit must END on a frame that emits the last token
                end_score = max(adv[-1], sc[-1] + emit[-1] if sc[-1] > NEG else NEG)
                end_start = adv_st[-1] if adv[-1] >= (sc[-1] + emit[-1] if sc[-1] > NEG else NEG) else st[-1]
                sc, st = np.where(take, adv, stay), np.where(take, adv_st, st)
                if end_score > NEG:
                    avg = end_score / (t - end_start + 1)
                    if avg >= threshold:
                        out.append((name, float(avg), int(end_start), t))
        out.sort(key=lambda h: -h[1])
        kept: List[Tuple[str, float, int, int]] = []
        for h in out:
            if all(h[3] < k[2] or h[2] > k[3] for k in kept):
                kept.append(h)
        return sorted(kept, key=lambda h: h[2])


def merge_alignment_with_ws_hyps(alignment: Sequence[int], ws_hyps: Sequence, id_to_token, blank: int, word_boundary: str = "▁",
                                 print_stats: bool = False) -> Tuple[str, List[Tuple[str, int, int]]]:
    """``alignment``: the frame-level greedy CTC labels.  Words of the greedy transcript (with their frame spans) that overlap a
    spotted phrase — by at least half of the word's span — are dropped and the phrase takes their place.  ``ws_hyps`` items have
    ``word``, ``start_frame``, ``end_frame`` (and ``score``).  Returns the text and the final ``(word, start, end)`` list."""
    words: List[Tuple[str, int, int]] = []
    cur, start, prev = "", 0, blank
    last = 0
    for t, a in enumerate(list(alignment) + [blank]):
        a = int(a)
        if a != blank and a != prev:
            piece = id_to_token(a)
            if piece.startswith(word_boundary) or not cur:
                if cur:
                    words.append((cur, start, last))
                cur, start = piece.lstrip(word_boundary), t
            else:
                cur += piece
        if a != blank:
            last = t
        prev = a
    if cur:
        words.append((cur, start, last))
    hyps = sorted(ws_hyps, key=lambda h: h.start_frame)
    used = [False] * len(words)
    merged: List[Tuple[str, int, int]] = []
    for h in hyps:
        for i, (w, a, b) in enumerate(words):
            inter = min(b, h.end_frame) - max(a, h.start_frame) + 1
            if inter > 0 and inter >= 0.5 * (b - a + 1):
                used[i] = True
        merged.append((h.word, h.start_frame, h.end_frame))
    merged += [w for w, u in zip(words, used) if not u]
    merged.sort(key=lambda x: x[1])
    if print_stats:
        print(f"{sum(used)} greedy words replaced by {len(hyps)} spotted phrases")
    return " ".join(w for w, _, _ in merged), merged

"""Lexicon-constrained CTC beam search with a word-level n-gram language model, and the same search driven by a compiled
token-lexicon graph (the "TL" part of a TLG decoding graph).

This is what the reference reaches through external C++ packages: the flashlight lexicon decoder and the Riva WFST decoder
(``parts/submodules/ctc_beam_decoding.py`` ``flashlight_beam_search`` / ``pyctcdecode``; ``parts/submodules/wfst_decoder.py``
``RivaGpuWfstDecoder``).  Here the search is written out:

* ``LexiconTrie`` — token-sequence trie of the lexicon (several spellings per word allowed); a path from the root to a node
  with words attached spells those words.
* ``WordNGramLM`` — back-off n-gram model over words read from an ARPA file (log10 -> natural log), with ``score(history, word)``.
* ``LexiconCTCBeamDecoder`` — prefix beam search over CTC posteriors where every hypothesis sits at a trie node: tokens that do
  not continue a lexicon word are pruned, a word is emitted when its last token is left (at the next non-continuing token or
  at the end), and emission adds ``lm_weight * log P(word | history) + word_score``.  Blank / repeat handling is the usual
  two-probability (ending in blank / ending in non-blank) recursion, merged per (trie node, last token, word history).
  ``unk_score`` lets out-of-lexicon spellings through as ``<unk>`` when finite.
* ``compile_lexicon_graph`` — the same lexicon as explicit arcs ``(state, token, next_state, word_or_None)``: a deterministic
  token-to-word transducer that ``LexiconCTCBeamDecoder`` can also run on (``graph=...``), which is the form a WFST tool chain
  exports and imports (OpenFst text format writer / reader included).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .ngram_lm import _parse_arpa

_LN10 = math.log(10.0)
NEG_INF = float("-inf")


def _logadd(a: float, b: float) -> float:
    if a == NEG_INF:
        return b
    if b == NEG_INF:
        return a
    m = max(a, b)
    return m + math.log1p(math.exp(-abs(a - b)))


class LexiconTrie:
    def __init__(self, lexicon: Dict[str, Iterable[Sequence[int]]]):
        self.children: List[Dict[int, int]] = [{}]
        self.words: List[List[str]] = [[]]
        for word, spellings in lexicon.items():
            for sp in spellings:
                node = 0
                for t in sp:
                    nxt = self.children[node].get(int(t))
                    if nxt is None:
                        nxt = len(self.children)
                        self.children[node][int(t)] = nxt
                        self.children.append({})
                        self.words.append([])
                    node = nxt
                if word not in self.words[node]:
                    self.words[node].append(word)

    @classmethod
    def from_tokenizer(cls, words: Iterable[str], tokenizer) -> "LexiconTrie":
        return cls({w: [tokenizer.text_to_ids(w)] for w in words})

    def step(self, node: int, token: int) -> Optional[int]:
        return self.children[node].get(token)


class WordNGramLM:
    def __init__(self, order: int, ngrams: Dict[Tuple[str, ...], Tuple[float, float]], unk: str = "<unk>"):
        self.order, self.ng, self.unk = order, ngrams, unk

    @classmethod
    def from_arpa(cls, path: str) -> "WordNGramLM":
        order, ngrams = _parse_arpa(path)
        return cls(order, ngrams)

    def score(self, history: Tuple[str, ...], word: str) -> float:
        """Natural-log P(word | history) with back-off."""
        if (word,) not in self.ng:
            word = self.unk
            if (word,) not in self.ng:
                return -100.0 * _LN10
        h = tuple(history[-(self.order - 1):]) if self.order > 1 else ()
        bo = 0.0
        while True:
            hit = self.ng.get(h + (word,))
            if hit is not None:
                return (hit[0] + bo) * _LN10
            if not h:
                return -100.0 * _LN10
            bo += self.ng.get(h, (0.0, 0.0))[1]
            h = h[1:]


def compile_lexicon_graph(trie: LexiconTrie) -> List[Tuple[int, int, int, Optional[str]]]:
    """Arcs (state, token, next_state, word): consuming ``token`` in ``state``.  A word label sits on the arc that LEAVES the
    word's last node back through the root, i.e. ``(node_with_word, t, root.step(t), word)`` for every token ``t`` that starts a
    word, next to the plain continuation arcs of the trie."""
    arcs: List[Tuple[int, int, int, Optional[str]]] = []
    starts = trie.children[0]
    for s, ch in enumerate(trie.children):
        for t, n in ch.items():
            arcs.append((s, t, n, None))
        for w in trie.words[s]:
            for t, n in starts.items():
                arcs.append((s, t, n, w))
    return arcs


def write_openfst_text(arcs: Sequence[Tuple[int, int, int, Optional[str]]], final_states: Iterable[int], path: str, eps: str = "<eps>") -> None:
    with open(path, "w", encoding="utf-8") as f:
        for s, t, n, w in arcs:
            f.write(f"{s}\t{n}\t{t}\t{w if w is not None else eps}\n")
        for s in sorted(set(final_states)):
            f.write(f"{s}\n")


def read_openfst_text(path: str, eps: str = "<eps>"):
    arcs, finals = [], []
    with open(path, encoding="utf-8") as f:
        for line in f:
            p = line.split()
            if len(p) >= 4:
                arcs.append((int(p[0]), int(p[2]), int(p[1]), None if p[3] == eps else p[3]))
            elif len(p) == 1:
                finals.append(int(p[0]))
    return arcs, finals


@dataclass
class _Hyp:
    p_b: float = NEG_INF           # log prob of all alignments of this prefix that end in blank
    p_nb: float = NEG_INF          # ... that end in the last token
    lm: float = 0.0                # accumulated LM + word-insertion score
    words: Tuple[str, ...] = ()
    word_frames: Tuple[int, ...] = ()

    @property
    def total(self) -> float:
        return _logadd(self.p_b, self.p_nb) + self.lm


@dataclass
class LexiconBeamResult:
    words: List[str]
    score: float
    word_frames: List[int] = field(default_factory=list)

    @property
    def text(self) -> str:
        return " ".join(self.words)


class LexiconCTCBeamDecoder:
    def __init__(self, trie: LexiconTrie, blank_id: int, lm: Optional[WordNGramLM] = None, beam_size: int = 16, lm_weight: float = 1.0,
                 word_score: float = 0.0, unk_score: float = NEG_INF, token_beam: int = 0, beam_threshold: float = 25.0,
                 graph: Optional[Sequence[Tuple[int, int, int, Optional[str]]]] = None):
        self.trie, self.blank, self.lm = trie, int(blank_id), lm
        self.beam, self.lmw, self.ws, self.unk = beam_size, lm_weight, word_score, unk_score
        self.token_beam, self.threshold = token_beam, beam_threshold
        # per state: token -> list of (next_state, emitted word or None)
        self.next: List[Dict[int, List[Tuple[int, Optional[str]]]]] = []
        if graph is None:
            graph = compile_lexicon_graph(trie)
        n_states = max([0] + [max(a[0], a[2]) for a in graph]) + 1
        self.next = [dict() for _ in range(n_states)]
        for s, t, n, w in graph:
            self.next[s].setdefault(t, []).append((n, w))
        self.final_words = [list(ws) for ws in trie.words] + [[] for _ in range(n_states - len(trie.words))]

    def _emit(self, h: _Hyp, word: str, frame: int) -> Tuple[float, Tuple[str, ...], Tuple[int, ...]]:
        s = self.ws + (self.lmw * self.lm.score(h.words, word) if self.lm is not None else 0.0)
        return h.lm + s, h.words + (word,), h.word_frames + (frame,)

    def decode(self, log_probs, length: Optional[int] = None, n_best: int = 1) -> List[LexiconBeamResult]:
        lp = np.asarray(log_probs.detach().float().cpu() if hasattr(log_probs, "detach") else log_probs, dtype=np.float64)
        T = int(length) if length is not None else lp.shape[0]
        # key: (state, last token, words)
        beams: Dict[Tuple[int, int, Tuple[str, ...]], _Hyp] = {(0, -1, ()): _Hyp(p_b=0.0)}
        for t in range(T):
            row = lp[t]
            cand = np.argsort(row)[::-1][: self.token_beam] if self.token_beam else np.arange(row.shape[0])
            new: Dict[Tuple[int, int, Tuple[str, ...]], _Hyp] = {}

            def put(key, p_b, p_nb, lm, words, frames):
                h = new.get(key)
                if h is None:
                    new[key] = _Hyp(p_b, p_nb, lm, words, frames)
                else:
                    h.p_b, h.p_nb = _logadd(h.p_b, p_b), _logadd(h.p_nb, p_nb)
            for (state, last, words), h in beams.items():
                tot = _logadd(h.p_b, h.p_nb)
                # blank: stay
                put((state, last, words), tot + row[self.blank], NEG_INF, h.lm, h.words, h.word_frames)
                # repeat of the last token without an intervening blank: same prefix
                if last >= 0 and h.p_nb > NEG_INF:
                    put((state, last, words), NEG_INF, h.p_nb + row[last], h.lm, h.words, h.word_frames)
                for tok in cand:
                    tok = int(tok)
                    if tok == self.blank:
                        continue
                    base = h.p_b if tok == last else tot      # a repeated token extends the prefix only after a blank
                    if base == NEG_INF:
                        continue
                    for nxt, w in self.next[state].get(tok, ()):  # continuation inside a word, or leave a finished word
                        if w is None:
                            put((nxt, tok, words), NEG_INF, base + row[tok], h.lm, h.words, h.word_frames)
                        else:
                            lm, ws, fr = self._emit(h, w, t)
                            put((nxt, tok, ws), NEG_INF, base + row[tok], lm, ws, fr)
            if not new:
                break
            ranked = sorted(new.items(), key=lambda kv: kv[1].total, reverse=True)
            best = ranked[0][1].total
            beams = dict((k, v) for k, v in ranked[: self.beam] if v.total >= best - self.threshold)
        # flush: a hypothesis must end on a node that spells a word (or at the root)
        final: Dict[Tuple[str, ...], Tuple[float, Tuple[int, ...]]] = {}
        for (state, last, words), h in beams.items():
            outs = []
            if state == 0:
                outs.append((h.total, h.words, h.word_frames))
            for w in self.final_words[state] if state < len(self.final_words) else []:
                lm, ws, fr = self._emit(h, w, T)
                outs.append((_logadd(h.p_b, h.p_nb) + lm, ws, fr))
            if not outs and self.unk > NEG_INF:
                outs.append((h.total + self.unk, h.words + ("<unk>",), h.word_frames + (T,)))
            for sc, ws, fr in outs:
                if self.lm is not None:
                    sc += self.lmw * self.lm.score(ws, "</s>")
                if ws not in final or final[ws][0] < sc:
                    final[ws] = (sc, fr)
        res = sorted(((sc, ws, fr) for ws, (sc, fr) in final.items()), key=lambda x: x[0], reverse=True)[:n_best]
        return [LexiconBeamResult(list(ws), float(sc), list(fr)) for sc, ws, fr in res]

    def decode_batch(self, log_probs, lengths) -> List[LexiconBeamResult]:
        out = []
        for b in range(log_probs.shape[0]):
            r = self.decode(log_probs[b], int(lengths[b]))
            out.append(r[0] if r else LexiconBeamResult([], NEG_INF))
        return out

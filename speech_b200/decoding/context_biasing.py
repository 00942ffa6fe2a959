"""Phrase boosting ("context biasing") for batched greedy / beam decoding.

``GPUBoostingTreeModel`` turns a list of tokenised phrases into an Aho-Corasick automaton in the same flat back-off form as
the n-gram LM (``ngram_lm.BackoffGraph``), so decoders call the same ``advance(states) -> (scores[B,V], next_states[B,V])``:

* following a phrase token earns ``context_score`` (scaled by ``depth_scaling`` per depth),
* leaving a partially matched phrase through a failure link gives back what the unfinished part earned,
* completing a phrase keeps its reward (optionally ``score_per_phrase`` on top).
``GPUBiasingMultiModel`` holds several trees and lets every stream of a batch pick its own (per-stream biasing).
Reference: ``parts/context_biasing/boosting_graph_batched.py:271``, ``biasing_multi_model.py:279``,
``context_graph_universal.py``; the CTC word spotter is ``ctc_word_spotter`` below.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .ngram_lm import BackoffGraph


@dataclass
class BoostingTreeModelConfig:
    key_phrases_file: Optional[str] = None
    key_phrases_list: Optional[List[str]] = None
    context_score: float = 1.0
    depth_scaling: float = 1.0
    unk_score: float = 0.0
    final_eos_score: float = 0.0
    score_per_phrase: float = 0.0
    source_lang: str = "en"
    use_triton: bool = False
    uniform_weights: bool = False
    use_bpe_dropout: bool = False
    num_of_transcriptions: int = 5
    bpe_alpha: float = 0.3


class _Node:
    __slots__ = ("children", "fail", "token_score", "node_score", "is_end", "depth", "id")

    def __init__(self, idx: int, depth: int):
        self.children: Dict[int, "_Node"] = {}
        self.fail: Optional["_Node"] = None
        self.token_score = 0.0
        self.node_score = 0.0
        self.is_end = False
        self.depth = depth
        self.id = idx


def build_boosting_arcs(phrases: Sequence[Sequence[int]], context_score: float = 1.0, depth_scaling: float = 1.0,
                        score_per_phrase: float = 0.0):
    root = _Node(0, 0)
    nodes = [root]
    for ph in phrases:
        cur = root
        for d, t in enumerate(ph):
            nx = cur.children.get(int(t))
            if nx is None:
                nx = _Node(len(nodes), d + 1)
                nx.token_score = context_score * (depth_scaling ** d)
                nx.node_score = cur.node_score + nx.token_score
                nodes.append(nx)
                cur.children[int(t)] = nx
            cur = nx
        if cur is not root:
            if not cur.is_end:
                cur.token_score += score_per_phrase
                cur.node_score += score_per_phrase
            cur.is_end = True
    # failure links (breadth first)
    q = deque()
    for ch in root.children.values():
        ch.fail = root
        q.append(ch)
    while q:
        n = q.popleft()
        for t, ch in n.children.items():
            f = n.fail
            while f is not None and t not in f.children:
                f = f.fail
            ch.fail = f.children[t] if f is not None and t in f.children else root
            if ch.fail is ch:
                ch.fail = root
            q.append(ch)
    # a completed phrase keeps its reward: nothing is owed when leaving an end node
    local = [0.0 if n.is_end else n.node_score for n in nodes]
    arcs, bw, bt = [], [0.0] * len(nodes), [0] * len(nodes)
    for n in nodes:
        for t, ch in n.children.items():
            arcs.append((n.id, t, ch.token_score, ch.id))
        if n is not root:
            bw[n.id] = local[n.fail.id] - local[n.id]
            bt[n.id] = n.fail.id
    max_depth = max(n.depth for n in nodes) + 1
    return arcs, bw, bt, max_depth


class GPUBoostingTreeModel(BackoffGraph):
    def __init__(self, vocab_size: int, phrases: Sequence[Sequence[int]], context_score: float = 1.0,
                 depth_scaling: float = 1.0, score_per_phrase: float = 0.0, unk_score: float = 0.0):
        arcs, bw, bt, depth = build_boosting_arcs(phrases, context_score, depth_scaling, score_per_phrase)
        super().__init__(vocab_size, arcs, bw, bt, max_depth=depth, default_score=unk_score)
        self.phrases = [list(map(int, p)) for p in phrases]

    @classmethod
    def from_config(cls, cfg, tokenizer=None, vocab_size: Optional[int] = None) -> "GPUBoostingTreeModel":
        get = (lambda k, d=None: cfg.get(k, d)) if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        phrases: List[str] = list(get("key_phrases_list") or [])
        if get("key_phrases_file"):
            with open(get("key_phrases_file"), encoding="utf-8") as f:
                phrases += [l.strip() for l in f if l.strip()]
        if tokenizer is None:
            raise ValueError("a tokenizer is needed to turn key phrases into token sequences")
        toks = [tokenizer.text_to_ids(p) for p in phrases]
        V = vocab_size or getattr(tokenizer, "vocab_size", None) or len(tokenizer.vocab)
        return cls(V, toks, context_score=get("context_score", 1.0), depth_scaling=get("depth_scaling", 1.0),
                   score_per_phrase=get("score_per_phrase", 0.0), unk_score=get("unk_score", 0.0))

    def get_final(self, states: torch.Tensor) -> torch.Tensor:
        """At end of utterance an unfinished partial match gives its reward back."""
        out = torch.zeros(states.shape, dtype=torch.float32, device=states.device)
        cur = states
        for _ in range(self.max_depth):
            out = out + self.backoff_w[cur]
            cur = self.backoff_to[cur]
        return out


class GPUBiasingMultiModel(torch.nn.Module):
    """Several boosting trees side by side; ``model_ids[B]`` selects the tree of each stream (-1 = none)."""

    def __init__(self, vocab_size: int):
        super().__init__()
        self.vocab_size = vocab_size
        self.models = torch.nn.ModuleList()
        self.alphas: List[float] = []
        self.free_ids: List[int] = []

    def add_model(self, model: GPUBoostingTreeModel, alpha: float = 1.0) -> int:
        if self.free_ids:
            i = self.free_ids.pop()
            self.models[i] = model
            self.alphas[i] = alpha
            return i
        self.models.append(model)
        self.alphas.append(alpha)
        return len(self.models) - 1

    def remove_model(self, model_id: int) -> None:
        self.models[model_id] = torch.nn.Identity()
        self.free_ids.append(model_id)

    def has_models(self) -> bool:
        return any(isinstance(m, GPUBoostingTreeModel) for m in self.models)

    def get_init_states(self, batch_size: int, bos: bool = True) -> torch.Tensor:
        dev = next((m.arc_keys.device for m in self.models if isinstance(m, GPUBoostingTreeModel)), None)
        return torch.zeros(batch_size, dtype=torch.long, device=dev)

    @torch.no_grad()
    def advance(self, states: torch.Tensor, model_ids: torch.Tensor):
        B = states.shape[0]
        scores = torch.zeros((B, self.vocab_size), dtype=torch.float32, device=states.device)
        nxt = torch.zeros((B, self.vocab_size), dtype=torch.long, device=states.device)
        for i, m in enumerate(self.models):
            if not isinstance(m, GPUBoostingTreeModel):
                continue
            sel = model_ids == i
            sc, nx = m.advance(torch.where(sel, states, torch.zeros_like(states)))
            scores = torch.where(sel[:, None], sc * self.alphas[i], scores)
            nxt = torch.where(sel[:, None], nx, nxt)
        return scores, nxt


@dataclass
class WordSpotterHyp:
    word: str
    score: float
    start_frame: int
    end_frame: int
    tokens: List[int] = field(default_factory=list)


def ctc_word_spotter(log_probs: torch.Tensor, phrases: Dict[str, Sequence[int]], blank: int, keyword_threshold: float = -3.0,
                     ctc_ali_token_weight: float = 0.5, beam_threshold: float = 7.0) -> List[WordSpotterHyp]:
    """Find occurrences of phrases in CTC log-probabilities ``[T, V]`` with a token-passing search over each phrase
    (reference: ``parts/context_biasing/ctc_based_word_spotter.py``).  The score of a hit is its mean per-frame
    log-probability; hits below ``keyword_threshold`` are dropped, overlapping hits keep the best."""
    lp = log_probs.detach().float().cpu()
    T = lp.shape[0]
    hits: List[WordSpotterHyp] = []
    for word, toks in phrases.items():
        toks = list(map(int, toks))
        n = len(toks)
        if n == 0:
            continue
        NEG = -1e30
        # score[k] = best path ending in token k at current frame; start[k] its start frame; frames[k] its length
        score, start = [NEG] * n, [0] * n
        for t in range(T):
            new_s, new_st = [NEG] * n, [0] * n
            for k in range(n):
                emit = float(lp[t, toks[k]])
                stay_blank = score[k] + float(lp[t, blank]) * ctc_ali_token_weight if score[k] > NEG else NEG
                stay_tok = score[k] + emit if score[k] > NEG else NEG
                cands = [(stay_tok, start[k]), (stay_blank, start[k])]
                if k == 0:
                    cands.append((emit, t))
                elif score[k - 1] > NEG:
                    cands.append((score[k - 1] + emit, start[k - 1]))
                new_s[k], new_st[k] = max(cands, key=lambda c: c[0])
                if k == n - 1:
                    # a hit ends on a frame that emits the last token (trailing blanks belong to what follows)
                    end_s, end_st = max([cands[0]] + cands[2:], key=lambda c: c[0])
            score, start = new_s, new_st
            if end_s > NEG:
                frames = t - end_st + 1
                avg = end_s / frames
                if avg >= keyword_threshold:
                    hits.append(WordSpotterHyp(word, avg, end_st, t, toks))
    hits.sort(key=lambda h: -h.score)
    kept: List[WordSpotterHyp] = []
    for h in hits:
        if all(h.end_frame < k.start_frame or h.start_frame > k.end_frame for k in kept):
            kept.append(h)
    kept.sort(key=lambda h: h.start_frame)
    return kept

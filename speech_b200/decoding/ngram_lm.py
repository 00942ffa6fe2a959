"""GPU n-gram language model for shallow fusion during batched decoding.

An ARPA model becomes a back-off automaton held in a handful of flat tensors: every n-gram context of length < order is a
state; ``arcs`` (sorted by ``state * V + token``) carry a log-probability and a destination state, every state has a
back-off weight and a back-off state.  ``advance(states[B])`` returns ``scores[B, V]`` (natural log) and
``next_states[B, V]`` for ALL tokens at once — no host synchronisation, no dense ``S x V`` table.  On a GPU this is one
kernel (``ops/csrc/decode_aux.cu``: the back-off chain is walked once per hypothesis, every token then searches the short arc
range of each level); on the CPU it is up to ``order`` rounds of a vectorised binary search over the arc keys.
Same contract as the reference's ``NGramGPULanguageModel`` (``parts/submodules/ngram_lm/ngram_lm_batched.py:505``;
``advance`` ``:1005-1129``), whose ARPA files store token ids as single characters ``chr(id + 100)``
(``kenlm_utils.py`` ``DEFAULT_TOKEN_OFFSET``).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

DEFAULT_TOKEN_OFFSET = 100
_LN10 = math.log(10.0)


class BackoffGraph(torch.nn.Module):
    """Flat-tensor back-off automaton shared by the n-gram LM and the boosting tree."""

    def __init__(self, vocab_size: int, arcs: Sequence[Tuple[int, int, float, int]], backoff_w: Sequence[float],
                 backoff_to: Sequence[int], max_depth: int, default_score: float = 0.0, start_state: int = 0,
                 bos_state: Optional[int] = None, final_w: Optional[Sequence[float]] = None):
        super().__init__()
        self.vocab_size = int(vocab_size)
        self.max_depth = int(max_depth)
        self.default_score = float(default_score)
        self.start_state = int(start_state)
        self.bos_state = int(bos_state if bos_state is not None else start_state)
        arcs = sorted(arcs, key=lambda a: a[0] * self.vocab_size + a[1])
        keys = torch.tensor([a[0] * self.vocab_size + a[1] for a in arcs], dtype=torch.long)
        self.register_buffer("arc_keys", keys if len(arcs) else torch.zeros(1, dtype=torch.long) - 1)
        self.register_buffer("arc_w", torch.tensor([a[2] for a in arcs] or [0.0], dtype=torch.float32))
        self.register_buffer("arc_to", torch.tensor([a[3] for a in arcs] or [0], dtype=torch.long))
        self.register_buffer("backoff_w", torch.tensor(list(backoff_w), dtype=torch.float32))
        self.register_buffer("backoff_to", torch.tensor(list(backoff_to), dtype=torch.long))
        self.register_buffer("final_w", torch.tensor(list(final_w) if final_w is not None else [0.0] * len(backoff_w),
                                                     dtype=torch.float32))
        self.register_buffer("_tok", torch.arange(self.vocab_size, dtype=torch.long))

    @property
    def num_states(self) -> int:
        return int(self.backoff_to.shape[0])

    def get_init_states(self, batch_size: int, bos: bool = True) -> torch.Tensor:
        return torch.full((batch_size,), self.bos_state if bos else self.start_state, dtype=torch.long,
                          device=self.arc_keys.device)

    @torch.no_grad()
    def advance(self, states: torch.Tensor, eos_id: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        from .. import ops

        return ops.ngram_advance(states, self.arc_keys, self.arc_w, self.arc_to, self.backoff_w, self.backoff_to, self.vocab_size,
                                 self.max_depth, self.default_score, self.start_state)

    forward = advance

    def get_final(self, states: torch.Tensor) -> torch.Tensor:
        """End-of-sequence score of each state."""
        return self.final_w[states]

    def score_sentence(self, tokens: Sequence[int], bos: bool = True) -> float:
        st = self.get_init_states(1, bos)
        total = 0.0
        for t in tokens:
            sc, nx = self.advance(st)
            total += float(sc[0, t])
            st = nx[:, t]
        return total


def _parse_arpa(path: str):
    order_counts: Dict[int, int] = {}
    ngrams: Dict[Tuple[str, ...], Tuple[float, float]] = {}
    cur = 0
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            if line.startswith("ngram ") and "=" in line:
                k, v = line[6:].split("=")
                order_counts[int(k)] = int(v)
            elif line.startswith("\\") and line.endswith("-grams:"):
                cur = int(line[1:].split("-")[0])
            elif line.startswith("\\"):
                continue
            elif cur:
                parts = line.split("\t") if "\t" in line else line.split()
                lp = float(parts[0])
                if "\t" in line:
                    words = tuple(parts[1].split(" "))
                    bo = float(parts[2]) if len(parts) > 2 else 0.0
                else:
                    words = tuple(parts[1:1 + cur])
                    bo = float(parts[1 + cur]) if len(parts) > 1 + cur else 0.0
                ngrams[words] = (lp, bo)
    return max(order_counts) if order_counts else cur, ngrams


class NGramGPULanguageModel(BackoffGraph):
    UNK_SCORE = -100.0 * _LN10

    @classmethod
    def from_arpa(cls, path: str, vocab_size: int, token_offset: int = DEFAULT_TOKEN_OFFSET,
                  normalize_unk: bool = True) -> "NGramGPULanguageModel":
        order, ngrams = _parse_arpa(path)

        def tok(w: str) -> Optional[int]:
            if w in ("<s>", "</s>", "<unk>"):
                return None
            if len(w) == 1:
                i = ord(w) - token_offset
                return i if 0 <= i < vocab_size else None
            try:
                i = int(w)
                return i if 0 <= i < vocab_size else None
            except ValueError:
                return None

        BOS = -1
        conv: Dict[Tuple[int, ...], Tuple[float, float]] = {}
        eos: Dict[Tuple[int, ...], float] = {}
        for words, (lp, bo) in ngrams.items():
            if words[-1] == "</s>":
                ctx = tuple(BOS if w == "<s>" else tok(w) for w in words[:-1])
                if None not in ctx:
                    eos[ctx] = lp * _LN10
                continue
            ids = tuple(BOS if w == "<s>" else tok(w) for w in words)
            if None in ids or BOS in ids[1:]:
                continue
            conv[ids] = (lp * _LN10, bo * _LN10)
        unk = ngrams.get(("<unk>",), (-100.0, 0.0))[0] * _LN10
        # states = contexts of length < order that exist as n-grams (plus the empty context)
        state_of: Dict[Tuple[int, ...], int] = {(): 0}
        for ids in sorted(conv, key=len):
            if len(ids) < order and ids not in state_of:
                state_of[ids] = len(state_of)

        def longest_suffix_state(ids: Tuple[int, ...]) -> int:
            ids = ids[-(order - 1):] if order > 1 else ()
            while ids not in state_of:
                ids = ids[1:]
            return state_of[ids]

        arcs = []
        for ids, (lp, _) in conv.items():
            if ids[-1] == BOS:
                continue
            ctx = ids[:-1]
            if ctx not in state_of:
                continue
            arcs.append((state_of[ctx], ids[-1], lp, longest_suffix_state(ids)))
        bw, bt, fw = [0.0] * len(state_of), [0] * len(state_of), [0.0] * len(state_of)
        for ctx, s in state_of.items():
            if ctx:
                bw[s] = conv[ctx][1]
                bt[s] = longest_suffix_state(ctx[1:]) if len(ctx) > 1 else 0

        def eos_score(ctx: Tuple[int, ...]) -> float:
            acc = 0.0
            while True:
                if ctx in eos:
                    return acc + eos[ctx]
                if not ctx:
                    return acc + unk
                acc += conv[ctx][1] if ctx in conv else 0.0
                ctx = ctx[1:]

        for ctx, s in state_of.items():
            fw[s] = eos_score(ctx)
        m = cls(vocab_size, arcs, bw, bt, max_depth=order, default_score=unk if not normalize_unk else unk,
                start_state=0, bos_state=state_of.get((BOS,), 0), final_w=fw)
        m.order = order
        return m

    @classmethod
    def from_file(cls, path: str, vocab_size: int, **kw) -> "NGramGPULanguageModel":
        if path.endswith((".pt", ".ckpt", ".nemo")):
            return cls.restore_from(path)
        return cls.from_arpa(path, vocab_size, **kw)

    @classmethod
    def dummy_unigram_lm(cls, vocab_size: int) -> "NGramGPULanguageModel":
        lp = -math.log(vocab_size)
        m = cls(vocab_size, [(0, t, lp, 0) for t in range(vocab_size)], [0.0], [0], max_depth=1, default_score=lp)
        m.order = 1
        return m

    # ------------------------------------------------------------------ persistence
    def save_to(self, path: str) -> None:
        torch.save({"vocab_size": self.vocab_size, "max_depth": self.max_depth, "default_score": self.default_score,
                    "start_state": self.start_state, "bos_state": self.bos_state, "order": getattr(self, "order", self.max_depth),
                    "tensors": {k: v.cpu() for k, v in self.state_dict().items()}}, path)

    @classmethod
    def restore_from(cls, path: str, map_location=None) -> "NGramGPULanguageModel":
        d = torch.load(path, map_location=map_location or "cpu", weights_only=False)
        t = d["tensors"]
        m = cls.__new__(cls)
        torch.nn.Module.__init__(m)
        m.vocab_size, m.max_depth, m.default_score = d["vocab_size"], d["max_depth"], d["default_score"]
        m.start_state, m.bos_state, m.order = d["start_state"], d["bos_state"], d["order"]
        for k, v in t.items():
            m.register_buffer(k, v)
        return m


def write_arpa(path: str, ngrams: Dict[Tuple[str, ...], Tuple[float, float]]) -> None:
    """Write an ARPA file from ``{words: (log10 prob, log10 backoff)}`` (used by tests and the LM training script)."""
    by_n: Dict[int, List[Tuple[Tuple[str, ...], Tuple[float, float]]]] = {}
    for w, v in ngrams.items():
        by_n.setdefault(len(w), []).append((w, v))
    with open(path, "w", encoding="utf-8") as f:
        f.write("\\data\\\n")
        for n in sorted(by_n):
            f.write(f"ngram {n}={len(by_n[n])}\n")
        for n in sorted(by_n):
            f.write(f"\n\\{n}-grams:\n")
            for w, (lp, bo) in by_n[n]:
                f.write(f"{lp:.6f}\t{' '.join(w)}" + (f"\t{bo:.6f}" if n < max(by_n) else "") + "\n")
        f.write("\n\\end\\\n")

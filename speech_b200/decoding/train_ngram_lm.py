"""Train a token-level n-gram language model for shallow fusion and write it as ARPA: ``python -m speech_b200.decoding.train_ngram_lm``.

Text is tokenised with the ASR model's tokenizer and every token id is written as the single character ``chr(id + 100)``
(the encoding ``NGramGPULanguageModel.from_arpa`` reads).  Probabilities use interpolated absolute discounting (one discount
per order, estimated from the count-of-counts as in Kneser-Ney) with lower orders built from continuation counts, so the model
normalises per context.  Role of ``scripts/asr_language_modeling/ngram_lm/train_kenlm.py`` in the reference (which shells out
to KenLM's ``lmplz``).
"""
from __future__ import annotations

import argparse
import json
import math
from collections import Counter, defaultdict
from typing import Dict, Iterable, List, Sequence, Tuple

from .ngram_lm import DEFAULT_TOKEN_OFFSET, write_arpa

BOS, EOS, UNK = "<s>", "</s>", "<unk>"


def train_ngram(sentences: Iterable[Sequence[int]], order: int = 3, vocab_size: int = 0, token_offset: int = DEFAULT_TOKEN_OFFSET
                ) -> Dict[Tuple[str, ...], Tuple[float, float]]:
    enc = lambda t: chr(int(t) + token_offset)  # noqa: E731
    counts: List[Counter] = [Counter() for _ in range(order + 1)]          # counts[n][ngram]
    for s in sentences:
        toks = [BOS] + [enc(t) for t in s] + [EOS]
        for n in range(1, order + 1):
            for i in range(len(toks) - n + 1):
                g = tuple(toks[i:i + n])
                if n > 1 or g[0] != BOS:
                    counts[n][g] += 1
                elif n == 1:
                    counts[n][g] += 0
    # lower orders use continuation counts (number of distinct left extensions), highest order uses raw counts
    adj: List[Dict[Tuple[str, ...], float]] = [dict() for _ in range(order + 1)]
    adj[order] = dict(counts[order])
    for n in range(order - 1, 0, -1):
        cont = Counter()
        for g in counts[n + 1]:
            cont[g[1:]] += 1
        adj[n] = {g: float(cont.get(g, 0)) for g in counts[n]}
        for g, c in counts[n].items():                                     # n-grams starting with <s> have no left context
            if g[0] == BOS:
                adj[n][g] = float(c) if n > 1 else 0.0
    discounts = [0.0] * (order + 1)
    for n in range(1, order + 1):
        n1 = sum(1 for c in adj[n].values() if round(c) == 1)
        n2 = sum(1 for c in adj[n].values() if round(c) == 2)
        discounts[n] = n1 / (n1 + 2.0 * n2) if n1 > 0 and n2 > 0 else 0.5
    vocab = sorted({g[0] for g in counts[1] if g[0] not in (BOS,)} | {EOS})
    V = max(len(vocab) + 1, vocab_size + 2)                                  # + <unk>
    # unigrams: discounted continuation probabilities interpolated with uniform
    total1 = sum(adj[1].get((w,), 0.0) for w in vocab)
    D1 = discounts[1]
    lam1 = D1 * sum(1 for w in vocab if adj[1].get((w,), 0.0) > 0) / max(total1, 1e-9)
    p1 = {w: max(adj[1].get((w,), 0.0) - D1, 0.0) / max(total1, 1e-9) + lam1 / V for w in vocab}
    p1[UNK] = lam1 / V
    prob: List[Dict[Tuple[str, ...], float]] = [dict() for _ in range(order + 1)]
    bow: List[Dict[Tuple[str, ...], float]] = [dict() for _ in range(order + 1)]
    prob[1] = {(w,): p for w, p in p1.items()}
    prob[1][(BOS,)] = 1e-99
    for n in range(2, order + 1):
        by_ctx: Dict[Tuple[str, ...], List[Tuple[str, float]]] = defaultdict(list)
        for g, c in adj[n].items():
            if c > 0:
                by_ctx[g[:-1]].append((g[-1], c))
        D = discounts[n]
        for ctx, items in by_ctx.items():
            tot = sum(c for _, c in items)
            lam = D * len(items) / tot
            bow[n - 1][ctx] = lam
            for w, c in items:
                lower = _backoff_prob(prob, bow, ctx[1:] + (w,), n - 1)
                prob[n][ctx + (w,)] = max(c - D, 0.0) / tot + lam * lower
    out: Dict[Tuple[str, ...], Tuple[float, float]] = {}
    for n in range(1, order + 1):
        for g, p in prob[n].items():
            b = bow[n].get(g, 1.0) if n < order else 1.0
            out[g] = (math.log10(max(p, 1e-99)), math.log10(max(b, 1e-99)) if n < order else 0.0)
    return out


def _backoff_prob(prob, bow, gram: Tuple[str, ...], n: int) -> float:
    if n == 0:
        return 0.0
    g = gram[-n:]
    if g in prob[n]:
        return prob[n][g]
    if n == 1:
        return prob[1].get((UNK,), 1e-10)
    return bow[n - 1].get(g[:-1], 1.0) * _backoff_prob(prob, bow, g[1:], n - 1)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.decoding.train_ngram_lm")
    ap.add_argument("--train-paths", nargs="+", required=True, help="text files (one sentence per line) or NeMo manifests (.json)")
    ap.add_argument("--tokenizer-model", help="SentencePiece tokenizer.model; omit for character models (use --labels)")
    ap.add_argument("--labels", help="file with one character label per line (character models)")
    ap.add_argument("--ngram-length", type=int, default=3)
    ap.add_argument("--output", required=True, help="ARPA file to write (a .pt file with the GPU automaton is written next to it)")
    args = ap.parse_args(argv)
    if args.tokenizer_model:
        from ..tokenizers import SentencePieceTokenizer

        tok = SentencePieceTokenizer(args.tokenizer_model)
        encode, V = tok.text_to_ids, tok.vocab_size
    else:
        labels = [l.rstrip("\n") for l in open(args.labels, encoding="utf-8")]
        idx = {c: i for i, c in enumerate(labels)}
        encode, V = (lambda s: [idx[c] for c in s if c in idx]), len(labels)

    def sentences():
        for p in args.train_paths:
            with open(p, encoding="utf-8") as f:
                for line in f:
                    line = line.strip()
                    if not line:
                        continue
                    text = json.loads(line)["text"] if p.endswith(".json") else line
                    yield encode(text)

    grams = train_ngram(sentences(), args.ngram_length, V)
    write_arpa(args.output, grams)
    from .ngram_lm import NGramGPULanguageModel

    NGramGPULanguageModel.from_arpa(args.output, V).save_to(args.output + ".pt")
    print(f"wrote {len(grams)} n-grams to {args.output}")


if __name__ == "__main__":
    main()

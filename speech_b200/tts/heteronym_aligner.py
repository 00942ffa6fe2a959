"""Heteronym disambiguation with an aligner: a word with several pronunciations is resolved by aligning every candidate phoneme sequence with the
recording and keeping the one the audio supports best.  The support of a candidate is the alignment log-likelihood (forward-sum over all
monotonic alignments of the token sequence to the spectrogram frames) per frame; the gap to the runner-up is the decision's confidence.
Reference: ``examples/tts/aligner_heteronym_disambiguation.py`` (same decision rule on an aligner's soft attention; there the score is the mean
distance between aligned frames and token embeddings).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .magpietts import ForwardSumLoss

_forward_sum = ForwardSumLoss()


@torch.no_grad()
def alignment_score(aligner: Callable, spec: torch.Tensor, spec_len: torch.Tensor, tokens: Sequence[int]) -> float:
    """Per-frame log-likelihood of ``tokens`` given ``spec [1, n_mels, T]`` under ``aligner(spec, spec_len, text, text_len) → (soft, log-probabilities
    [1, 1, T, U])``; higher is better."""
    text = torch.tensor([list(tokens)], dtype=torch.long, device=spec.device)
    text_len = torch.tensor([len(tokens)], device=spec.device)
    _, logp = aligner(spec, spec_len, text, text_len)
    nll = _forward_sum(logp.squeeze(1), text_len, spec_len)
    return -float(nll) / max(int(spec_len[0]), 1)


def disambiguate_heteronyms(aligner: Callable, spec: torch.Tensor, spec_len: torch.Tensor, words: Sequence[str], pronunciations: Dict[str, List[List[str]]],
                            encode: Callable[[List[str]], List[int]], default: Optional[Callable[[str], List[str]]] = None, space: Optional[str] = " ",
                            min_confidence: float = 0.0) -> Tuple[List[List[str]], List[Dict]]:
    """``words``: the utterance split into words; ``pronunciations[word]``: candidate phoneme lists (one entry = not ambiguous); ``default(word)``
    gives the symbols of a word without an entry (its letters when omitted).  Heteronyms are resolved left to right, each against the current best guess
    of the others (first candidate until resolved).  Returns the chosen symbols per word and one record per heteronym: ``{index, word, choice, scores,
    confidence}``; a decision whose confidence is below ``min_confidence`` keeps ``choice = None`` and the first candidate."""
    default = default or (lambda w: list(w))
    current: List[List[str]] = [list(pronunciations[w][0]) if w in pronunciations else list(default(w)) for w in words]

    def flat(seq: List[List[str]]) -> List[str]:
        out: List[str] = []
        for k, s in enumerate(seq):
            if k and space is not None:
                out.append(space)
            out.extend(s)
        return out

    decisions = []
    for i, w in enumerate(words):
        cands = pronunciations.get(w)
        if not cands or len(cands) < 2:
            continue
        scores = []
        for c in cands:
            trial = current[:i] + [list(c)] + current[i + 1:]
            scores.append(alignment_score(aligner, spec, spec_len, encode(flat(trial))))
        order = sorted(range(len(cands)), key=lambda k: -scores[k])
        conf = scores[order[0]] - scores[order[1]]
        choice = order[0] if conf >= min_confidence else None
        current[i] = list(cands[choice if choice is not None else 0])
        decisions.append({"index": i, "word": w, "choice": choice, "scores": scores, "confidence": conf})
    return current, decisions

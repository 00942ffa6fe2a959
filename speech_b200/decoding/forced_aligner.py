"""Forced alignment with a CTC model: token / word / segment time stamps for known transcripts.

``python -m speech_b200.decoding.forced_aligner model_path=m.nemo manifest_filepath=in.json output_dir=out`` writes one CTM
file per utterance and level plus an output manifest — the role of ``tools/nemo_forced_aligner/align.py`` (Viterbi over the
CTC trellis of ``blank tok1 blank tok2 ... blank``; ``parts/utils/aligner_utils.py``) and, for cutting long recordings into
utterances given their text, of ``tools/ctc_segmentation``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class AlignedToken:
    token_id: int
    text: str
    start_frame: int
    end_frame: int          # inclusive
    score: float = 0.0


@dataclass
class AlignedWord:
    text: str
    start: float
    end: float
    tokens: List[AlignedToken] = field(default_factory=list)


def viterbi_ctc_alignment(log_probs: torch.Tensor, tokens: Sequence[int], blank: int) -> List[Tuple[int, int, float]]:
    """log_probs [T, V]; returns per token (first frame, last frame, mean log-prob) of the best monotonic alignment in which
    every token occupies at least one frame and blanks may separate tokens."""
    lp = log_probs.detach().float().cpu()
    T = lp.shape[0]
    U = len(tokens)
    if U == 0:
        return []
    S = 2 * U + 1
    if T < U:
        raise ValueError(f"{T} frames cannot hold {U} tokens")
    ext = [blank] * S
    ext[1::2] = list(tokens)
    ext_t = torch.tensor(ext)
    NEG = -1e30
    score = torch.full((S,), NEG)
    score[0] = lp[0, blank]
    score[1] = lp[0, ext[1]]
    back = torch.zeros((T, S), dtype=torch.int8)
    can_skip = torch.zeros(S, dtype=torch.bool)
    for s in range(3, S, 2):
        can_skip[s] = ext[s] != ext[s - 2]
    for t in range(1, T):
        stay = score
        step1 = torch.cat([torch.full((1,), NEG), score[:-1]])
        step2 = torch.where(can_skip, torch.cat([torch.full((2,), NEG), score[:-2]]), torch.full((S,), NEG))
        cand = torch.stack([stay, step1, step2])
        best, arg = cand.max(dim=0)
        score = best + lp[t, ext_t]
        back[t] = arg.to(torch.int8)
    s = S - 1 if score[S - 1] >= score[S - 2] else S - 2
    path = [0] * T
    for t in range(T - 1, -1, -1):
        path[t] = s
        s -= int(back[t, s])
    out = []
    for u in range(U):
        frames = [t for t in range(T) if path[t] == 2 * u + 1]
        out.append((frames[0], frames[-1], float(sum(lp[t, tokens[u]] for t in frames) / len(frames))))
    return out


def align_utterance(model, audio, text: str, sample_rate: int = 16000):
    """Returns (token alignments, word alignments, seconds per frame) for one utterance."""
    x = torch.as_tensor(audio, dtype=torch.float32).reshape(1, -1).to(model.device)
    with torch.no_grad():
        out = model.forward(input_signal=x, input_signal_length=torch.tensor([x.shape[1]], device=model.device))
        if len(out) == 3:
            log_probs, enc_len = out[0], out[1]
        else:                                        # hybrid / transducer model: use the auxiliary CTC head
            enc, enc_len = out
            log_probs = model.ctc_decoder(encoder_output=enc)
    decoding = model.ctc_decoding if hasattr(model, "ctc_decoding") else model.decoding
    blank = int(decoding.blank_id)
    tok = getattr(model, "tokenizer", None)
    if tok is not None:
        ids = list(tok.text_to_ids(text))
        pieces = tok.ids_to_tokens(ids)
    else:
        vocab = list(model.decoder.vocabulary)
        ids = [vocab.index(c) for c in text if c in vocab]
        pieces = [vocab[i] for i in ids]
    T = int(enc_len[0])
    spans = viterbi_ctc_alignment(log_probs[0, :T], ids, blank)
    feat = getattr(model.preprocessor, "featurizer", model.preprocessor)
    spf = feat.hop_length / feat.sample_rate * model.encoder.subsampling_factor
    toks = [AlignedToken(i, p, a, b, s) for i, p, (a, b, s) in zip(ids, pieces, spans)]
    words: List[AlignedWord] = []
    is_char = tok is None
    for t in toks:
        starts = t.text.startswith("▁") if not is_char else False
        if is_char:
            if t.text == " ":
                words.append(AlignedWord("", 0.0, 0.0))
                continue
            if not words:
                words.append(AlignedWord("", t.start_frame * spf, 0.0))
            w = words[-1]
            if not w.tokens:
                w.start = t.start_frame * spf
            w.text += t.text
        else:
            if starts or not words:
                words.append(AlignedWord("", t.start_frame * spf, 0.0))
            w = words[-1]
            w.text += t.text.replace("▁", "").replace("##", "")
        w.tokens.append(t)
        w.end = (t.end_frame + 1) * spf
    words = [w for w in words if w.tokens]
    return toks, words, spf


def write_ctm(path: str, utt_id: str, items: Sequence[Tuple[str, float, float]]) -> None:
    with open(path, "w", encoding="utf-8") as f:
        for text, start, end in items:
            f.write(f"{utt_id} 1 {start:.3f} {max(end - start, 0.0):.3f} {text}\n")


def segment_long_audio(model, audio, sentences: Sequence[str], sample_rate: int = 16000) -> List[Tuple[float, float, str, float]]:
    """Cut a long recording at sentence boundaries: align the concatenated text, return (start, end, sentence, score)."""
    toks, words, spf = align_utterance(model, audio, " ".join(sentences), sample_rate)
    out, k = [], 0
    for s in sentences:
        n = len(s.split())
        ws = words[k:k + n]
        k += n
        if ws:
            sc = [t.score for w in ws for t in w.tokens]
            out.append((ws[0].start, ws[-1].end, s, float(sum(sc) / max(len(sc), 1))))
    return out


def main(argv=None):
    from ..core.config import OmegaConf, apply_overrides
    from ..data.audio_to_text import load_audio, read_manifest
    from ..models.asr_model import ASRModel
    import sys

    cfg = OmegaConf.create({"model_path": None, "manifest_filepath": None, "output_dir": "nfa_output", "additional_segment_grouping_separator": None})
    cfg = apply_overrides(cfg, list(sys.argv[1:] if argv is None else argv))
    model = ASRModel.restore_from(cfg.model_path).eval()
    os.makedirs(os.path.join(cfg.output_dir, "ctm", "tokens"), exist_ok=True)
    os.makedirs(os.path.join(cfg.output_dir, "ctm", "words"), exist_ok=True)
    out_items = []
    for it in read_manifest(cfg.manifest_filepath):
        utt = os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        toks, words, spf = align_utterance(model, load_audio(it["audio_filepath"]), it["text"])
        tp = os.path.join(cfg.output_dir, "ctm", "tokens", utt + ".ctm")
        wp = os.path.join(cfg.output_dir, "ctm", "words", utt + ".ctm")
        write_ctm(tp, utt, [(t.text, t.start_frame * spf, (t.end_frame + 1) * spf) for t in toks])
        write_ctm(wp, utt, [(w.text, w.start, w.end) for w in words])
        out_items.append(dict(it, token_level_ctm_filepath=tp, word_level_ctm_filepath=wp))
    with open(os.path.join(cfg.output_dir, "manifest_with_output_file_paths.json"), "w", encoding="utf-8") as f:
        for it in out_items:
            f.write(json.dumps(it, ensure_ascii=False) + "\n")


if __name__ == "__main__":
    main()

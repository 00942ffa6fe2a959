"""CTC segmentation: cut a long recording into utterances given its transcript and a CTC model.

Steps, each usable on its own and as sub-commands of ``python -m speech_b200.decoding.ctc_segmentation``:

1. ``split_text``      — normalise a transcript to the model's vocabulary and split it into utterance-sized lines.
2. ``ctc_segment``     — align the utterance list to the frame log-probabilities with a free start and a free end (audio
   before the first and after the last utterance is skipped at no cost) and score every utterance by its *worst* window: the
   minimum over windows of ``score_window`` frames of the mean aligned log-probability, so that one badly matching stretch
   marks the whole utterance.
3. ``cut_audio``       — write clips and manifests, split by a score threshold into kept / low-score / deleted stretches.
4. ``add_metrics`` / ``filter_manifest`` — transcribe the clips, add WER / CER / edge CER / length ratios, and filter.

References: ``tools/ctc_segmentation/scripts/{prepare_data,run_ctc_segmentation,utils,cut_audio,get_metrics_and_filter}.py``
(which call the external ``ctc_segmentation`` package for step 2; the alignment here is this file's own dynamic programme).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = ["Segment", "add_metrics", "ctc_segment", "cut_audio", "filter_manifest", "split_text", "write_segments", "read_segments"]

NEG = -1e30


@dataclass
class Segment:
    start: float
    end: float
    score: float
    text: str


# ------------------------------------------------------------------------------------------------ 1. text
_ABBREV = {"mr.": "mister", "mrs.": "misses", "dr.": "doctor", "st.": "saint", "vs.": "versus", "etc.": "et cetera", "no.": "number"}


def split_text(text: str, vocabulary: Sequence[str], max_length: int = 100, min_length: int = 0, additional_split_symbols: str = "",
               remove_brackets: bool = True, do_lower_case: bool = True, number_to_words: Optional[Callable[[str], str]] = None
               ) -> Tuple[List[str], List[str]]:
    """Returns ``(original sentences, normalised sentences)`` line by line.  Sentences end at ``.?!`` (+ ``additional_split_symbols``)
    and are split further at commas / spaces when longer than ``max_length`` words; short neighbours are merged up to
    ``min_length`` words.  The normalised line keeps only characters of ``vocabulary`` (numbers spelled with ``number_to_words``
    when given, else dropped)."""
    text = re.sub(r"\s+", " ", text.replace("\n", " ")).strip()
    if remove_brackets:
        text = re.sub(r"(\[.*?\])|(\(.*?\))|(\{.*?\})|(<.*?>)", " ", text)
    text = re.sub(r"[“”«»]", '"', text).replace("’", "'").replace("…", "...")
    for k, v in _ABBREV.items():
        text = re.sub(r"\b" + re.escape(k), v + " ", text, flags=re.IGNORECASE)
    enders = ".?!" + additional_split_symbols
    parts = re.split(r"(?<=[" + re.escape(enders) + r"])\s+", text)
    sents: List[str] = []
    for p in parts:
        p = p.strip()
        if not p:
            continue
        words = p.split()
        while len(words) > max_length:
            cut = max_length
            for k in range(max_length, max_length // 2, -1):            # prefer a comma near the limit
                if words[k - 1].endswith((",", ";", ":")):
                    cut = k
                    break
            sents.append(" ".join(words[:cut]))
            words = words[cut:]
        if words:
            sents.append(" ".join(words))
    if min_length > 0:
        merged: List[str] = []
        for s in sents:
            if merged and len(merged[-1].split()) < min_length:
                merged[-1] += " " + s
            else:
                merged.append(s)
        sents = merged
    vocab = set(vocabulary)
    norm = []
    for s in sents:
        t = s.lower() if do_lower_case else s
        if number_to_words is not None:
            t = re.sub(r"\d+(?:[.,]\d+)?", lambda m: " " + number_to_words(m.group(0)) + " ", t)
        t = t.replace("-", " ").replace("&", " and ")
        t = "".join(c if (c in vocab or c == " ") else " " for c in t)
        norm.append(re.sub(r"\s+", " ", t).strip())
    keep = [i for i, n in enumerate(norm) if n]
    return [sents[i] for i in keep], [norm[i] for i in keep]


# ------------------------------------------------------------------------------------------------ 2. alignment
def ctc_segment(log_probs: torch.Tensor, utterances: Sequence[Sequence[int]], blank: int, frame_duration: float, score_window: int = 30,
                texts: Optional[Sequence[str]] = None, max_states_in_memory: int = 400_000_000) -> List[Segment]:
    """``log_probs`` [T, V]; ``utterances``: token ids per utterance in reading order.  Returns one ``Segment`` per utterance."""
    lp = log_probs.detach().float().cpu()
    T = lp.shape[0]
    tokens: List[int] = []
    owner: List[int] = []
    for u, toks in enumerate(utterances):
        tokens += list(toks)
        owner += [u] * len(toks)
    U = len(tokens)
    if U == 0:
        return []
    S = 2 * U + 1
    if T < U:
        raise ValueError(f"{T} frames cannot hold {U} tokens")
    if T * S > max_states_in_memory:
        raise MemoryError(f"trellis of {T} x {S} states exceeds max_states_in_memory={max_states_in_memory}: segment the recording first "
                          f"(e.g. per chapter) or raise the limit")
    ext = torch.full((S,), blank, dtype=torch.long)
    ext[1::2] = torch.tensor(tokens)
    can_skip = torch.zeros(S, dtype=torch.bool)
    can_skip[3::2] = ext[3::2] != ext[1:-2:2]
    score = torch.full((S,), NEG)
    score[0] = 0.0                                                     # waiting before the first utterance costs nothing
    score[1] = lp[0, ext[1]]
    back = torch.zeros((T, S), dtype=torch.int8)
    final = torch.full((T,), NEG)                                      # best score of a path whose last token ends at frame t
    final[0] = score[S - 2] if S >= 2 else NEG
    neg1, neg2 = torch.full((1,), NEG), torch.full((2,), NEG)
    emit_cols = ext
    for t in range(1, T):
        stay = score
        step1 = torch.cat([neg1, score[:-1]])
        step2 = torch.where(can_skip, torch.cat([neg2, score[:-2]]), torch.full((S,), NEG))
        best, arg = torch.stack([stay, step1, step2]).max(dim=0)
        emit = lp[t, emit_cols]
        new = best + emit
        new[0] = 0.0                                                   # still waiting: free
        back[t] = arg.to(torch.int8)
        back[t, 0] = 0
        score = new
        final[t] = score[S - 2]
    t_end = int(final.argmax())                                        # everything after the last token is skipped for free
    path = np.zeros(t_end + 1, dtype=np.int64)
    s = S - 2
    for t in range(t_end, -1, -1):
        path[t] = s
        s -= int(back[t, s])
    frame_lp = lp[torch.arange(t_end + 1), ext[torch.from_numpy(path)]].numpy()
    top = lp.argmax(dim=-1).numpy()
    out: List[Segment] = []
    first_state = {}
    k = 0
    for u, toks in enumerate(utterances):
        first_state[u] = (2 * k + 1, 2 * (k + len(toks)) - 1)
        k += len(toks)
    for u, toks in enumerate(utterances):
        lo, hi = first_state[u]
        if not len(toks):
            out.append(Segment(0.0, 0.0, NEG, texts[u] if texts else ""))
            continue
        idx = np.nonzero((path >= lo) & (path <= hi))[0]
        a, b = int(idx[0]), int(idx[-1])
        # free waiting is cheaper than even a confident token frame, so the free ends of the path hug the tokens: give back the
        # frames on which the first / last token is still the most likely symbol
        if u == 0:
            while a > 0 and int(top[a - 1]) == int(toks[0]):
                a -= 1
        if u == len(utterances) - 1:
            while b + 1 < T and int(top[b + 1]) == int(toks[-1]):
                b += 1
        seg_lp = frame_lp[max(a, int(idx[0])):min(b, int(idx[-1])) + 1]
        if len(seg_lp) <= score_window:
            sc = float(seg_lp.mean())
        else:
            c = np.concatenate([[0.0], np.cumsum(seg_lp)])
            starts = np.arange(0, len(seg_lp) - score_window + 1, max(1, score_window // 2))
            sc = float(((c[starts + score_window] - c[starts]) / score_window).min())
        out.append(Segment(a * frame_duration, (b + 1) * frame_duration, sc, texts[u] if texts else ""))
    return out


def write_segments(path: str, audio_path: str, segments: Sequence[Segment], original_texts: Optional[Sequence[str]] = None):
    """First line: the audio path; then ``start end score | normalised text | original text`` per utterance."""
    with open(path, "w", encoding="utf-8") as f:
        f.write(str(audio_path) + "\n")
        for i, s in enumerate(segments):
            orig = original_texts[i] if original_texts else s.text
            f.write(f"{s.start:.3f} {s.end:.3f} {s.score:.4f} | {s.text} | {orig}\n")


def read_segments(path: str) -> Tuple[str, List[Segment], List[str]]:
    lines = open(path, encoding="utf-8").read().splitlines()
    segs, orig = [], []
    for l in lines[1:]:
        head, text, o = [x.strip() for x in l.split("|", 2)]
        a, b, sc = head.split()
        segs.append(Segment(float(a), float(b), float(sc), text))
        orig.append(o)
    return lines[0], segs, orig


# ------------------------------------------------------------------------------------------------ 3. cutting
def cut_audio(segments_file: str, output_dir: str, threshold: float = -2.0, offset_ms: float = 0.0, max_duration: float = 20.0) -> Dict[str, str]:
    """Writes ``clips/``, ``low_score_clips/`` and ``deleted_clips/`` (stretches between utterances) with one manifest each."""
    from ..data.audio_to_text import load_audio_file, save_wav as write_wav

    audio_path, segs, orig = read_segments(segments_file)
    audio, sr = load_audio_file(audio_path)
    audio = np.asarray(audio)
    if audio.ndim > 1:
        audio = audio.mean(axis=1)
    base = os.path.splitext(os.path.basename(audio_path))[0]
    dirs = {k: os.path.join(output_dir, k) for k in ("clips", "low_score_clips", "deleted_clips")}
    for d in dirs.values():
        os.makedirs(d, exist_ok=True)
    manifests = {k: os.path.join(output_dir, "manifests", f"{base}_{k}.json") for k in dirs}
    os.makedirs(os.path.join(output_dir, "manifests"), exist_ok=True)
    files = {k: open(p, "w", encoding="utf-8") for k, p in manifests.items()}
    off = offset_ms / 1e3
    prev_end = 0.0
    try:
        for i, (s, o) in enumerate(zip(segs, orig)):
            a, b = max(0.0, s.start - off), min(len(audio) / sr, s.end + off)
            kind = "clips" if s.score > threshold and (b - a) <= max_duration else "low_score_clips"
            p = os.path.join(dirs[kind], f"{base}_{i:04d}.wav")
            write_wav(p, audio[int(a * sr): int(b * sr)], sr)
            files[kind].write(json.dumps({"audio_filepath": p, "duration": round(b - a, 3), "text": s.text, "text_no_preprocessing": o,
                                          "score": s.score, "start_abs": a, "end_abs": b}, ensure_ascii=False) + "\n")
            if a - prev_end > 0.05:
                dp = os.path.join(dirs["deleted_clips"], f"{base}_del_{i:04d}.wav")
                write_wav(dp, audio[int(prev_end * sr): int(a * sr)], sr)
                files["deleted_clips"].write(json.dumps({"audio_filepath": dp, "duration": round(a - prev_end, 3), "text": "_"}) + "\n")
            prev_end = b
        if len(audio) / sr - prev_end > 0.05:
            dp = os.path.join(dirs["deleted_clips"], f"{base}_del_end.wav")
            write_wav(dp, audio[int(prev_end * sr):], sr)
            files["deleted_clips"].write(json.dumps({"audio_filepath": dp, "duration": round(len(audio) / sr - prev_end, 3), "text": "_"}) + "\n")
    finally:
        for f in files.values():
            f.close()
    return manifests


# ------------------------------------------------------------------------------------------------ 4. metrics and filtering
def _er(hyp: Sequence, ref: Sequence) -> float:
    prev = list(range(len(ref) + 1))
    for i, x in enumerate(hyp, 1):
        cur = [i]
        for j, y in enumerate(ref, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1] / max(1, len(ref))


def add_metrics(manifest: str, manifest_out: str, transcribe: Optional[Callable[[List[str]], List[str]]] = None, edge_len: int = 5) -> List[dict]:
    """Adds ``pred_text`` (via ``transcribe(paths)`` unless already there), WER, CER, CER of the first / last ``edge_len``
    characters (cut-off words show there), word-count and character-rate statistics."""
    rows = [json.loads(l) for l in open(manifest, encoding="utf-8") if l.strip()]
    if transcribe is not None:
        for r, p in zip(rows, transcribe([r["audio_filepath"] for r in rows])):
            r["pred_text"] = p
    for r in rows:
        ref, hyp = r["text"], r.get("pred_text", "")
        r["WER"] = round(100 * _er(hyp.split(), ref.split()), 2)
        r["CER"] = round(100 * _er(list(hyp), list(ref)), 2)
        r["start_CER"] = round(100 * _er(list(hyp[:edge_len]), list(ref[:edge_len])), 2)
        r["end_CER"] = round(100 * _er(list(hyp[-edge_len:]), list(ref[-edge_len:])), 2)
        r["len_diff_ratio"] = round(abs(len(ref) - len(hyp)) / max(1, len(ref)), 4)
        r["char_rate"] = round(len(ref) / max(1e-6, r.get("duration", 0.0)), 2) if r.get("duration") else None
    with open(manifest_out, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    return rows


def filter_manifest(manifest: str, manifest_out: str, max_cer: float = 30.0, max_wer: float = 75.0, max_len_diff_ratio: float = 0.3,
                    max_edge_cer: float = 60.0, min_duration: float = 1.0, max_duration: float = 20.0) -> Tuple[float, float]:
    """Keeps the rows inside all limits; returns ``(kept hours, dropped hours)``."""
    kept = dropped = 0.0
    with open(manifest_out, "w", encoding="utf-8") as f:
        for l in open(manifest, encoding="utf-8"):
            if not l.strip():
                continue
            r = json.loads(l)
            d = float(r.get("duration", 0.0))
            ok = (r["CER"] <= max_cer and r["WER"] <= max_wer and r["len_diff_ratio"] <= max_len_diff_ratio and r["start_CER"] <= max_edge_cer
                  and r["end_CER"] <= max_edge_cer and min_duration <= d <= max_duration)
            if ok:
                kept += d
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
            else:
                dropped += d
    return kept / 3600.0, dropped / 3600.0


# ------------------------------------------------------------------------------------------------ command line
def segment_file(model, audio_path: str, transcript_path: str, output_file: str, max_length: int = 30, score_window: int = 30) -> List[Segment]:
    """Runs steps 1-2 for one recording with a CTC model of this package."""
    from ..data.audio_to_text import load_audio

    vocab = list(getattr(model.decoder, "vocabulary", None) or [])
    tok = getattr(model, "tokenizer", None)
    chars = set("".join(vocab)) - {"▁", "#"} if vocab else set("abcdefghijklmnopqrstuvwxyz'")
    orig, norm = split_text(open(transcript_path, encoding="utf-8").read(), sorted(chars), max_length=max_length)
    ids = [tok.text_to_ids(n) if tok is not None else [vocab.index(c) for c in n if c in vocab] for n in norm]
    audio = torch.as_tensor(np.asarray(load_audio(audio_path)), dtype=torch.float32).unsqueeze(0)
    with torch.no_grad():
        dev = next(model.parameters()).device
        out = model.forward(input_signal=audio.to(dev), input_signal_length=torch.tensor([audio.shape[1]], device=dev))
    lp = out[0][0]
    blank = lp.shape[-1] - 1
    spf = audio.shape[1] / 16000.0 / lp.shape[0]
    segs = ctc_segment(lp, ids, blank, spf, score_window=score_window, texts=norm)
    write_segments(output_file, audio_path, segs, orig)
    return segs


def main(argv=None):
    import argparse

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("segment")
    a.add_argument("--model", required=True), a.add_argument("--audio", required=True), a.add_argument("--transcript", required=True)
    a.add_argument("--output", required=True), a.add_argument("--max_length", type=int, default=30), a.add_argument("--window", type=int, default=30)
    c = sub.add_parser("cut")
    c.add_argument("--segments", required=True), c.add_argument("--output_dir", required=True), c.add_argument("--threshold", type=float, default=-2.0)
    c.add_argument("--offset_ms", type=float, default=0.0), c.add_argument("--max_duration", type=float, default=20.0)
    f = sub.add_parser("filter")
    f.add_argument("--manifest", required=True), f.add_argument("--output", required=True), f.add_argument("--model", default=None)
    f.add_argument("--max_cer", type=float, default=30.0), f.add_argument("--max_wer", type=float, default=75.0)
    args = ap.parse_args(argv)
    if args.cmd == "segment":
        from ..models.asr_model import ASRModel

        model = ASRModel.restore_from(args.model).eval()
        segs = segment_file(model, args.audio, args.transcript, args.output, args.max_length, args.window)
        print(f"{len(segs)} segments -> {args.output}")
    elif args.cmd == "cut":
        print(json.dumps(cut_audio(args.segments, args.output_dir, args.threshold, args.offset_ms, args.max_duration)))
    else:
        transcribe = None
        if args.model:
            from ..models.asr_model import ASRModel

            model = ASRModel.restore_from(args.model).eval()
            transcribe = lambda paths: [h.text if hasattr(h, "text") else h for h in model.transcribe(paths)]  # noqa: E731
        tmp = args.output + ".metrics"
        add_metrics(args.manifest, tmp, transcribe)
        kept, dropped = filter_manifest(tmp, args.output, max_cer=args.max_cer, max_wer=args.max_wer)
        print(f"kept {kept:.3f} h, dropped {dropped:.3f} h")


if __name__ == "__main__":
    main()

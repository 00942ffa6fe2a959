"""Data-preparation tools beyond bucketing and tarring; each is a function and a sub-command of
``python -m speech_b200.data.tools_extra``.

* ``kaldi2json``                   — Kaldi data directory (``wav.scp``, ``text``, optional ``segments`` / ``utt2spk`` / ``utt2dur``) → manifest.
* ``filelist_to_manifest``         — speaker-task manifest from a list of files (label = a path component), optional train / dev split.
* ``pathfiles_to_diarize_manifest``— lists of audio / RTTM / UEM / CTM / text files joined on the file stem → diarization manifest.
* ``add_noise``                    — mixes noise recordings into every utterance at the given SNRs, writes audio + manifests.
* ``code_switching_manifest``      — samples utterance sequences alternating between two monolingual manifests up to a duration;
  ``code_switching_audio`` renders them with pauses.
* ``add_eob_labels`` / ``clean_eou_manifest`` — end-of-utterance / backchannel labels by utterance length and text cleaning.
* ``keyword_fscore``               — precision / recall / F-score of key phrases in recognised text.
* ``confidence_benchmark``         — AUC-ROC, AUC-PR (errors as positives), normalised cross-entropy and expected calibration
  error of word confidences.
* ``estimate_token_bins``          — bucket edges over token counts of text / conversation data.
* ``export_conversations_to_tar``  — multimodal conversations with their audio into numbered tar shards.
* ``write_transcribed_files``      — merges per-rank prediction shards of pseudo-labelling back into manifests.

References: ``scripts/dataset_processing/{kaldi2json,add_noise}.py``, ``scripts/speaker_tasks/{filelist_to_manifest,
pathfiles_to_diarize_manifest}.py``, ``scripts/speech_recognition/code_switching/*``, ``scripts/asr_eou/{add_eob_labels,clean_manifest}.py``,
``scripts/asr_context_biasing/compute_key_words_fscore.py``, ``scripts/speech_recognition/confidence/benchmark_asr_confidence.py``,
``scripts/speechlm2/{estimate_token_bins,export_conversations_to_tar}.py``, ``scripts/pseudo_labeling/write_transcribed_files.py``.
"""
from __future__ import annotations

import argparse
import glob
import io
import json
import os
import re
import tarfile
from collections import defaultdict
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .audio_to_text import load_audio, load_audio_file, read_manifest, save_wav, write_manifest

__all__ = ["add_eob_labels", "add_noise", "clean_eou_manifest", "code_switching_audio", "code_switching_manifest", "confidence_benchmark",
           "estimate_token_bins", "export_conversations_to_tar", "filelist_to_manifest", "kaldi2json", "keyword_fscore",
           "pathfiles_to_diarize_manifest", "write_transcribed_files"]


def _read_kv(path: str) -> Dict[str, str]:
    out = {}
    if os.path.exists(path):
        for line in open(path, encoding="utf-8"):
            parts = line.rstrip("\n").split(maxsplit=1)
            if parts:
                out[parts[0]] = parts[1] if len(parts) > 1 else ""
    return out


def _duration(path: str) -> float:
    x, sr = load_audio_file(path)
    return len(x) / float(sr)


# ------------------------------------------------------------------------------------------------ Kaldi
def kaldi2json(data_dir: str, manifest: str, with_aux_data: bool = True, duration_fn: Callable[[str], float] = _duration) -> int:
    """``wav.scp`` entries that are commands (ending in ``|``) are rejected: the audio must exist as files."""
    wavs, text = _read_kv(os.path.join(data_dir, "wav.scp")), _read_kv(os.path.join(data_dir, "text"))
    segments = _read_kv(os.path.join(data_dir, "segments"))
    aux = {k: _read_kv(os.path.join(data_dir, k)) for k in ("utt2spk", "utt2dur", "utt2lang", "utt2gender")} if with_aux_data else {}
    rows = []
    for w in wavs.values():
        if w.rstrip().endswith("|"):
            raise ValueError("wav.scp holds a command pipeline; extract the audio to files first")
    if segments:
        for utt, rest in segments.items():
            rec, a, b = rest.split()
            rows.append({"audio_filepath": wavs[rec], "offset": float(a), "duration": round(float(b) - float(a), 4), "text": text.get(utt, ""), "utt": utt})
    else:
        for utt, path in wavs.items():
            d = float(aux.get("utt2dur", {}).get(utt, 0.0)) or duration_fn(path)
            rows.append({"audio_filepath": path, "duration": round(d, 4), "text": text.get(utt, ""), "utt": utt})
    for r in rows:
        for k, name in (("utt2spk", "speaker"), ("utt2lang", "lang"), ("utt2gender", "gender")):
            if r["utt"] in aux.get(k, {}):
                r[name] = aux[k][r["utt"]]
    write_manifest(manifest, rows)
    return len(rows)


# ------------------------------------------------------------------------------------------------ speaker tasks
def filelist_to_manifest(filelist: Sequence[str], manifest: str, id_index: int = -2, split_fraction: float = 0.0, min_spkrs_count: int = 0,
                         seed: int = 0, duration_fn: Callable[[str], float] = _duration) -> Tuple[int, int]:
    """The label is the ``id_index``-th component of the path.  ``split_fraction`` > 0 holds out that share of every speaker's files
    into ``<manifest>_dev``; speakers with fewer than ``min_spkrs_count`` files are dropped."""
    by = defaultdict(list)
    for p in filelist:
        p = p.strip()
        if p:
            by[p.split(os.sep)[id_index]].append(p)
    rng = np.random.default_rng(seed)
    train, dev = [], []
    for spk, files in sorted(by.items()):
        if len(files) < min_spkrs_count:
            continue
        files = sorted(files)
        rng.shuffle(files)
        n_dev = int(round(len(files) * split_fraction)) if split_fraction > 0 else 0
        for i, f in enumerate(files):
            (dev if i < n_dev else train).append({"audio_filepath": f, "offset": 0, "duration": round(duration_fn(f), 4), "label": spk})
    write_manifest(manifest, train)
    if split_fraction > 0:
        base, ext = os.path.splitext(manifest)
        write_manifest(base + "_dev" + ext, dev)
    return len(train), len(dev)


def _by_stem(paths: Optional[Sequence[str]]) -> Dict[str, str]:
    return {os.path.splitext(os.path.basename(p.strip()))[0]: p.strip() for p in (paths or []) if p.strip()}


def pathfiles_to_diarize_manifest(audio_paths: Sequence[str], manifest: str, text_paths=None, rttm_paths=None, uem_paths=None, ctm_paths=None,
                                  add_duration: bool = False, duration_fn: Callable[[str], float] = _duration) -> int:
    rt, ue, ct, tx = _by_stem(rttm_paths), _by_stem(uem_paths), _by_stem(ctm_paths), _by_stem(text_paths)
    rows = []
    for stem, p in _by_stem(audio_paths).items():
        n_spk = None
        if stem in rt:
            n_spk = len({l.split()[7] for l in open(rt[stem], encoding="utf-8") if l.startswith("SPEAKER")})
        text = open(tx[stem], encoding="utf-8").read().strip() if stem in tx else "-"
        rows.append({"audio_filepath": p, "offset": 0, "duration": round(duration_fn(p), 4) if add_duration else None, "label": "infer", "text": text,
                     "num_speakers": n_spk, "rttm_filepath": rt.get(stem), "uem_filepath": ue.get(stem), "ctm_filepath": ct.get(stem)})
    write_manifest(manifest, rows)
    return len(rows)


# ------------------------------------------------------------------------------------------------ noise
def add_noise(manifest: str, noise_manifest: str, out_dir: str, snrs: Sequence[float] = (0, 5, 10, 15), sample_rate: int = 16000, seed: int = 0) -> List[str]:
    """One output manifest (and audio folder) per SNR.  A noise recording is drawn per utterance, looped or cropped to length and
    scaled so that ``10 log10(P_speech / P_noise)`` equals the SNR."""
    rng = np.random.default_rng(seed)
    items, noises = read_manifest(manifest), read_manifest(noise_manifest)
    outs = []
    for snr in snrs:
        d = os.path.join(out_dir, f"snr_{snr:g}")
        os.makedirs(d, exist_ok=True)
        rows = []
        for it in items:
            x = np.asarray(load_audio(it["audio_filepath"], target_sr=sample_rate, offset=float(it.get("offset", 0) or 0), duration=it.get("duration")), dtype=np.float32)
            nz = np.asarray(load_audio(noises[int(rng.integers(len(noises)))]["audio_filepath"], target_sr=sample_rate), dtype=np.float32)
            if len(nz) < len(x):
                nz = np.tile(nz, int(np.ceil(len(x) / max(1, len(nz)))))
            s = int(rng.integers(0, len(nz) - len(x) + 1))
            nz = nz[s:s + len(x)]
            ps, pn = float(np.mean(x ** 2)) + 1e-12, float(np.mean(nz ** 2)) + 1e-12
            y = x + nz * np.sqrt(ps / (pn * 10 ** (snr / 10.0)))
            peak = np.abs(y).max()
            y = y / peak * 0.99 if peak > 0.99 else y
            p = os.path.join(d, os.path.basename(it["audio_filepath"]))
            save_wav(p, y.astype(np.float32), sample_rate)
            rows.append({**it, "audio_filepath": p, "offset": 0, "snr": snr})
        mp = os.path.join(out_dir, f"manifest_snr_{snr:g}.json")
        write_manifest(mp, rows)
        outs.append(mp)
    return outs


# ------------------------------------------------------------------------------------------------ code switching
def code_switching_manifest(manifest1: str, manifest2: str, out_manifest: str, id1: str, id2: str, max_sample_duration: float = 30.0,
                            min_sample_duration: float = 10.0, dataset_size_hours: float = 1.0, prob1: float = 0.5, seed: int = 0) -> int:
    """Every output line describes one synthetic sample: ``lang_ids``, ``paths``, ``durations`` (and ``texts``) of utterances drawn
    from the two corpora (language 1 with probability ``prob1``) until the sample is between the duration limits."""
    rng = np.random.default_rng(seed)
    a, b = read_manifest(manifest1), read_manifest(manifest2)
    total, rows = 0.0, []
    while total < dataset_size_hours * 3600.0:
        cur, ids, paths, durs, texts = 0.0, [], [], [], []
        target = float(rng.uniform(min_sample_duration, max_sample_duration))
        for _ in range(1000):
            first = rng.random() < prob1
            it = (a if first else b)[int(rng.integers(len(a if first else b)))]
            d = float(it["duration"])
            if cur + d > max_sample_duration:
                if cur >= min_sample_duration:
                    break
                continue
            ids.append(id1 if first else id2), paths.append(it["audio_filepath"]), durs.append(d), texts.append(it.get("text", ""))
            cur += d
            if cur >= target:
                break
        if not paths:
            break
        rows.append({"lang_ids": ids, "paths": paths, "durations": durs, "texts": texts, "duration": round(cur, 4)})
        total += cur
    write_manifest(out_manifest, rows)
    return len(rows)


def code_switching_audio(cs_manifest: str, out_dir: str, out_manifest: str, sample_rate: int = 16000, pause_start: float = 0.02, pause_join: float = 0.08,
                         pause_end: float = 0.02, db_norm: float = -25.0, seed: int = 0) -> int:
    """Renders the samples: every utterance is level-normalised to ``db_norm`` dBFS RMS, joined with a short pause whose edges
    are faded, and the result is written with the concatenated text and per-word language ids."""
    os.makedirs(out_dir, exist_ok=True)
    rows = []
    for k, it in enumerate(read_manifest(cs_manifest)):
        parts = [np.zeros(int(pause_start * sample_rate), dtype=np.float32)]
        for j, p in enumerate(it["paths"]):
            x = np.asarray(load_audio(p, target_sr=sample_rate), dtype=np.float32)
            rms = float(np.sqrt(np.mean(x ** 2))) + 1e-9
            x = x * (10 ** (db_norm / 20.0) / rms)
            fade = min(len(x) // 2, int(0.005 * sample_rate))
            if fade:
                ramp = np.linspace(0, 1, fade, dtype=np.float32)
                x[:fade] *= ramp
                x[-fade:] *= ramp[::-1]
            parts.append(x)
            parts.append(np.zeros(int((pause_join if j + 1 < len(it["paths"]) else pause_end) * sample_rate), dtype=np.float32))
        y = np.clip(np.concatenate(parts), -1, 1)
        path = os.path.join(out_dir, f"cs_{k:06d}.wav")
        save_wav(path, y, sample_rate)
        rows.append({"audio_filepath": path, "duration": round(len(y) / sample_rate, 4), "text": " ".join(t for t in it["texts"] if t),
                     "lang_ids": it["lang_ids"], "word_lang_ids": [l for l, t in zip(it["lang_ids"], it["texts"]) for _ in t.split()]})
    write_manifest(out_manifest, rows)
    return len(rows)


# ------------------------------------------------------------------------------------------------ end of utterance
def clean_eou_manifest(manifest: str, out: str, lower: bool = True, keep: str = "a-z' ", min_words: int = 1) -> int:
    rows = []
    for it in read_manifest(manifest):
        t = it.get("text", "").lower() if lower else it.get("text", "")
        t = re.sub(rf"[^{keep}]", " ", t.replace("-", " "))
        t = re.sub(r"\s+", " ", t).strip()
        if len(t.split()) >= min_words:
            rows.append({**it, "text": t})
    write_manifest(out, rows)
    return len(rows)


def add_eob_labels(manifest: str, out: str, backchannels: Sequence[str] = ("yeah", "uh huh", "mhm", "okay", "right", "i see", "hmm", "oh"),
                   max_backchannel_words: int = 2, eou_token: str = "<EOU>", eob_token: str = "<EOB>") -> Tuple[int, int]:
    """Utterances that consist only of a backchannel phrase get ``eob_token`` (end of backchannel), all others ``eou_token``."""
    bc = {b.lower() for b in backchannels}
    n_eou = n_eob = 0
    rows = []
    for it in read_manifest(manifest):
        t = it.get("text", "").strip().lower()
        is_bc = t in bc or (len(t.split()) <= max_backchannel_words and all(w in bc for w in t.split()) and t != "")
        rows.append({**it, "is_backchannel": is_bc, "eou_label": eob_token if is_bc else eou_token})
        n_eob, n_eou = n_eob + int(is_bc), n_eou + int(not is_bc)
    write_manifest(out, rows)
    return n_eou, n_eob


# ------------------------------------------------------------------------------------------------ evaluation helpers
def keyword_fscore(manifest_or_rows, key_words: Sequence[str], pred_field: str = "pred_text", ref_field: str = "text") -> Dict[str, float]:
    """A key phrase counts once per occurrence in the reference; a hit is an occurrence in the hypothesis of the same utterance
    (at most as many hits as reference occurrences), extra hypothesis occurrences are false positives."""
    rows = read_manifest(manifest_or_rows) if isinstance(manifest_or_rows, str) else list(manifest_or_rows)
    tp = fn = fp = 0
    for r in rows:
        ref, hyp = f" {r[ref_field].lower()} ", f" {r.get(pred_field, '').lower()} "
        for kw in key_words:
            k = f" {kw.lower()} "
            nr, nh = _count_overlapping(ref, k), _count_overlapping(hyp, k)
            tp, fn, fp = tp + min(nr, nh), fn + max(0, nr - nh), fp + max(0, nh - nr)
    prec, rec = tp / max(1, tp + fp), tp / max(1, tp + fn)
    return {"precision": prec, "recall": rec, "fscore": 2 * prec * rec / max(1e-9, prec + rec), "tp": tp, "fn": fn, "fp": fp}


def _count_overlapping(text: str, pat: str) -> int:
    n, i = 0, text.find(pat)
    while i >= 0:
        n, i = n + 1, text.find(pat, i + len(pat) - 1)
    return n


def _auc(x: np.ndarray, y: np.ndarray) -> float:
    return float(np.trapezoid(y, x)) if hasattr(np, "trapezoid") else float(np.trapz(y, x))


def confidence_benchmark(confidences: Sequence[float], correct: Sequence[bool], n_bins: int = 10) -> Dict[str, float]:
    """``confidences`` in [0, 1] for words, ``correct`` whether each word was right.  AUC-ROC (confidence ranks correct words above
    wrong ones), AUC-PR with correct words as positives and ``auc_nt`` with wrong words as positives (negative-class PR),
    normalised cross-entropy (1 = perfect, 0 = as informative as the accuracy alone), expected and maximum calibration error."""
    c, y = np.clip(np.asarray(confidences, dtype=np.float64), 1e-9, 1 - 1e-9), np.asarray(correct, dtype=bool)
    order = np.argsort(-c, kind="stable")
    ys = y[order]
    tps, fps = np.cumsum(ys), np.cumsum(~ys)
    P, N = max(1, int(y.sum())), max(1, int((~y).sum()))
    roc = _auc(np.concatenate([[0], fps / N]), np.concatenate([[0], tps / P]))
    prec = tps / np.maximum(1, tps + fps)
    pr = _auc(np.concatenate([[0], tps / P]), np.concatenate([[prec[0]], prec]))
    order_n = np.argsort(c, kind="stable")
    yn = ~y[order_n]
    tn, fn_ = np.cumsum(yn), np.cumsum(~yn)
    prec_n = tn / np.maximum(1, tn + fn_)
    nt = _auc(np.concatenate([[0], tn / N]), np.concatenate([[prec_n[0]], prec_n]))
    acc = float(y.mean())
    h_prior = -(acc * np.log(max(acc, 1e-9)) + (1 - acc) * np.log(max(1 - acc, 1e-9)))
    h_cond = -float(np.mean(np.where(y, np.log(c), np.log(1 - c))))
    nce = (h_prior - h_cond) / h_prior if h_prior > 0 else 0.0
    edges = np.linspace(0, 1, n_bins + 1)
    ece = mce = 0.0
    for lo, hi in zip(edges[:-1], edges[1:]):
        m = (c > lo) & (c <= hi) if lo > 0 else (c >= lo) & (c <= hi)
        if m.any():
            gap = abs(float(y[m].mean()) - float(c[m].mean()))
            ece, mce = ece + gap * m.mean(), max(mce, gap)
    return {"auc_roc": roc, "auc_pr": pr, "auc_nt": nt, "nce": float(nce), "ece": float(ece), "mce": float(mce), "accuracy": acc}


# ------------------------------------------------------------------------------------------------ speech-LM data
def estimate_token_bins(token_counts: Iterable[int], num_buckets: int, num_subbuckets: Optional[int] = None,
                        second_dim: Optional[Iterable[int]] = None, max_tokens: Optional[int] = None) -> List:
    """Bucket edges with an equal share of the total tokens per bucket (not of the examples: long examples dominate the cost).  With
    ``second_dim`` (e.g. output tokens per example) every bucket gets ``num_subbuckets`` 2-D edges ``(input, output)``."""
    a = np.asarray(list(token_counts), dtype=np.int64)
    b = np.asarray(list(second_dim), dtype=np.int64) if second_dim is not None else None
    if max_tokens is not None:
        keep = a <= max_tokens
        a, b = a[keep], (b[keep] if b is not None else None)
    order = np.argsort(a, kind="stable")
    a = a[order]
    csum = np.cumsum(a)
    edges = []
    for k in range(1, num_buckets):
        i = int(np.searchsorted(csum, csum[-1] * k / num_buckets))
        edges.append(int(a[min(i, len(a) - 1)]))
    edges.append(int(a[-1]))
    edges = sorted(set(edges))                                          # a heavy tail can put several cuts on one value
    if b is None:
        return edges
    b = b[order]
    out, lo = [], 0
    for e in edges:
        hi = int(np.searchsorted(a, e, side="right"))
        sub = np.sort(b[lo:hi]) if hi > lo else np.asarray([0])
        n = num_subbuckets or 2
        for j in range(1, n + 1):
            out.append((e, int(sub[min(len(sub) - 1, int(np.ceil(len(sub) * j / n)) - 1)])))
        lo = hi
    return out


def export_conversations_to_tar(conversations: Iterable[Dict[str, Any]], out_dir: str, shard_size: int = 100, prefix: str = "conversations") -> List[str]:
    """Each conversation ``{"id", "conversations": [{"from", "value", "type": "text" | "audio", "duration"?}]}``: audio turns are
    copied into the shard under ``<id>_<turn>.<ext>`` and their ``value`` rewritten to that name; the JSON goes in as
    ``<id>.json``.  Shards hold ``shard_size`` conversations; a ``<prefix>_NNNNNN.jsonl`` manifest mirrors every tar."""
    os.makedirs(out_dir, exist_ok=True)
    shards, cur, tf, mf = [], 0, None, None

    def open_shard():
        nonlocal tf, mf
        name = os.path.join(out_dir, f"{prefix}_{len(shards):06d}")
        tf, mf = tarfile.open(name + ".tar", "w"), open(name + ".jsonl", "w", encoding="utf-8")
        shards.append(name + ".tar")

    for conv in conversations:
        if tf is None or cur == shard_size:
            if tf is not None:
                tf.close(), mf.close()
            open_shard()
            cur = 0
        conv = json.loads(json.dumps(conv))
        for t, turn in enumerate(conv["conversations"]):
            if turn.get("type") == "audio":
                ext = os.path.splitext(turn["value"])[1] or ".wav"
                arc = f"{conv['id']}_{t}{ext}"
                tf.add(turn["value"], arcname=arc)
                turn["value"] = arc
        data = json.dumps(conv, ensure_ascii=False).encode("utf-8")
        info = tarfile.TarInfo(f"{conv['id']}.json")
        info.size = len(data)
        tf.addfile(info, io.BytesIO(data))
        mf.write(data.decode("utf-8") + "\n")
        cur += 1
    if tf is not None:
        tf.close(), mf.close()
    return shards


def write_transcribed_files(prediction_glob: str, manifests: Sequence[str], out_suffix: str = "_pl", text_field: str = "text", pred_field: str = "pred_text",
                            keep_original_as: str = "orig_text") -> List[str]:
    """Pseudo-labelling: predictions written by several ranks (JSON lines with ``audio_filepath`` and ``pred_text``) are joined to
    the source manifests by audio path; the prediction becomes the new ``text``."""
    preds: Dict[str, str] = {}
    for p in sorted(glob.glob(prediction_glob)):
        for it in read_manifest(p):
            preds[it["audio_filepath"]] = it[pred_field]
    outs = []
    for m in manifests:
        rows = []
        for it in read_manifest(m):
            if it["audio_filepath"] in preds:
                it = {**it, keep_original_as: it.get(text_field, ""), text_field: preds[it["audio_filepath"]]}
                rows.append(it)
        base, ext = os.path.splitext(m)
        write_manifest(base + out_suffix + ext, rows)
        outs.append(base + out_suffix + ext)
    return outs


# ------------------------------------------------------------------------------------------------ command line
def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.data.tools_extra")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("kaldi2json"); a.add_argument("--data_dir", required=True); a.add_argument("--manifest", required=True)
    a = sub.add_parser("filelist-to-manifest"); a.add_argument("--filelist", required=True); a.add_argument("--manifest", required=True)
    a.add_argument("--id", type=int, default=-2); a.add_argument("--split", type=float, default=0.0); a.add_argument("--min_spkrs_count", type=int, default=0)
    a = sub.add_parser("diarize-manifest"); a.add_argument("--paths2audio_files", required=True); a.add_argument("--manifest_filepath", required=True)
    a.add_argument("--paths2rttm_files"); a.add_argument("--paths2uem_files"); a.add_argument("--paths2ctm_files"); a.add_argument("--paths2txt_files")
    a.add_argument("--add_duration", action="store_true")
    a = sub.add_parser("add-noise"); a.add_argument("--input_manifest", required=True); a.add_argument("--noise_manifest", required=True)
    a.add_argument("--out_dir", required=True); a.add_argument("--snrs", type=float, nargs="+", default=[0, 5, 10, 15]); a.add_argument("--seed", type=int, default=0)
    a = sub.add_parser("keyword-fscore"); a.add_argument("--input_manifest", required=True); a.add_argument("--key_words_file", required=True)
    a = sub.add_parser("add-eob-labels"); a.add_argument("manifest"); a.add_argument("out")
    args = ap.parse_args(argv)
    lines = lambda p: open(p, encoding="utf-8").read().splitlines() if p else None  # noqa: E731
    if args.cmd == "kaldi2json":
        print(kaldi2json(args.data_dir, args.manifest))
    elif args.cmd == "filelist-to-manifest":
        print(filelist_to_manifest(lines(args.filelist), args.manifest, args.id, args.split, args.min_spkrs_count))
    elif args.cmd == "diarize-manifest":
        print(pathfiles_to_diarize_manifest(lines(args.paths2audio_files), args.manifest_filepath, lines(args.paths2txt_files), lines(args.paths2rttm_files),
                                            lines(args.paths2uem_files), lines(args.paths2ctm_files), args.add_duration))
    elif args.cmd == "add-noise":
        print("\n".join(add_noise(args.input_manifest, args.noise_manifest, args.out_dir, args.snrs, seed=args.seed)))
    elif args.cmd == "keyword-fscore":
        kws = [l.split("_")[0].strip() for l in lines(args.key_words_file) if l.strip()]
        print(json.dumps(keyword_fscore(args.input_manifest, kws)))
    elif args.cmd == "add-eob-labels":
        print(add_eob_labels(args.manifest, args.out))


if __name__ == "__main__":
    main()

"""Dataset preparation commands: ``python -m speech_b200.data.tools <command> ...``.

* ``estimate-duration-bins``  — bucket edges with equal total duration per bucket, 1-D (duration) or 2-D (duration × tokens)
  (reference: ``scripts/speech_recognition/estimate_duration_bins.py`` / ``estimate_duration_bins_2d.py``)
* ``estimate-data-weights``   — per-dataset sampling weights from total hours with a temperature
  (``scripts/speech_recognition/estimate_data_weights.py``)
* ``convert-to-tarred``       — shuffle a manifest into ``num_shards`` tar shards + per-shard manifests
  (``scripts/speech_recognition/convert_to_tarred_audio_dataset.py``)
* ``filter-manifest``         — duration / characters-per-second / token-per-second filters
"""
from __future__ import annotations

import argparse
import json
import os
import tarfile
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .audio_to_text import read_manifest, write_manifest
from .cuts import determine_bucket_duration_bins


def estimate_duration_bins(manifests: Sequence[str], num_buckets: int, min_duration: Optional[float] = None,
                           max_duration: Optional[float] = None) -> List[float]:
    durs = [float(it["duration"]) for m in manifests for it in read_manifest(m, min_duration=min_duration, max_duration=max_duration)]
    return determine_bucket_duration_bins(durs, num_buckets)


def estimate_duration_bins_2d(manifests: Sequence[str], tokenizer, num_buckets: int, num_subbuckets: int = 2,
                              min_duration: Optional[float] = None, max_duration: Optional[float] = None,
                              max_tps: Optional[float] = None) -> List[Tuple[float, int]]:
    """Duration bins first, then inside each duration bin ``num_subbuckets`` token-count bins with equal counts."""
    items = [it for m in manifests for it in read_manifest(m, min_duration=min_duration, max_duration=max_duration)]
    durs = np.asarray([float(it["duration"]) for it in items])
    toks = np.asarray([len(tokenizer.text_to_ids(it.get("text", ""))) for it in items])
    if max_tps:
        keep = toks / np.maximum(durs, 1e-6) <= max_tps
        durs, toks = durs[keep], toks[keep]
    edges = determine_bucket_duration_bins(durs.tolist(), num_buckets) + [float(durs.max())]
    out: List[Tuple[float, int]] = []
    lo = 0.0
    for hi in edges:
        sel = toks[(durs > lo) & (durs <= hi)] if lo > 0 else toks[durs <= hi]
        if len(sel) == 0:
            sel = np.asarray([1])
        qs = np.quantile(sel, [(k + 1) / num_subbuckets for k in range(num_subbuckets)])
        for q in qs:
            out.append((round(float(hi), 3), int(np.ceil(q))))
        lo = hi
    return out


def estimate_data_weights(manifests: Dict[str, str], temperature: float = 1.0) -> Dict[str, float]:
    hours = {k: sum(float(it["duration"]) for it in read_manifest(v)) / 3600.0 for k, v in manifests.items()}
    w = np.asarray(list(hours.values())) ** temperature
    w = w / w.sum()
    return {k: float(x) for k, x in zip(hours, w)}


def convert_to_tarred(manifest: str, target_dir: str, num_shards: int, shuffle: bool = True, seed: int = 0,
                      max_duration: Optional[float] = None, min_duration: Optional[float] = None, sort_in_shards: bool = False) -> Dict:
    items = read_manifest(manifest, min_duration=min_duration, max_duration=max_duration)
    if shuffle:
        np.random.default_rng(seed).shuffle(items)
    os.makedirs(target_dir, exist_ok=True)
    per = len(items) // num_shards
    if per == 0:
        raise ValueError(f"{len(items)} utterances cannot fill {num_shards} shards")
    all_entries = []
    for s in range(num_shards):
        chunk = items[s * per:(s + 1) * per]                    # the remainder is dropped so that shards are equal
        if sort_in_shards:
            chunk = sorted(chunk, key=lambda it: it["duration"])
        entries = []
        with tarfile.open(os.path.join(target_dir, f"audio_{s}.tar"), "w") as tf:
            for k, it in enumerate(chunk):
                name = f"{s}_{k}_{os.path.basename(it['audio_filepath'])}"
                tf.add(it["audio_filepath"], arcname=name)
                entries.append({**{kk: vv for kk, vv in it.items() if kk != "audio_filepath"}, "audio_filepath": name, "shard_id": s})
        write_manifest(os.path.join(target_dir, f"manifest_{s}.json"), entries)
        all_entries += entries
    write_manifest(os.path.join(target_dir, "tarred_audio_manifest.json"), all_entries)
    meta = {"num_shards": num_shards, "num_samples_per_shard": per, "dropped": len(items) - per * num_shards, "shuffle": shuffle, "seed": seed}
    with open(os.path.join(target_dir, "metadata.yaml"), "w") as f:
        for k, v in meta.items():
            f.write(f"{k}: {v}\n")
    return meta


def filter_manifest(manifest: str, out: str, min_duration=None, max_duration=None, max_cps: Optional[float] = None,
                    min_cps: Optional[float] = None) -> int:
    kept = []
    for it in read_manifest(manifest, min_duration=min_duration, max_duration=max_duration):
        cps = len(it.get("text", "")) / max(float(it["duration"]), 1e-6)
        if (max_cps is None or cps <= max_cps) and (min_cps is None or cps >= min_cps):
            kept.append(it)
    write_manifest(out, kept)
    return len(kept)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.data.tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("estimate-duration-bins")
    a.add_argument("manifests", nargs="+")
    a.add_argument("-b", "--buckets", type=int, default=30)
    a.add_argument("-l", "--min-duration", type=float)
    a.add_argument("-u", "--max-duration", type=float)
    a.add_argument("--tokenizer", help="tokenizer.model (SentencePiece): switches to 2-D bins")
    a.add_argument("-s", "--sub-buckets", type=int, default=2)
    a = sub.add_parser("estimate-data-weights")
    a.add_argument("manifests", nargs="+", help="name=path pairs")
    a.add_argument("-t", "--temperature", type=float, default=1.0)
    a = sub.add_parser("convert-to-tarred")
    a.add_argument("--manifest-path", required=True)
    a.add_argument("--target-dir", required=True)
    a.add_argument("--num-shards", type=int, required=True)
    a.add_argument("--no-shuffle", action="store_true")
    a.add_argument("--shuffle-seed", type=int, default=0)
    a.add_argument("--max-duration", type=float)
    a.add_argument("--min-duration", type=float)
    a.add_argument("--sort-in-shards", action="store_true")
    a = sub.add_parser("filter-manifest")
    a.add_argument("manifest")
    a.add_argument("out")
    a.add_argument("--min-duration", type=float)
    a.add_argument("--max-duration", type=float)
    a.add_argument("--max-cps", type=float)
    a.add_argument("--min-cps", type=float)
    args = ap.parse_args(argv)
    if args.cmd == "estimate-duration-bins":
        if args.tokenizer:
            from ..tokenizers import SentencePieceTokenizer

            bins = estimate_duration_bins_2d(args.manifests, SentencePieceTokenizer(args.tokenizer), args.buckets, args.sub_buckets,
                                             args.min_duration, args.max_duration)
            print("bucket_duration_bins=[" + ",".join(f"[{d},{t}]" for d, t in bins) + "]")
        else:
            bins = estimate_duration_bins(args.manifests, args.buckets, args.min_duration, args.max_duration)
            print("bucket_duration_bins=[" + ",".join(f"{b:.3f}" for b in bins) + "]")
    elif args.cmd == "estimate-data-weights":
        print(json.dumps(estimate_data_weights(dict(p.split("=", 1) for p in args.manifests), args.temperature), indent=1))
    elif args.cmd == "convert-to-tarred":
        print(json.dumps(convert_to_tarred(args.manifest_path, args.target_dir, args.num_shards, not args.no_shuffle, args.shuffle_seed,
                                           args.max_duration, args.min_duration, args.sort_in_shards)))
    elif args.cmd == "filter-manifest":
        print(filter_manifest(args.manifest, args.out, args.min_duration, args.max_duration, args.max_cps, args.min_cps))


if __name__ == "__main__":
    main()

"""Build a tokenizer for ASR training from manifests or text files:
``python -m speech_b200.tokenizers.process_asr_text_tokenizer --manifest train.json --data_root out --vocab_size 1024 --tokenizer spe``
writes ``out/tokenizer_spe_<type>_v<size>/tokenizer.model`` (+ ``vocab.txt``), or a WordPiece ``vocab.txt`` for ``--tokenizer wpe``
(reference: ``scripts/tokenizers/process_asr_text_tokenizer.py``)."""
from __future__ import annotations

import argparse
import json
import os
from collections import Counter

from . import create_spt_model


def build_document(manifests, data_files, out_dir: str, lower_case: bool) -> str:
    os.makedirs(out_dir, exist_ok=True)
    doc = os.path.join(out_dir, "text_corpus", "document.txt")
    os.makedirs(os.path.dirname(doc), exist_ok=True)
    with open(doc, "w", encoding="utf-8") as out:
        for m in manifests or []:
            with open(m, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        t = json.loads(line)["text"]
                        out.write((t.lower() if lower_case else t) + "\n")
        for p in data_files or []:
            with open(p, encoding="utf-8") as f:
                for line in f:
                    out.write((line.lower() if lower_case else line).rstrip("\n") + "\n")
    return doc


def build_wordpiece_vocab(doc: str, vocab_size: int, out_dir: str) -> str:
    """Greedy sub-word inventory: all characters, then the most frequent word-initial and ``##``-continuation pieces."""
    words = Counter()
    with open(doc, encoding="utf-8") as f:
        for line in f:
            words.update(line.split())
    chars = Counter()
    pieces = Counter()
    for w, c in words.items():
        for i, ch in enumerate(w):
            chars[ch if i == 0 else "##" + ch] += c
        for n in range(2, min(len(w), 8) + 1):
            pieces[w[:n]] += c
            for s in range(1, len(w) - n + 1):
                pieces["##" + w[s:s + n]] += c
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [c for c, _ in chars.most_common()]
    for p, _ in pieces.most_common():
        if len(vocab) >= vocab_size:
            break
        if p not in vocab:
            vocab.append(p)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "vocab.txt")
    with open(path, "w", encoding="utf-8") as f:
        f.write("\n".join(vocab) + "\n")
    return path


def main(argv=None):
    ap = argparse.ArgumentParser(prog="speech_b200.tokenizers.process_asr_text_tokenizer")
    ap.add_argument("--manifest", default=None, help="comma-separated manifests")
    ap.add_argument("--data_file", default=None, help="comma-separated text files")
    ap.add_argument("--data_root", required=True)
    ap.add_argument("--vocab_size", type=int, required=True)
    ap.add_argument("--tokenizer", choices=["spe", "wpe"], default="spe")
    ap.add_argument("--spe_type", choices=["bpe", "unigram", "char", "word"], default="unigram")
    ap.add_argument("--spe_character_coverage", type=float, default=1.0)
    ap.add_argument("--spe_sample_size", type=int, default=-1)
    ap.add_argument("--spe_user_defined_symbols", nargs="*", default=None)
    ap.add_argument("--spe_bos", action="store_true")
    ap.add_argument("--spe_eos", action="store_true")
    ap.add_argument("--spe_pad", action="store_true")
    ap.add_argument("--no_lower_case", action="store_true")
    a = ap.parse_args(argv)
    doc = build_document(a.manifest.split(",") if a.manifest else None, a.data_file.split(",") if a.data_file else None, a.data_root,
                         not a.no_lower_case)
    if a.tokenizer == "spe":
        out = os.path.join(a.data_root, f"tokenizer_spe_{a.spe_type}_v{a.vocab_size}")
        model, vocab = create_spt_model(doc, a.vocab_size, a.spe_sample_size, not a.no_lower_case, a.spe_type, out, a.spe_character_coverage,
                                        a.spe_user_defined_symbols, a.spe_bos, a.spe_eos, a.spe_pad)
        print(f"tokenizer model: {model}\nvocabulary: {vocab}")
    else:
        out = os.path.join(a.data_root, f"tokenizer_wpe_v{a.vocab_size}")
        print(f"vocabulary: {build_wordpiece_vocab(doc, a.vocab_size, out)}")


if __name__ == "__main__":
    main()

"""Resolve heteronyms in a TTS manifest with a trained aligner: for every word that the pronunciation dictionary lists with several pronunciations, the
candidate that aligns best with the recording is written out.

python examples/tts/aligner_heteronym_disambiguation.py model=aligner.nemo manifest=train.json out=train_disambiguated.json phoneme_dict=cmudict.txt \
    [heteronyms=heteronyms.txt] [confidence=0.0]
Output lines carry ``text_phonemes`` (the chosen symbols, ``|``-separated per word) and ``heteronym_decisions`` (word, chosen index, scores, confidence).
(reference script: ``examples/tts/aligner_heteronym_disambiguation.py``)."""
import json
import re

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.tts.classic import AlignerModel
from speech_b200.tts.heteronym_aligner import disambiguate_heteronyms
from speech_b200.utils.logging import logging

DEFAULTS = {"model": None, "manifest": None, "out": "disambiguated.json", "phoneme_dict": None, "heteronyms": None, "confidence": 0.0, "cuda": None}


def read_pronunciations(path, only=None):
    """CMUdict-style lines ``WORD  PH1 PH2 ...`` (``WORD(2)`` for alternatives) → ``{word: [[phonemes], ...]}`` lower-cased."""
    out = {}
    with open(path, encoding="latin-1") as f:
        for line in f:
            if not line.strip() or line.startswith(";;;"):
                continue
            word, *ph = line.split()
            word = re.sub(r"\(\d+\)$", "", word).lower()
            if only is None or word in only:
                if ph not in out.setdefault(word, []):
                    out[word].append(ph)
    return out


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if not torch.cuda.is_available() or (cfg.cuda is not None and int(cfg.cuda) < 0) else f"cuda:{cfg.cuda or 0}"
    model = AlignerModel.restore_from(cfg.model, map_location=dev).to(dev).eval()
    only = set(open(cfg.heteronyms).read().lower().split()) if cfg.heteronyms else None
    prons = read_pronunciations(cfg.phoneme_dict)
    ambiguous = {w for w, p in prons.items() if len(p) > 1 and (only is None or w in only)}
    tok = model.tokenizer
    encode = (lambda symbols: tok.encode_from_g2p(symbols)) if hasattr(tok, "encode_from_g2p") else (lambda symbols: tok.text_to_ids("".join(symbols)))
    n_dec = 0
    with open(cfg.out, "w", encoding="utf-8") as fout:
        for it in read_manifest(cfg.manifest):
            words = re.findall(r"[\w']+", it["text"].lower())
            table = {w: (prons[w] if w in ambiguous else prons[w][:1]) for w in set(words) if w in prons}
            audio = torch.as_tensor(load_audio(it["audio_filepath"], int(model.cfg.get("sample_rate", 22050))), device=dev)[None]
            with torch.no_grad():
                spec = model.mel.mel(audio)
            chosen, decisions = disambiguate_heteronyms(model, spec, torch.tensor([spec.shape[-1]], device=dev), words, table, encode, min_confidence=float(cfg.confidence))
            n_dec += len(decisions)
            fout.write(json.dumps({**it, "text_phonemes": "|".join(" ".join(s) for s in chosen), "heteronym_decisions": decisions}, ensure_ascii=False) + "\n")
    logging.info(f"wrote {cfg.out}: {n_dec} heteronym decisions")


if __name__ == "__main__":
    main()

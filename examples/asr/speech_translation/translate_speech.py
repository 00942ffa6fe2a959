"""Translate speech with a trained speech-translation (or multitask) checkpoint; reports corpus BLEU when the manifest has
reference translations.

python examples/asr/speech_translation/translate_speech.py model_path=st.nemo dataset_manifest=test.json output_filename=out.json [beam_size=4 len_pen=0.6]
(reference script: ``examples/asr/speech_translation/translate_speech.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.models.transformer_bpe_models import corpus_bleu
from speech_b200.utils.logging import logging

DEFAULTS = {"model_path": None, "dataset_manifest": None, "output_filename": "translations.json", "batch_size": 16, "beam_size": None, "len_pen": None,
            "cuda": None, "target_field": "text"}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    model = ASRModel.restore_from(cfg.model_path, map_location=dev).to(dev).eval()
    if cfg.beam_size is not None and hasattr(model, "change_decoding_strategy"):
        model.change_decoding_strategy(OmegaConf.create({"strategy": "beam", "beam": {"beam_size": int(cfg.beam_size), "len_pen": float(cfg.len_pen or 0.0)}}))
    items = read_manifest(cfg.dataset_manifest)
    hyps = model.transcribe([it["audio_filepath"] for it in items], batch_size=cfg.batch_size)
    texts = [h.text if hasattr(h, "text") else h for h in hyps]
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, t in zip(items, texts):
            f.write(json.dumps(dict(it, pred_translation=t), ensure_ascii=False) + "\n")
    if all(it.get(cfg.target_field) for it in items):
        bleu = corpus_bleu(texts, [it[cfg.target_field] for it in items])
        logging.info(f"BLEU = {bleu:.2f}")
        print(f"BLEU: {bleu:.2f}")
    return texts


if __name__ == "__main__":
    main()

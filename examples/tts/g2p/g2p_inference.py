"""Convert the graphemes of a manifest to phonemes with a trained G2P model; adds ``pred_text`` and reports PER when the manifest
has reference phonemes.

python examples/tts/g2p/g2p_inference.py pretrained_model=g2p.nemo manifest_filepath=in.json output_file=out.json [grapheme_field=text_graphemes phoneme_field=text]
(reference script: ``examples/tts/g2p/g2p_inference.py``)."""
import json

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.tts.g2p import IpaG2p, phoneme_error_rate
from speech_b200.utils.logging import logging


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"pretrained_model": None, "manifest_filepath": None, "output_file": None, "grapheme_field": "text_graphemes",
                                            "phoneme_field": "text", "batch_size": 32}), cfg)
    model = ModelPT.restore_from(cfg.pretrained_model, map_location="cpu").eval()
    preds = model.convert_graphemes_to_phonemes(cfg.manifest_filepath, cfg.output_file, grapheme_field=cfg.grapheme_field, batch_size=cfg.batch_size)
    rows = [json.loads(l) for l in open(cfg.manifest_filepath, encoding="utf-8") if l.strip()]
    if all(cfg.phoneme_field in r for r in rows):
        refs = [r[cfg.phoneme_field].split() if " " in r[cfg.phoneme_field] else IpaG2p.split_ipa(r[cfg.phoneme_field]) for r in rows]
        per = phoneme_error_rate([p.split() for p in preds], refs)
        logging.info(f"PER {100 * per:.2f}%")
        print(f"PER: {per:.4f}")
    return preds


if __name__ == "__main__":
    main()

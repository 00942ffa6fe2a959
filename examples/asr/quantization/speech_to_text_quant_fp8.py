"""Post-training FP8 (e4m3) quantisation of an ASR model's linear layers: calibrate on a manifest, report, evaluate WER.

python examples/asr/quantization/speech_to_text_quant_fp8.py model_path=model.nemo calib_manifest=calib.json \
    eval_manifest=test.json num_calib_batches=16 batch_size=16 percentile=99.9 skip='[joint,decoder]' output=model_fp8.pt
(reference scripts: ``examples/asr/quantization/speech_to_text_calibrate.py`` and ``speech_to_text_quant_infer.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate
from speech_b200.utils.quantization import calibrate, quantization_report, quantize_model, save_quantized

DEFAULTS = {"model_path": None, "calib_manifest": None, "eval_manifest": None, "num_calib_batches": 16, "batch_size": 16, "percentile": 99.9,
            "include": ["encoder"], "skip": [], "output": "model_fp8.pt", "cuda": None}


def _wer(model, items, batch_size):
    hyps = model.transcribe([it["audio_filepath"] for it in items], batch_size=batch_size)
    texts = [h.text if hasattr(h, "text") else h for h in hyps]
    return word_error_rate(texts, [it["text"] for it in items])


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if not torch.cuda.is_available() or (cfg.cuda is not None and int(cfg.cuda) < 0) else f"cuda:{cfg.cuda or 0}"
    model = ASRModel.restore_from(cfg.model_path, map_location=dev).to(dev).eval()
    calib = read_manifest(cfg.calib_manifest)
    paths = [it["audio_filepath"] for it in calib][: int(cfg.num_calib_batches) * int(cfg.batch_size)]
    batches = [paths[i:i + cfg.batch_size] for i in range(0, len(paths), cfg.batch_size)]
    amax = calibrate(model, batches, forward=lambda m, b: m.transcribe(b, batch_size=len(b)), include=list(cfg.include) or None,
                     skip=list(cfg.skip) or None, percentile=float(cfg.percentile))
    report = quantization_report(model, amax)
    logging.info("most sensitive layers (weight SQNR, dB): " + json.dumps(report[:8]))
    before = _wer(model, read_manifest(cfg.eval_manifest), cfg.batch_size) if cfg.eval_manifest else None
    done = quantize_model(model, amax)
    logging.info(f"quantised {len(done)} linear layers to e4m3")
    if cfg.eval_manifest:
        after = _wer(model, read_manifest(cfg.eval_manifest), cfg.batch_size)
        logging.info(f"WER before {100 * before:.2f}%  after {100 * after:.2f}%")
    save_quantized(model, cfg.output)
    logging.info(f"wrote {cfg.output}")


if __name__ == "__main__":
    main()

"""Transcribe audio files or a manifest with any ASR checkpoint and optionally report WER and RTFx.

python examples/asr/transcribe_speech.py model_path=model.nemo dataset_manifest=test.json output_filename=out.json \
    batch_size=32 cuda=0 compute_dtype=bfloat16 calculate_rtfx=true decoder_type=rnnt timestamps=false
(reference script: ``examples/asr/transcribe_speech.py``; RTFx option ``:80,403-502``)."""
import json
import os
import time

import torch

from speech_b200 import ops
from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"model_path": None, "pretrained_name": None, "audio_dir": None, "dataset_manifest": None, "output_filename": None,
            "batch_size": 32, "num_workers": 0, "cuda": None, "compute_dtype": "bfloat16", "decoder_type": None, "timestamps": False,
            "calculate_wer": True, "calculate_rtfx": False, "warmup_steps": 1, "run_steps": 1, "decoding": None, "audio_type": "wav",
            "overwrite_transcripts": True, "return_hypotheses": False}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    if cfg.model_path is None and cfg.pretrained_name is None:
        raise ValueError("one of model_path / pretrained_name is required")
    dev = torch.device("cpu" if cfg.cuda is not None and int(cfg.cuda) < 0 or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}")
    model = ASRModel.restore_from(cfg.model_path, map_location=str(dev)) if cfg.model_path else ASRModel.from_pretrained(cfg.pretrained_name)
    model = model.to(dev).eval()
    if cfg.decoder_type and hasattr(model, "change_decoding_strategy") and hasattr(model, "cur_decoder"):
        model.change_decoding_strategy(cfg.decoding, decoder_type=cfg.decoder_type)
    elif cfg.decoding is not None:
        model.change_decoding_strategy(cfg.decoding)
    if cfg.dataset_manifest:
        items = read_manifest(cfg.dataset_manifest)
    else:
        files = sorted(os.path.join(cfg.audio_dir, f) for f in os.listdir(cfg.audio_dir) if f.endswith("." + cfg.audio_type))
        items = [{"audio_filepath": f} for f in files]
    paths = [it["audio_filepath"] for it in items]
    total_audio = sum(float(it.get("duration", 0.0) or 0.0) for it in items)
    cdt = {"bfloat16": torch.bfloat16, "float16": torch.float16}.get(str(cfg.compute_dtype)) if dev.type == "cuda" else None
    elapsed = None
    with ops.compute_dtype(cdt):
        for _ in range(int(cfg.warmup_steps) if cfg.calculate_rtfx else 0):
            model.transcribe(paths[: cfg.batch_size], batch_size=cfg.batch_size)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(max(1, int(cfg.run_steps)) if cfg.calculate_rtfx else 1):
            hyps = model.transcribe(paths, batch_size=cfg.batch_size, return_hypotheses=True, timestamps=bool(cfg.timestamps))
        if dev.type == "cuda":
            torch.cuda.synchronize()
        elapsed = (time.perf_counter() - t0) / (max(1, int(cfg.run_steps)) if cfg.calculate_rtfx else 1)
    texts = [h.text if hasattr(h, "text") else h for h in hyps]
    out = cfg.output_filename or (os.path.splitext(cfg.dataset_manifest)[0] + "_transcribed.json" if cfg.dataset_manifest else "transcripts.json")
    with open(out, "w", encoding="utf-8") as f:
        for it, t, h in zip(items, texts, hyps):
            rec = dict(it, pred_text=t)
            if cfg.timestamps and getattr(h, "timestamp", None) is not None and isinstance(h.timestamp, dict):
                rec["word_timestamps"] = h.timestamp.get("word")
            f.write(json.dumps(rec, ensure_ascii=False) + "\n")
    logging.info(f"wrote {len(texts)} transcripts to {out}")
    if cfg.calculate_wer and items and "text" in items[0] and any(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(texts, [it['text'] for it in items]):.2f}%")
    if cfg.calculate_rtfx and total_audio > 0:
        logging.info(f"RTFx: {total_audio / elapsed:.1f}  ({total_audio:.1f} s of audio in {elapsed:.2f} s)")
    return out


if __name__ == "__main__":
    main()

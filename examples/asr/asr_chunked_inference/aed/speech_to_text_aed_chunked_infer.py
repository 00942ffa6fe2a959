"""Chunked inference of an attention encoder-decoder (Canary-style) model on long recordings: fixed windows, each transcribed with
the prompt of its manifest line, texts joined.

python .../speech_to_text_aed_chunked_infer.py model_path=m.nemo dataset_manifest=test.json chunk_len_in_secs=40 batch_size=8 \\
       [decoding.beam.beam_size=1] [source_lang=en target_lang=en task=asr pnc=yes]
(reference script: ``examples/asr/asr_chunked_inference/aed/speech_to_text_aed_chunked_infer.py``)."""
import json

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate
from speech_b200.utils.streaming_utils import FrameBatchMultiTaskAED

PROMPT_KEYS = ("source_lang", "target_lang", "task", "taskname", "pnc", "itn", "timestamp", "diarize")


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "output_filename": "aed_chunked_transcripts.json",
                                            "chunk_len_in_secs": 40.0, "batch_size": 8, "decoding": None, "source_lang": None, "target_lang": None,
                                            "task": None, "pnc": None}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    if cfg.decoding is not None:
        model.change_decoding_strategy(cfg.decoding)
    asr = FrameBatchMultiTaskAED(model, chunk_len=cfg.chunk_len_in_secs, batch_size=cfg.batch_size)
    items = read_manifest(cfg.dataset_manifest)
    preds = []
    for it in items:
        # prompt slots: command line first, then the manifest line, then the model's defaults
        slots = {k: (cfg.get(k) if cfg.get(k) is not None else it.get(k)) for k in PROMPT_KEYS}
        slots = {k: v for k, v in slots.items() if v is not None}
        asr.read_audio_file(it["audio_filepath"], meta_data={"prompt": slots} if slots else None)
        preds.append(asr.transcribe())
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, p in zip(items, preds):
            f.write(json.dumps(dict(it, pred_text=p), ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(preds, [it['text'] for it in items]):.2f}%")
    return preds


if __name__ == "__main__":
    main()

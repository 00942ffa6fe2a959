"""Buffered (chunked with left/right context) inference for long recordings with a CTC model.

python .../speech_to_text_buffered_infer_ctc.py model_path=m.nemo dataset_manifest=test.json chunk_len_in_secs=1.6 total_buffer_in_secs=4.0
(reference script: ``examples/asr/asr_chunked_inference/ctc/speech_to_text_buffered_infer_ctc.py``)."""
import json

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate
from speech_b200.utils.streaming_utils import FrameBatchASR


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "output_filename": "buffered_transcripts.json",
                                            "chunk_len_in_secs": 1.6, "total_buffer_in_secs": 4.0, "batch_size": 32}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    asr = FrameBatchASR(model, frame_len=cfg.chunk_len_in_secs, total_buffer=cfg.total_buffer_in_secs, batch_size=cfg.batch_size)
    items = read_manifest(cfg.dataset_manifest)
    preds = []
    for it in items:
        asr.reset()
        asr.read_audio_file(it["audio_filepath"])
        preds.append(asr.transcribe())
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, p in zip(items, preds):
            f.write(json.dumps(dict(it, pred_text=p), ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(preds, [it['text'] for it in items]):.2f}%")
    return preds


if __name__ == "__main__":
    main()

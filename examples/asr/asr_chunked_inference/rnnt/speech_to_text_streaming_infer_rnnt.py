"""Streaming inference for transducer models with a limited left context and a look-ahead (no left padding, decoder state carried
between chunks); latency = chunk + right context.

python .../speech_to_text_streaming_infer_rnnt.py model_path=m.nemo dataset_manifest=test.json chunk_secs=2 left_context_secs=10 right_context_secs=2
(reference script: ``examples/asr/asr_chunked_inference/rnnt/speech_to_text_streaming_infer_rnnt.py``)."""
import json

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate
from speech_b200.utils.streaming_buffers import AudioBatch, SimpleAudioDataset, streaming_transcribe_rnnt


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "output_filename": "streaming_transcripts.json",
                                            "chunk_secs": 2.0, "left_context_secs": 10.0, "right_context_secs": 2.0, "batch_size": 16}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    items = read_manifest(cfg.dataset_manifest)
    loader = torch.utils.data.DataLoader(SimpleAudioDataset([it["audio_filepath"] for it in items]), batch_size=cfg.batch_size,
                                         collate_fn=AudioBatch.collate_fn)
    preds = [""] * len(items)
    for batch in loader:
        hyps = streaming_transcribe_rnnt(model, batch.audio_signals, batch.audio_signal_lengths, cfg.chunk_secs, cfg.left_context_secs,
                                         cfg.right_context_secs)
        for i, h in zip(batch.ids.tolist(), hyps):
            preds[i] = h.text if getattr(h, "text", None) else model.decoding.decode_tokens_to_str([int(t) for t in h.y_sequence])
    with open(cfg.output_filename, "w", encoding="utf-8") as f:
        for it, p in zip(items, preds):
            f.write(json.dumps(dict(it, pred_text=p), ensure_ascii=False) + "\n")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate(preds, [it['text'] for it in items]):.2f}%")
    logging.info(f"latency {cfg.chunk_secs + cfg.right_context_secs:.2f} s")
    return preds


if __name__ == "__main__":
    main()

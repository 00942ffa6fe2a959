"""Simulate cache-aware streaming for one model over a manifest, chunk by chunk, and compare with offline decoding.

python .../speech_to_text_cache_aware_streaming_infer.py model_path=m.nemo dataset_manifest=test.json att_context_size=[70,13] batch_size=16
(reference script: ``examples/asr/asr_cache_aware_streaming/speech_to_text_cache_aware_streaming_infer.py``)."""
import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate
from speech_b200.utils.streaming_utils import CacheAwareStreamingAudioBuffer


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "dataset_manifest": None, "att_context_size": None, "batch_size": 16,
                                            "compare_vs_offline": True, "pad_and_drop_preencoded": False}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    if cfg.att_context_size is not None:
        model.encoder.set_default_att_context_size(list(cfg.att_context_size))
    model.encoder.setup_streaming_params()
    items = read_manifest(cfg.dataset_manifest)
    preds = []
    for s in range(0, len(items), cfg.batch_size):
        buf = CacheAwareStreamingAudioBuffer(model, pad_and_drop_preencoded=cfg.pad_and_drop_preencoded)
        for it in items[s:s + cfg.batch_size]:
            buf.append_audio(load_audio(it["audio_filepath"]))
        B = len(buf)
        clc, clt, clcl = model.encoder.get_initial_cache_state(batch_size=B)
        hyps, pred_out = None, None
        for step, (chunk, lens) in enumerate(buf):
            with torch.no_grad():
                out = model.conformer_stream_step(chunk, lens, clc, clt, clcl, keep_all_outputs=buf.is_buffer_empty(),
                                                  previous_hypotheses=hyps, previous_pred_out=pred_out,
                                                  drop_extra_pre_encoded=0 if step == 0 and not cfg.pad_and_drop_preencoded else None)
            pred_out, hyps, clc, clt, clcl = out[0], out[1], out[2], out[3], out[4]
        preds += [h.text for h in hyps]
    refs = [it.get("text", "") for it in items]
    if any(refs):
        logging.info(f"streaming WER: {100 * word_error_rate(preds, refs):.2f}%")
    if cfg.compare_vs_offline:
        off = model.transcribe([it["audio_filepath"] for it in items], batch_size=cfg.batch_size)
        off = [h.text if hasattr(h, "text") else h for h in off]
        logging.info(f"streaming vs offline disagreement: {100 * word_error_rate(preds, off):.2f}%")
    return preds


if __name__ == "__main__":
    main()

"""Streaming inference with continuous batching (cache-aware or buffered pipelines); reports RTFx.

python examples/asr/asr_streaming_inference/asr_streaming_infer.py --config-path ../conf/asr_streaming_inference \
    --config-name cache_aware_rnnt asr.model_name=model.nemo audio_file=manifest.json
(reference script: ``examples/asr/asr_streaming_inference/asr_streaming_infer.py``; RTFx ``:104-112``)."""
import json
import os

from speech_b200.core.config import hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.inference.pipelines import PipelineBuilder
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate


@hydra_runner(config_path="../conf/asr_streaming_inference", config_name="cache_aware_rnnt")
def main(cfg):
    src = cfg.audio_file
    if str(src).endswith(".json"):
        items = read_manifest(src)
    elif os.path.isdir(src):
        items = [{"audio_filepath": os.path.join(src, f)} for f in sorted(os.listdir(src)) if f.endswith(".wav")]
    else:
        items = [{"audio_filepath": src}]
    pipeline = PipelineBuilder.build_pipeline(cfg)
    outputs = pipeline.run([it["audio_filepath"] for it in items])
    out = cfg.get("output_filename") or "streaming_transcripts.json"
    with open(out, "w", encoding="utf-8") as f:
        for i, it in enumerate(items):
            o = outputs[i]
            f.write(json.dumps(dict(it, pred_text=o.text, words=[w.to_dict() for w in o.words]), ensure_ascii=False) + "\n")
    logging.info(f"wrote {len(items)} transcripts to {out}")
    if all(it.get("text") for it in items):
        logging.info(f"WER: {100 * word_error_rate([outputs[i].text for i in range(len(items))], [it['text'] for it in items]):.2f}%")
    if cfg.get("calculate_rtfx", True):
        logging.info(f"RTFx: {pipeline.rtfx():.1f} over {len(pipeline.step_times)} steps")


if __name__ == "__main__":
    main()

"""Evaluate an ASR model with (or without) one of its adapters on a manifest: WER with the adapter enabled, and with all adapters
disabled for comparison.

Usage: python examples/asr/asr_adapters/eval_asr_adapter.py model_path=adapted.nemo manifest=test.json [adapter_path=adapters.pt] \\
           [adapter_name=encoder:domain] [batch_size=16]
(reference script: ``examples/asr/asr_adapters/eval_asr_adapter.py``)."""
import json

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.metrics import word_error_rate


def evaluate(model, files, refs, batch_size):
    hyps = model.transcribe(files, batch_size=batch_size)
    texts = [h.text if hasattr(h, "text") else h for h in hyps]
    return word_error_rate(texts, refs)


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "manifest": None, "adapter_path": None, "adapter_name": None, "batch_size": 16}), cfg)
    model = ASRModel.restore_from(cfg.model_path).eval()
    if cfg.adapter_path:
        model.load_adapters(cfg.adapter_path, name=cfg.adapter_name)
    files, refs = [], []
    with open(cfg.manifest, encoding="utf-8") as f:
        for line in f:
            if line.strip():
                it = json.loads(line)
                files.append(it["audio_filepath"])
                refs.append(it.get("text", ""))
    results = {}
    if model.is_adapter_available():
        model.set_enabled_adapters(enabled=False)
        results["wer_without_adapters"] = evaluate(model, files, refs, cfg.batch_size)
        if cfg.adapter_name:
            model.set_enabled_adapters(cfg.adapter_name, True)
        else:
            model.set_enabled_adapters(enabled=True)
        results["wer_with_adapter"] = evaluate(model, files, refs, cfg.batch_size)
        results["enabled_adapters"] = model.get_enabled_adapters()
    else:
        results["wer_without_adapters"] = evaluate(model, files, refs, cfg.batch_size)
    print(json.dumps(results))
    return results


if __name__ == "__main__":
    main()

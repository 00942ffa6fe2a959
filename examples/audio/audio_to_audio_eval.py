"""Process the inputs of a manifest with an audio-to-audio model and score the outputs against the targets: SDR, SI-SDR, STOI,
and reference-free estimates when an estimator checkpoint is given.

python examples/audio/audio_to_audio_eval.py model_path=enh.nemo dataset_manifest=test.json input_key=noisy_filepath target_key=clean_filepath \
    metrics=[sdr,sisdr,stoi] output_dir=eval_out
(reference script: ``examples/audio/audio_to_audio_eval.py``)."""
import json
import os

import torch

from speech_b200.audio.metrics import AudioMetricWrapper, stoi
from speech_b200.audio.modules import sdr, si_sdr
from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT
from speech_b200.data.audio_to_text import load_audio, read_manifest, save_wav
from speech_b200.utils.logging import logging

DEFAULTS = {"model_path": None, "dataset_manifest": None, "input_key": "input_filepath", "target_key": "target_filepath", "output_dir": "a2a_eval",
            "metrics": ["sdr", "sisdr"], "sample_rate": 16000, "cuda": None, "write_audio": True, "only_score_manifest": False, "processed_key": "processed_filepath"}


def metric_fn(name: str, sr: int):
    if name == "sdr":
        return lambda p, t: sdr(p[:, None], t[:, None])[:, 0]
    if name == "sisdr":
        return lambda p, t: si_sdr(p[:, None], t[:, None])[:, 0]
    if name in ("stoi", "estoi"):
        return lambda p, t: torch.stack([stoi(a, b, sr, extended=(name == "estoi")) for a, b in zip(p, t)])
    raise ValueError(f"unknown metric {name}")


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    items = read_manifest(cfg.dataset_manifest)
    os.makedirs(cfg.output_dir, exist_ok=True)
    model = None
    if not cfg.only_score_manifest:
        dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
        model = ModelPT.restore_from(cfg.model_path, map_location=dev).to(dev).eval()
    sr = int(cfg.sample_rate)
    metrics = {m: AudioMetricWrapper(metric_fn(m, sr)) for m in cfg.metrics}
    rows = []
    for k, it in enumerate(items):
        tgt = torch.as_tensor(load_audio(it[cfg.target_key], target_sr=sr), dtype=torch.float32)
        if model is not None:
            x = torch.as_tensor(load_audio(it[cfg.input_key], target_sr=sr), dtype=torch.float32).to(next(model.parameters()).device)
            with torch.no_grad():
                out, _ = model(input_signal=x[None, None], input_length=torch.tensor([x.numel()], device=x.device))
            est = out[0, 0].float().cpu()
            if cfg.write_audio:
                p = os.path.join(cfg.output_dir, f"processed_{k:05d}.wav")
                save_wav(p, est.numpy(), sr)
                it = dict(it, **{cfg.processed_key: p})
        else:
            est = torch.as_tensor(load_audio(it[cfg.processed_key], target_sr=sr), dtype=torch.float32)
        n = min(est.numel(), tgt.numel())
        row = dict(it)
        for name, m in metrics.items():
            row[name] = float(m(est[None, :n], tgt[None, :n]))
        rows.append(row)
    with open(os.path.join(cfg.output_dir, "scores.json"), "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    summary = {name: float(m.compute()) for name, m in metrics.items()}
    logging.info(json.dumps(summary))
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()

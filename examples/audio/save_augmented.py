"""Write what the training pipeline would feed the model: every manifest entry passed through the configured perturbations
(noise, impulse responses, gain, speed, ...) and saved as audio with an updated manifest; for listening checks and for
freezing an augmented evaluation set.

python examples/audio/save_augmented.py manifest=clean.json output_dir=aug "augmentor={noise: {prob: 1.0, manifest_path: noise.json, min_snr_db: 5, max_snr_db: 15}}" [num_copies=1 seed=0]
(reference script: ``examples/audio/save_augmented.py``)."""
import json
import os

import numpy as np

from speech_b200.core.config import OmegaConf, hydra_runner, to_container
from speech_b200.data.audio_to_text import load_audio, read_manifest, save_wav
from speech_b200.data.perturb import AudioSegment, process_augmentations


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"manifest": None, "output_dir": "augmented", "augmentor": None, "num_copies": 1, "sample_rate": 16000, "seed": 0}), cfg)
    aug = process_augmentations(to_container(cfg.augmentor, resolve=True)) if cfg.augmentor is not None else None
    os.makedirs(cfg.output_dir, exist_ok=True)
    np.random.seed(int(cfg.seed))
    if aug is not None:
        import random

        aug._rng = random.Random(int(cfg.seed))
    rows = []
    for it in read_manifest(cfg.manifest):
        x = load_audio(it["audio_filepath"], target_sr=cfg.sample_rate, offset=float(it.get("offset", 0) or 0), duration=it.get("duration"))
        for c in range(int(cfg.num_copies)):
            y = x
            if aug is not None:
                seg = AudioSegment(x.copy(), cfg.sample_rate)
                aug.perturb(seg)
                y = seg.samples
            name = os.path.splitext(os.path.basename(it["audio_filepath"]))[0] + f"_aug{c}.wav"
            p = os.path.join(cfg.output_dir, name)
            save_wav(p, np.asarray(y, dtype=np.float32), cfg.sample_rate)
            rows.append(dict(it, audio_filepath=p, offset=0, duration=round(len(y) / cfg.sample_rate, 4), source_audio_filepath=it["audio_filepath"]))
    with open(os.path.join(cfg.output_dir, "manifest.json"), "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    return rows


if __name__ == "__main__":
    main()

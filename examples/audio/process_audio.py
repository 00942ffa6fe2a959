"""Run an audio-to-audio model over files and write the processed audio (reference: ``examples/audio/process_audio.py``).

python examples/audio/process_audio.py model_path=enh.nemo audio_dir=noisy/ output_dir=enhanced/"""
import os

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.core.modelpt import ModelPT


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create({"model_path": None, "audio_dir": None, "output_dir": "processed"}), cfg)
    model = ModelPT.restore_from(cfg.model_path).eval()
    files = sorted(os.path.join(cfg.audio_dir, f) for f in os.listdir(cfg.audio_dir) if f.endswith(".wav"))
    model.process(files, output_dir=cfg.output_dir)


if __name__ == "__main__":
    main()

"""Train an audio-to-audio (enhancement / separation) model; ``model_class`` in the config picks the class
(reference script: ``examples/audio/audio_to_audio_train.py``).

python examples/audio/audio_to_audio_train.py --config-name flow_matching_generative model.train_ds.manifest_filepath=train.json ..."""
from speech_b200.audio import models as audio_models
from speech_b200.core.config import hydra_runner
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="conf", config_name="flow_matching_generative")
def main(cfg):
    run_training(getattr(audio_models, cfg.get("model_class", "EncMaskDecAudioToAudioModel")), cfg)


if __name__ == "__main__":
    main()

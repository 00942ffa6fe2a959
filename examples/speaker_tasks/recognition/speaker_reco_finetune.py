"""Fine-tune a speaker model on new speakers: the encoder is initialised from a checkpoint (``init_from_nemo_model`` /
``init_from_pretrained_model`` with ``exclude: [decoder.final]`` so that the classification layer is rebuilt for the new label set).

Usage: python examples/speaker_tasks/recognition/speaker_reco_finetune.py +init_from_nemo_model.model0.path=titanet.nemo \
    "+init_from_nemo_model.model0.exclude=[decoder.final]" model.decoder.num_classes=<n> model.train_ds.manifest_filepath=...
(reference script: ``examples/speaker_tasks/recognition/speaker_reco_finetune.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecSpeakerLabelModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../diarization/conf", config_name="titanet-small")
def main(cfg):
    if not (cfg.get("init_from_nemo_model") or cfg.get("init_from_pretrained_model") or cfg.get("init_from_ptl_ckpt")):
        raise ValueError("fine-tuning needs init_from_nemo_model / init_from_pretrained_model / init_from_ptl_ckpt")
    run_training(EncDecSpeakerLabelModel, cfg)


if __name__ == "__main__":
    main()

"""Train the FastPitch variant that is conditioned on self-supervised content and speaker embeddings (voice conversion / zero-shot TTS back end).
The features come from a trained ``SSLDisentangler`` (content embeddings, speaker embedding) and are stored per utterance as ``.pt`` dictionaries
named by ``feature_filepath`` in the manifest; ``hifi_ckpt_path`` names the vocoder used to render validation audio.

python examples/tts/fastpitch_ssl.py model.train_ds.manifest_filepath=train_feats.json model.validation_ds.manifest_filepath=val_feats.json \
    [hifi_ckpt_path=hifigan.nemo] [finetune=true +init_from_nemo_model=base.nemo]
(reference script: ``examples/tts/fastpitch_ssl.py``)."""
from speech_b200.core.config import OmegaConf, hydra_runner, to_container
from speech_b200.tts.fastpitch_ssl import FastPitchModel_SSL
from speech_b200.utils.exp_manager import exp_manager
from speech_b200.utils.launch import build_trainer


@hydra_runner(config_path="conf", config_name="fastpitch_ssl")
def main(cfg):
    trainer = build_trainer(cfg)
    exp_manager(trainer, cfg.get("exp_manager", None))
    vocoder = None
    if cfg.get("hifi_ckpt_path"):
        from speech_b200.tts.classic import HifiGanModel

        vocoder = HifiGanModel.restore_from(cfg.hifi_ckpt_path, map_location="cpu").eval()
    model = FastPitchModel_SSL(cfg=OmegaConf.create(to_container(cfg.model, resolve=True)), trainer=trainer, vocoder=vocoder)
    if cfg.get("finetune", False):
        model.maybe_init_from_pretrained_checkpoint(cfg)
    trainer.fit(model)
    return model


if __name__ == "__main__":
    main()

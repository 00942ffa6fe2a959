"""Train a speech-translation model: Conformer encoder + Transformer decoder with a sub-word tokenizer on the target language,
validated with BLEU.

Usage: python examples/asr/speech_translation/speech_to_text_transformer.py model.train_ds.manifest_filepath=... key=value ...
(reference script: ``examples/asr/speech_translation/speech_to_text_transformer.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecTransfModelBPE
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/speech_translation", config_name="fast-conformer_transformer")
def main(cfg):
    run_training(EncDecTransfModelBPE, cfg)


if __name__ == "__main__":
    main()

"""Train a multi-talker transducer: speaker kernels inside the encoder select one speaker of an overlapped recording; batches
carry the target speaker's activity and the activity of everyone else.

Usage: python examples/asr/asr_transducer/speech_to_text_mt_rnnt_bpe.py model.spk_kernel_layers=[0] model.add_bg_spk_kernel=true key=value ...
(reference script: ``examples/asr/asr_transducer/speech_to_text_mt_rnnt_bpe.py``)."""
from speech_b200.core.config import hydra_runner
from speech_b200.models import EncDecMultiTalkerRNNTBPEModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf/fastconformer", config_name="fast-conformer_transducer_bpe")
def main(cfg):
    run_training(EncDecMultiTalkerRNNTBPEModel, cfg)


if __name__ == "__main__":
    main()

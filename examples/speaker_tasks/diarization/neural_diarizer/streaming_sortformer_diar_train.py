"""Train the streaming Sortformer diarizer: the same network as the offline model run chunk by chunk with its speaker cache and
FIFO during training, so that the cache-update rule is learned in the loop.

Usage: python .../streaming_sortformer_diar_train.py model.streaming_mode=true model.sortformer_modules.chunk_len=188 key=value ...
(reference script: ``examples/speaker_tasks/diarization/neural_diarizer/streaming_sortformer_diar_train.py``)."""
from speech_b200.core.config import hydra_runner, open_dict
from speech_b200.models import SortformerEncLabelModel
from speech_b200.utils.launch import run_training


@hydra_runner(config_path="../conf", config_name="sortformer_diarizer_4spk")
def main(cfg):
    with open_dict(cfg):
        cfg.model.streaming_mode = True
    run_training(SortformerEncLabelModel, cfg)


if __name__ == "__main__":
    main()

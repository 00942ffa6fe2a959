"""Transcribe a manifest with a transducer exported to ONNX (``encoder.onnx`` + ``decoder_joint.onnx``) through ONNX Runtime and compare with the
framework's greedy decoding.  Needs the ``onnx`` and ``onnxruntime`` packages; without them the script says so and exits (use the TorchScript
variant next to this file instead).

python examples/asr/export/transducer/infer_transducer_onnx.py nemo_model=model.nemo dataset_manifest=test.json onnx_encoder=encoder.onnx onnx_decoder=decoder_joint.onnx
(reference script: ``examples/asr/export/transducer/infer_transducer_onnx.py``)."""
import sys

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.decoding.exported_rnnt import ONNXGreedyBatchedRNNTInfer
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"nemo_model": None, "pretrained_model": None, "dataset_manifest": None, "onnx_encoder": None, "onnx_decoder": None, "batch_size": 8,
            "max_symbols_per_step": 10}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    model = (ASRModel.restore_from(cfg.nemo_model, map_location="cpu") if cfg.nemo_model else ASRModel.from_pretrained(cfg.pretrained_model)).eval()
    try:
        infer = ONNXGreedyBatchedRNNTInfer(cfg.onnx_encoder, cfg.onnx_decoder, blank_id=model.decoding.blank_id, pred_layers=model.decoder.pred_rnn_layers,
                                           pred_hidden=model.decoder.pred_hidden, max_symbols_per_step=cfg.max_symbols_per_step,
                                           durations=list(getattr(model.decoding, "durations", None) or []))
    except RuntimeError as e:
        logging.error(str(e))
        sys.exit(2)
    from infer_transducer_ts import transcribe_exported            # same loop over the manifest; only the graph runner differs

    items = read_manifest(cfg.dataset_manifest)
    exported = transcribe_exported(model, infer, items, int(cfg.batch_size))
    native = [h.text if hasattr(h, "text") else h for h in model.transcribe([it["audio_filepath"] for it in items], batch_size=int(cfg.batch_size))]
    refs = [it.get("text", "") for it in items]
    logging.info(f"WER ONNX {100 * word_error_rate(exported, refs):.2f}%  framework {100 * word_error_rate(native, refs):.2f}%")


if __name__ == "__main__":
    main()

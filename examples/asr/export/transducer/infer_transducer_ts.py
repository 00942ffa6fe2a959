"""Export a transducer's encoder and decoder+joint step to TorchScript, transcribe a manifest with the exported graphs only, and compare with
the framework's own greedy decoding (WER of both, and how many transcripts differ).

python examples/asr/export/transducer/infer_transducer_ts.py nemo_model=model.nemo dataset_manifest=test.json export_dir=exported batch_size=8
python examples/asr/export/transducer/infer_transducer_ts.py nemo_model=model.nemo dataset_manifest=test.json \
    ts_encoder=exported/encoder.ts ts_decoder=exported/decoder_joint.ts        # reuse graphs exported earlier
(reference script: ``examples/asr/export/transducer/infer_transducer_ts.py``)."""
import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.decoding.exported_rnnt import TorchscriptGreedyBatchedRNNTInfer, export_transducer_subnets
from speech_b200.models.asr_model import ASRModel
from speech_b200.utils.logging import logging
from speech_b200.utils.metrics import word_error_rate

DEFAULTS = {"nemo_model": None, "pretrained_model": None, "dataset_manifest": None, "export_dir": "exported_transducer", "ts_encoder": None, "ts_decoder": None,
            "batch_size": 8, "max_symbols_per_step": 10, "cuda": None}


def build_exported_decoder(model, cfg):
    enc_path, dec_path = cfg.ts_encoder, cfg.ts_decoder
    if not enc_path or not dec_path:
        enc_path, dec_path = export_transducer_subnets(model, cfg.export_dir)
        logging.info(f"exported {enc_path} and {dec_path}")
    durations = list(getattr(model.decoding, "durations", None) or [])
    return TorchscriptGreedyBatchedRNNTInfer(enc_path, dec_path, blank_id=model.decoding.blank_id, pred_layers=model.decoder.pred_rnn_layers,
                                             pred_hidden=model.decoder.pred_hidden, max_symbols_per_step=cfg.max_symbols_per_step, durations=durations,
                                             device=str(next(model.parameters()).device))


def transcribe_exported(model, infer, items, batch_size):
    dev = next(model.parameters()).device
    sr = model.preprocessor._sample_rate if hasattr(model.preprocessor, "_sample_rate") else 16000
    texts = []
    for s in range(0, len(items), batch_size):
        xs = [torch.as_tensor(load_audio(it["audio_filepath"], sr)) for it in items[s:s + batch_size]]
        lens = torch.tensor([len(x) for x in xs])
        audio = torch.nn.utils.rnn.pad_sequence(xs, batch_first=True)
        with torch.no_grad():
            feats, flen = model.preprocessor(input_signal=audio.to(dev), length=lens.to(dev))       # the front end stays in the framework; the graphs start at features
        for ids in infer(feats, flen):
            texts.append(model.decoding.decode_tokens_to_str(ids))
    return texts


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if not torch.cuda.is_available() or (cfg.cuda is not None and int(cfg.cuda) < 0) else f"cuda:{cfg.cuda or 0}"
    model = (ASRModel.restore_from(cfg.nemo_model, map_location=dev) if cfg.nemo_model else ASRModel.from_pretrained(cfg.pretrained_model)).to(dev).eval()
    items = read_manifest(cfg.dataset_manifest)
    infer = build_exported_decoder(model, cfg)
    exported = transcribe_exported(model, infer, items, int(cfg.batch_size))
    native = [h.text if hasattr(h, "text") else h for h in model.transcribe([it["audio_filepath"] for it in items], batch_size=int(cfg.batch_size))]
    refs = [it.get("text", "") for it in items]
    differ = sum(a != b for a, b in zip(exported, native))
    logging.info(f"WER exported graphs {100 * word_error_rate(exported, refs):.2f}%  framework {100 * word_error_rate(native, refs):.2f}%  transcripts that differ: {differ} / {len(items)}")
    return exported, native


if __name__ == "__main__":
    main()

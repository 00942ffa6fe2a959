"""Turn a hybrid transducer + CTC checkpoint into a plain CTC (or plain transducer) checkpoint: the encoder and the chosen head
are kept, the other head and its loss are dropped.  Works on the archive itself (config + weights + tokenizer artifacts), so the
hybrid model is never built.

python convert_nemo_asr_hybrid_to_ctc.py -i hybrid.nemo -o ctc.nemo -t ctc
(reference script: ``examples/asr/asr_hybrid_transducer_ctc/helpers/convert_nemo_asr_hybrid_to_ctc.py``)."""
import argparse
import os
import tempfile

import torch

from speech_b200.core.config import OmegaConf, open_dict
from speech_b200.core.save_restore import SaveRestoreConnector


def convert(src: str, dst: str, model_type: str = "ctc") -> str:
    conn = SaveRestoreConnector()
    with tempfile.TemporaryDirectory() as tmp:
        conn._unpack_nemo_file(src, tmp)
        cfg_path, w_path = os.path.join(tmp, conn.model_config_yaml), os.path.join(tmp, conn.model_weights_ckpt)
        cfg = OmegaConf.load(cfg_path)
        if "aux_ctc" not in cfg:
            raise ValueError("the checkpoint has no aux_ctc section: not a hybrid model")
        bpe = cfg.get("tokenizer") is not None
        sd = torch.load(w_path, map_location="cpu", weights_only=False)
        with open_dict(cfg):
            aux = cfg.pop("aux_ctc")
            if model_type == "ctc":
                for k in ("joint", "loss", "decoding"):
                    cfg.pop(k, None)
                cfg.decoder = aux.decoder
                if aux.get("decoding") is not None:
                    cfg.decoding = aux.decoding
                cfg.target = "speech_b200.models.ctc_models." + ("EncDecCTCModelBPE" if bpe else "EncDecCTCModel")
                keep = {}
                for k, v in sd.items():
                    if k.startswith("ctc_decoder."):
                        keep["decoder." + k[len("ctc_decoder."):]] = v
                    elif not k.startswith(("decoder.", "joint.", "ctc_")):
                        keep[k] = v
                if cfg.decoder.get("feat_in") is None:
                    cfg.decoder.feat_in = int(next(v for k, v in keep.items() if k.startswith("decoder.") and v.dim() >= 2).shape[1])
                n_out = int(next(v for k, v in keep.items() if k.startswith("decoder.") and v.dim() >= 2).shape[0])
                if int(cfg.decoder.get("num_classes", -1) or -1) < 1:
                    cfg.decoder.num_classes = n_out - 1
            else:
                cfg.target = "speech_b200.models.rnnt_models." + ("EncDecRNNTBPEModel" if bpe else "EncDecRNNTModel")
                keep = {k: v for k, v in sd.items() if not k.startswith("ctc_")}
        OmegaConf.save(cfg, cfg_path)
        torch.save(keep, w_path)
        conn._make_nemo_file_from_folder(os.path.abspath(dst), tmp)
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--input", required=True)
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("-t", "--model_type", choices=["ctc", "rnnt"], default="ctc")
    a = ap.parse_args()
    print(convert(a.input, a.output, a.model_type))

"""Who-spoke-what transcription of overlapped recordings, chunk by chunk: a streaming diarizer finds the active speakers and the
multi-talker transducer keeps one cache-aware instance per speaker.  Output: SegLST (one record per sentence and speaker).

python .../speech_to_text_multitalker_streaming_infer.py asr_model=mt.nemo diar_model=sortformer.nemo manifest_file=mix.json output_path=out.seglst.json \
    [offline=false max_num_of_spks=4 att_context_size=[70,13]]
(reference script: ``examples/asr/asr_cache_aware_streaming/speech_to_text_multitalker_streaming_infer.py``)."""
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import load_audio, read_manifest
from speech_b200.models import EncDecMultiTalkerRNNTBPEModel, SortformerEncLabelModel
from speech_b200.models.multitalker import SpeakerTaggedASR, write_seglst
from speech_b200.utils.logging import logging

DEFAULTS = {"asr_model": None, "diar_model": None, "manifest_file": None, "audio_file": None, "output_path": "output.seglst.json", "offline": False,
            "max_num_of_spks": 4, "threshold": 0.5, "att_context_size": None, "masked_asr": False, "sentence_max_gap": 1.0, "cuda": None}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    asr = EncDecMultiTalkerRNNTBPEModel.restore_from(cfg.asr_model, map_location=dev).to(dev).eval()
    diar = SortformerEncLabelModel.restore_from(cfg.diar_model, map_location=dev).to(dev).eval()
    if cfg.att_context_size is not None:
        asr.encoder.set_default_att_context_size(list(cfg.att_context_size))
    diar.streaming_mode = not cfg.offline

    def diarize(audio, lens):
        with torch.no_grad():
            return diar(audio_signal=audio, audio_signal_length=lens)

    tagger = SpeakerTaggedASR(asr, diarize, threshold=cfg.threshold, max_num_of_spks=cfg.max_num_of_spks, max_gap=cfg.sentence_max_gap, masked_asr=cfg.masked_asr)
    items = read_manifest(cfg.manifest_file) if cfg.manifest_file else [{"audio_filepath": cfg.audio_file}]
    seglst = []
    for it in items:
        x = torch.as_tensor(load_audio(it["audio_filepath"]), dtype=torch.float32, device=dev)
        sid = it.get("session_id") or os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        if cfg.offline:
            seglst += tagger.transcribe_offline(x[None], torch.tensor([x.numel()], device=dev), [sid])
        else:
            seglst += tagger.stream(x, session_id=sid)
    write_seglst(cfg.output_path, seglst)
    logging.info(f"{len(seglst)} sentences of {len({(d['session_id'], d['speaker']) for d in seglst})} speakers -> {cfg.output_path}")
    return seglst


if __name__ == "__main__":
    main()

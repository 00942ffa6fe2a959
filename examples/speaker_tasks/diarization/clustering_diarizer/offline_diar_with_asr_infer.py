"""Diarization joined with recognition: words with timestamps from an ASR model are assigned to the speaker who is active at
the middle of the word; output is a per-recording JSON with speaker-labelled sentences and a SegLST file.

python .../offline_diar_with_asr_infer.py diarizer.manifest_filepath=m.json diarizer.out_dir=out diarizer.asr.model_path=asr.nemo \
    diarizer.speaker_embeddings.model_path=titanet.nemo [diarizer.vad.model_path=vad.nemo]
(reference script: ``examples/speaker_tasks/diarization/clustering_diarizer/offline_diar_with_asr_infer.py``)."""
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.models.diarizers import ClusteringDiarizer
from speech_b200.models.diar_with_asr import OfflineDiarWithASR
from speech_b200.models.multitalker import write_seglst
from speech_b200.utils.logging import logging


def words_with_times(model, path: str):
    """``[{"word", "start_time", "end_time"}]`` from the model's word timestamps (frame offsets times the encoder frame length
    unless the hypothesis already carries seconds)."""
    h = model.transcribe([path], batch_size=1, return_hypotheses=True, timestamps=True)[0]
    ts = h.timestamp if isinstance(h.timestamp, dict) else {}
    spf = float(model.cfg.preprocessor.get("window_stride", 0.01)) * int(model.encoder.subsampling_factor)
    out = []
    for w in ts.get("word", []):
        a = float(w["start"]) if "start" in w else float(w.get("start_offset", 0)) * spf
        b = float(w["end"]) if "end" in w else float(w.get("end_offset", 0)) * spf
        out.append({"word": w["word"], "start_time": a, "end_time": b})
    return out


@hydra_runner(config_path="../conf", config_name="diar_infer_general")
def main(cfg):
    d = cfg.diarizer
    os.makedirs(d.out_dir, exist_ok=True)
    diar = ClusteringDiarizer(cfg)
    asr = ASRModel.restore_from(d.asr.model_path, map_location="cuda" if torch.cuda.is_available() else "cpu").eval()
    pipe = OfflineDiarWithASR(word_anchor=d.get("asr", {}).get("word_ts_anchor_pos", "mid") if d.get("asr") else "mid")
    diar_labels, word_ts = {}, {}
    for it in read_manifest(d.manifest_filepath):
        uid = os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        segs = list(diar.diarize([it["audio_filepath"]], [it.get("num_speakers")]).values())[0]
        diar_labels[uid] = [f"{a:.3f} {b:.3f} {s}" for a, b, s in segs]
        word_ts[uid] = words_with_times(asr, it["audio_filepath"])
    result = pipe.get_transcript_with_speaker_labels(diar_labels, word_ts)
    OfflineDiarWithASR.write_outputs(result, d.out_dir)
    seglst = [{"session_id": uid, "speaker": s["speaker"], "start_time": round(s["start_time"], 3), "end_time": round(s["end_time"], 3), "words": s["text"]}
              for uid, r in result.items() for s in r["sentences"]]
    write_seglst(os.path.join(d.out_dir, "all.seglst.json"), seglst)
    logging.info(f"{len(seglst)} sentences -> {d.out_dir}")
    return result


if __name__ == "__main__":
    main()

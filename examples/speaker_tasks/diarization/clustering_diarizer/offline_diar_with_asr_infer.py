"""Diarization joined with recognition: words with timestamps from an ASR model are assigned to the speaker who is active at
the middle of the word; output is a per-recording JSON with speaker-labelled sentences and a SegLST file.

python .../offline_diar_with_asr_infer.py diarizer.manifest_filepath=m.json diarizer.out_dir=out diarizer.asr.model_path=asr.nemo \
    diarizer.speaker_embeddings.model_path=titanet.nemo [diarizer.vad.model_path=vad.nemo]
(reference script: ``examples/speaker_tasks/diarization/clustering_diarizer/offline_diar_with_asr_infer.py``)."""
import json
import os

import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models.asr_model import ASRModel
from speech_b200.models.diarizers import ClusteringDiarizer
from speech_b200.models.multitalker import sentences_from_words, write_seglst
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


def assign_speakers(words, segments):
    """``segments``: ``(start, end, speaker)``; a word goes to the segment that holds its mid-point, else to the nearest one."""
    out = []
    for w in words:
        mid = 0.5 * (w["start_time"] + w["end_time"])
        best = min(segments, key=lambda s: 0.0 if s[0] <= mid <= s[1] else min(abs(mid - s[0]), abs(mid - s[1]))) if segments else (0, 0, "speaker_0")
        out.append(dict(w, speaker=best[2]))
    return out


@hydra_runner(config_path="../conf", config_name="diar_infer_general")
def main(cfg):
    d = cfg.diarizer
    os.makedirs(d.out_dir, exist_ok=True)
    diar = ClusteringDiarizer(cfg)
    asr = ASRModel.restore_from(d.asr.model_path, map_location="cuda" if torch.cuda.is_available() else "cpu").eval()
    seglst = []
    for it in read_manifest(d.manifest_filepath):
        uid = os.path.splitext(os.path.basename(it["audio_filepath"]))[0]
        segs = list(diar.diarize([it["audio_filepath"]], [it.get("num_speakers")]).values())[0]
        words = assign_speakers(words_with_times(asr, it["audio_filepath"]), segs)
        sents = []
        for spk in sorted({w["speaker"] for w in words}):
            sents += sentences_from_words([w for w in words if w["speaker"] == spk], uid, spk)
        sents.sort(key=lambda s: s["start_time"])
        with open(os.path.join(d.out_dir, uid + ".json"), "w", encoding="utf-8") as f:
            json.dump({"session_id": uid, "speaker_count": len({s["speaker"] for s in sents}), "sentences": sents, "words": words}, f, indent=2)
        seglst += sents
    write_seglst(os.path.join(d.out_dir, "all.seglst.json"), seglst)
    logging.info(f"{len(seglst)} sentences -> {d.out_dir}")


if __name__ == "__main__":
    main()

"""Write the speaker embedding of every manifest entry to a pickle ``{unique id: vector}``.

python examples/speaker_tasks/recognition/extract_speaker_embeddings.py --manifest=m.json --model_path=titanet.nemo --embedding_dir=out/
(reference script: ``examples/speaker_tasks/recognition/extract_speaker_embeddings.py``)."""
import argparse
import os
import pickle

import numpy as np
import torch

from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models import EncDecSpeakerLabelModel


def unique_id(path: str, levels: int = 3) -> str:
    """The last ``levels`` path components joined by ``@`` (speaker / session / file in the usual corpus layouts)."""
    return "@".join(os.path.splitext(path)[0].split(os.sep)[-levels:])


def extract(model, manifest: str, embedding_dir: str, batch_size: int = 32) -> str:
    items = read_manifest(manifest)
    embs = np.asarray(model.batch_inference([it["audio_filepath"] for it in items], batch_size=batch_size)[0])
    embs = embs / np.maximum(np.linalg.norm(embs, axis=1, keepdims=True), 1e-9)
    out = {unique_id(it["audio_filepath"]): e for it, e in zip(items, embs)}
    os.makedirs(os.path.join(embedding_dir, "embeddings"), exist_ok=True)
    path = os.path.join(embedding_dir, "embeddings", os.path.splitext(os.path.basename(manifest))[0] + "_embeddings.pkl")
    with open(path, "wb") as f:
        pickle.dump(out, f)
    return path


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--manifest", required=True)
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--embedding_dir", default="./")
    ap.add_argument("--batch_size", type=int, default=32)
    a = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    m = (EncDecSpeakerLabelModel.restore_from(a.model_path, map_location=dev) if a.model_path.endswith(".nemo") else EncDecSpeakerLabelModel.from_pretrained(a.model_path)).to(dev).eval()
    print(extract(m, a.manifest, a.embedding_dir, a.batch_size))

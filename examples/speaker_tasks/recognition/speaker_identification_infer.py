"""Identify the speaker of test utterances among enrolled speakers: by cosine similarity to the enrolled speakers' mean embeddings
(``backend=cosine_similarity``) or by a small classifier trained on the enrolment embeddings (``backend=neural_classifier``).

python examples/speaker_tasks/recognition/speaker_identification_infer.py model_path=titanet.nemo data.enrollment_manifest=enroll.json \
    data.test_manifest=test.json data.out_manifest=out.json backend.backend_model=cosine_similarity
(reference script: ``examples/speaker_tasks/recognition/speaker_identification_infer.py``)."""
import json

import numpy as np
import torch

from speech_b200.core.config import OmegaConf, hydra_runner
from speech_b200.data.audio_to_text import read_manifest
from speech_b200.models import EncDecSpeakerLabelModel
from speech_b200.utils.logging import logging

DEFAULTS = {"model_path": None, "batch_size": 32, "cuda": None,
            "data": {"enrollment_manifest": None, "test_manifest": None, "out_manifest": "speaker_id_out.json", "sample_rate": 16000},
            "backend": {"backend_model": "cosine_similarity", "cosine_similarity": {"threshold": None},
                        "neural_classifier": {"epochs": 200, "lr": 0.05, "weight_decay": 1e-3}}}


@hydra_runner(config_path=None, config_name=None)
def main(cfg):
    cfg = OmegaConf.merge(OmegaConf.create(DEFAULTS), cfg)
    dev = "cpu" if (cfg.cuda is not None and int(cfg.cuda) < 0) or not torch.cuda.is_available() else f"cuda:{cfg.cuda or 0}"
    model = EncDecSpeakerLabelModel.restore_from(cfg.model_path, map_location=dev).to(dev).eval()
    enroll, test = read_manifest(cfg.data.enrollment_manifest), read_manifest(cfg.data.test_manifest)
    norm = lambda e: e / np.maximum(np.linalg.norm(e, axis=1, keepdims=True), 1e-9)  # noqa: E731
    e_emb = norm(np.asarray(model.batch_inference([it["audio_filepath"] for it in enroll], batch_size=cfg.batch_size)[0]))
    t_emb = norm(np.asarray(model.batch_inference([it["audio_filepath"] for it in test], batch_size=cfg.batch_size)[0]))
    speakers = sorted({it["label"] for it in enroll})
    ids = np.asarray([speakers.index(it["label"]) for it in enroll])
    if cfg.backend.backend_model == "cosine_similarity":
        center = e_emb.mean(0, keepdims=True)                     # the part all speakers share carries no identity
        e_emb, t_emb = norm(e_emb - center), norm(t_emb - center)
        cents = norm(np.stack([e_emb[ids == k].mean(0) for k in range(len(speakers))]))
        sim = t_emb @ cents.T
        pred, score = sim.argmax(1), sim.max(1)
        thr = cfg.backend.cosine_similarity.threshold
        names = [speakers[p] if thr is None or s >= float(thr) else "unknown" for p, s in zip(pred, score)]
    elif cfg.backend.backend_model == "neural_classifier":
        nc = cfg.backend.neural_classifier
        clf = torch.nn.Linear(e_emb.shape[1], len(speakers))
        opt = torch.optim.Adam(clf.parameters(), lr=nc.lr, weight_decay=nc.weight_decay)
        mu, sd = e_emb.mean(0, keepdims=True), e_emb.std(0, keepdims=True) + 1e-6        # embeddings of one model share a large common part
        e_emb, t_emb = (e_emb - mu) / sd, (t_emb - mu) / sd
        X, Y = torch.tensor(e_emb, dtype=torch.float32), torch.tensor(ids)
        for _ in range(int(nc.epochs)):
            opt.zero_grad()
            torch.nn.functional.cross_entropy(clf(X), Y).backward()
            opt.step()
        with torch.no_grad():
            prob = torch.softmax(clf(torch.tensor(t_emb, dtype=torch.float32)), -1)
        score, pred = prob.max(1)
        names, score = [speakers[int(p)] for p in pred], score.numpy()
    else:
        raise ValueError(f"unknown backend {cfg.backend.backend_model}")
    with open(cfg.data.out_manifest, "w", encoding="utf-8") as f:
        for it, n, s in zip(test, names, score):
            f.write(json.dumps(dict(it, infer=n, score=float(s))) + "\n")
    if all("label" in it for it in test):
        acc = float(np.mean([n == it["label"] for n, it in zip(names, test)]))
        logging.info(f"identification accuracy {100 * acc:.2f}%")
        print(f"accuracy: {acc:.4f}")
    return names


if __name__ == "__main__":
    main()

"""Equal error rate and minimum detection cost of a trial list scored by cosine similarity of stored embeddings.

python examples/speaker_tasks/recognition/voxceleb_eval.py --trial_file=trials.txt --emb=embeddings.pkl
Trial file lines: ``<1|0> <utterance a> <utterance b>`` (paths; ids are derived as in ``extract_speaker_embeddings.py``).
(reference script: ``examples/speaker_tasks/recognition/voxceleb_eval.py``)."""
import argparse
import pickle

import numpy as np

from extract_speaker_embeddings import unique_id


def eer_and_min_dcf(scores: np.ndarray, labels: np.ndarray, p_target: float = 0.05, c_miss: float = 1.0, c_fa: float = 1.0):
    """Sweeps the threshold over the sorted scores: EER where miss rate = false-alarm rate (linear interpolation between the two
    neighbouring operating points), and the minimum of the normalised detection cost."""
    order = np.argsort(-scores, kind="stable")
    y = labels[order].astype(bool)
    n_t, n_n = max(1, int(y.sum())), max(1, int((~y).sum()))
    fa = np.concatenate([[0.0], np.cumsum(~y) / n_n])
    miss = np.concatenate([[1.0], 1.0 - np.cumsum(y) / n_t])
    d = miss - fa
    k = int(np.argmax(d <= 0))
    if k == 0:
        eer = float(fa[0])
    else:
        t = d[k - 1] / (d[k - 1] - d[k]) if d[k - 1] != d[k] else 0.0
        eer = float(fa[k - 1] + t * (fa[k] - fa[k - 1]))
    dcf = c_miss * miss * p_target + c_fa * fa * (1 - p_target)
    return eer, float(dcf.min() / min(c_miss * p_target, c_fa * (1 - p_target)))


def evaluate(trial_file: str, emb_file: str):
    emb = pickle.load(open(emb_file, "rb"))
    scores, labels = [], []
    for line in open(trial_file, encoding="utf-8"):
        parts = line.split()
        if len(parts) != 3:
            continue
        a, b = emb[unique_id(parts[1])], emb[unique_id(parts[2])]
        scores.append(float(np.dot(a, b) / max(1e-9, np.linalg.norm(a) * np.linalg.norm(b))))
        labels.append(int(parts[0]))
    return eer_and_min_dcf(np.asarray(scores), np.asarray(labels))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--trial_file", required=True)
    ap.add_argument("--emb", required=True)
    a = ap.parse_args()
    eer, dcf = evaluate(a.trial_file, a.emb)
    print(f"EER: {100 * eer:.2f}%  minDCF: {dcf:.4f}")

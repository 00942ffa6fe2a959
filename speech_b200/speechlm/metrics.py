"""Evaluation metrics of the speech-LLM collection: turn taking of duplex models, multiple-choice answer extraction and
accuracy, empty-response rate, and a results logger that merges per-rank prediction files.

Behaviour follows ``speechlm2/parts/metrics`` of the reference (``turn_taking.py:18-130``: first user end-of-turn against the first
agent start, tolerance in frames, latency = frames x frame duration; ``mcq_evaluator.py:94-260``: the letter chosen in free-form
answers; ``empty_text.py``; ``results_logger.py:77-350``: per-rank JSON-lines files merged on rank 0 with per-dataset metrics).
WER / BLEU / token accuracy / perplexity live in ``speechlm/parts.py``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Dict, Iterable, List, Optional, Sequence

import torch


# ------------------------------------------------------------------------------------------------ turn taking
def compute_turn_taking_metrics(source_tokens: torch.Tensor, pred_tokens: torch.Tensor, eos_token_id: int, bos_token_id: int,
                                tolerance: int = 13, latency_multiplier: float = 0.08):
    """``source_tokens`` [B, T]: the user's channel (its first ``eos_token_id`` ends the user's turn); ``pred_tokens`` [B, T]: the
    agent's channel (its first ``bos_token_id`` starts the answer).  A turn counts as taken when the two are at most ``tolerance``
    frames apart.  Returns ``(accuracy over rows with a user end, mean latency in seconds of the successful rows)``; a row in
    which the agent never starts counts as a failure."""
    src, prd = source_tokens.detach().cpu(), pred_tokens.detach().cpu()
    ok = total = 0
    lat: List[float] = []
    for b in range(src.shape[0]):
        e = (src[b] == eos_token_id).nonzero().flatten()
        if e.numel() == 0:
            continue
        total += 1
        s = (prd[b] == bos_token_id).nonzero().flatten()
        if s.numel() == 0:
            continue
        diff = int(s[0]) - int(e[0])
        if abs(diff) <= tolerance:
            ok += 1
            lat.append(diff * latency_multiplier)
    return (ok / total if total else 0.0), (sum(lat) / len(lat) if lat else 0.0)


class TurnTakingMetrics:
    """Accumulates turn-taking statistics per dataset name over validation batches."""

    def __init__(self, eos_token_id: int, bos_token_id: int, tolerance: int = 13, latency_multiplier: float = 0.08):
        self.eos, self.bos, self.tol, self.mult = eos_token_id, bos_token_id, tolerance, latency_multiplier
        self.reset()

    def reset(self):
        self._acc: Dict[str, List[float]] = {}
        self._lat: Dict[str, List[float]] = {}

    def update(self, name: str, source_tokens: torch.Tensor, pred_tokens: torch.Tensor) -> None:
        a, l = compute_turn_taking_metrics(source_tokens, pred_tokens, self.eos, self.bos, self.tol, self.mult)
        self._acc.setdefault(name, []).append(a)
        self._lat.setdefault(name, []).append(l)

    def compute(self) -> Dict[str, torch.Tensor]:
        out = {}
        for name in self._acc:
            out[f"turn_taking_acc_{name}"] = torch.tensor(sum(self._acc[name]) / len(self._acc[name]))
            out[f"turn_taking_latency_{name}"] = torch.tensor(sum(self._lat[name]) / len(self._lat[name]))
        self.reset()
        return out


# ------------------------------------------------------------------------------------------------ multiple choice
_LETTER = r"([a-d])"
_PATTERNS = [re.compile(p) for p in (
    r"(?:answer|choice|option)\s*(?:to [^.:]*?)?\s*(?:is|would be|should be|:)\s*[:\-]?\s*(?:option\s*)?[\(\[\"'\*\s]*" + _LETTER + r"\b",
    r"答案(?:是|应该是|为)\s*(?:选项)?\s*[\(\[\"'\*]*" + _LETTER,
    r"(?:would|will|i'd|i)\s+(?:select|choose|pick|go with)\s+(?:option\s*)?[\(\[\"'\*]*" + _LETTER + r"\b",
    r"[\(\[\"'\*]+" + _LETTER + r"[\)\]\"'\*]+\s+(?:is|would be)\s+(?:the\s+)?(?:best|correct|right)",
    r"\b" + _LETTER + r"\s+is\s+the\s+(?:best|correct|right)\s+(?:answer|choice|option)",
    r"(?:^|[:\n]\s*)\**[\(\[]?" + _LETTER + r"[\)\]\.\:,]",
    r"\*\*\s*[\(\[]?" + _LETTER + r"[\)\]\.\:]?\s*",
    r"\(" + _LETTER + r"\)",
)]


def extract_answer(response: Optional[str]) -> Optional[str]:
    """The option letter (A-D) a free-form answer settles on, or ``None``.  Tried in order: "the answer is X" phrasings (English
    and Chinese), "I would choose X", "(X) is the best answer", a leading ``X.`` / ``X)`` / ``X:``, a bold ``**X**``, a lone
    ``(X)``; a response that is just the letter counts too.  A leading ``<1>`` / ``<2>`` / ``<3>`` tag is ignored."""
    if not response or not response.strip():
        return None
    r = response.strip().lower()
    r = re.sub(r"^<[123]>\s*", "", r)
    if r in ("a", "b", "c", "d"):
        return r.upper()
    for pat in _PATTERNS:
        m = pat.search(r)
        if m:
            return m.group(1).upper()
    return None


class MCQEvaluator:
    """Accuracy of multiple-choice answers.  ``manifest_dir/<dataset>.jsonl`` lists ``{"id", "answer"}`` (or ``"label"``) per
    question; predictions are ``{"id", "pred_text"}``."""

    def __init__(self, manifest_dir: str):
        self.manifest_dir = manifest_dir
        self._keys: Dict[str, Dict[str, str]] = {}

    def load_dataset_manifest(self, dataset_name: str) -> Dict[str, str]:
        if dataset_name not in self._keys:
            path = os.path.join(self.manifest_dir, f"{dataset_name}.jsonl")
            gold = {}
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        it = json.loads(line)
                        ans = it.get("answer", it.get("label"))
                        if ans is not None:
                            gold[str(it["id"])] = str(ans).strip().upper()[:1]
            self._keys[dataset_name] = gold
        return self._keys[dataset_name]

    def evaluate(self, dataset_name: str, predictions: Sequence[Dict[str, Any]]) -> Dict[str, float]:
        gold = self.load_dataset_manifest(dataset_name)
        correct = answered = total = 0
        for p in predictions:
            g = gold.get(str(p.get("id")))
            if g is None:
                continue
            total += 1
            a = extract_answer(p.get("pred_text", ""))
            answered += a is not None
            correct += a == g
        return {"mcq_acc": correct / total if total else 0.0, "mcq_answered": answered / total if total else 0.0, "mcq_total": float(total)}


# ------------------------------------------------------------------------------------------------ empty responses
class EmptyTextMetric:
    """Share of hypotheses that are empty after stripping (a duplex model that never speaks scores 1.0)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self._n: Dict[str, int] = {}
        self._empty: Dict[str, int] = {}

    def update(self, name: str, hyps: Iterable[str]) -> None:
        for h in hyps:
            self._n[name] = self._n.get(name, 0) + 1
            self._empty[name] = self._empty.get(name, 0) + (not (h or "").strip())

    def compute(self) -> Dict[str, torch.Tensor]:
        out = {f"empty_text_rate_{k}": torch.tensor(self._empty[k] / max(1, n)) for k, n in self._n.items()}
        self.reset()
        return out


# ------------------------------------------------------------------------------------------------ results logger
class ResultsLogger:
    """Writes predictions of every rank to ``<save_path>/<dataset>_rank<r>.jsonl`` while validation runs; ``compute_and_save``
    (called by every rank) merges them on rank 0 into ``<dataset>.jsonl`` sorted by id, removes duplicates that distributed
    samplers pad in, and returns per-dataset metrics: WER and BLEU of ``pred_text`` against ``target_text``, the empty-response
    rate, and MCQ accuracy when an evaluator and a manifest for the dataset exist."""

    def __init__(self, save_path: str, rank: Optional[int] = None, world_size: Optional[int] = None, mcq_evaluator: Optional[MCQEvaluator] = None):
        import torch.distributed as dist

        self.dir = save_path
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
        self.world = world_size if world_size is not None else (dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1)
        self.mcq = mcq_evaluator
        os.makedirs(save_path, exist_ok=True)
        self._open: Dict[str, Any] = {}

    def _file(self, dataset: str):
        if dataset not in self._open:
            self._open[dataset] = open(os.path.join(self.dir, f"{dataset}_rank{self.rank}.jsonl"), "w", encoding="utf-8")
        return self._open[dataset]

    def reset(self):
        for f in self._open.values():
            f.close()
        self._open = {}

    def update(self, dataset: str, ids: Sequence[str], pred_text: Sequence[str], target_text: Optional[Sequence[str]] = None,
               extra: Optional[Sequence[Dict[str, Any]]] = None) -> None:
        f = self._file(dataset)
        for i, sid in enumerate(ids):
            rec = {"id": str(sid), "pred_text": pred_text[i]}
            if target_text is not None:
                rec["target_text"] = target_text[i]
            if extra is not None:
                rec.update(extra[i])
            f.write(json.dumps(rec, ensure_ascii=False) + "\n")
        f.flush()

    def _merge(self, dataset: str) -> List[Dict[str, Any]]:
        seen, out = set(), []
        for r in range(self.world):
            path = os.path.join(self.dir, f"{dataset}_rank{r}.jsonl")
            if not os.path.exists(path):
                continue
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        rec = json.loads(line)
                        if rec["id"] not in seen:
                            seen.add(rec["id"])
                            out.append(rec)
        out.sort(key=lambda r: r["id"])
        return out

    def compute_and_save(self, datasets: Optional[Sequence[str]] = None) -> Dict[str, float]:
        import torch.distributed as dist

        from ..utils.metrics import word_error_rate
        from .parts import bleu

        names = list(datasets) if datasets is not None else sorted(self._open)
        self.reset()
        if self.world > 1 and dist.is_available() and dist.is_initialized():
            dist.barrier()                      # every rank's file is complete
        metrics: Dict[str, float] = {}
        if self.rank == 0:
            for d in names:
                recs = self._merge(d)
                with open(os.path.join(self.dir, f"{d}.jsonl"), "w", encoding="utf-8") as f:
                    for r in recs:
                        f.write(json.dumps(r, ensure_ascii=False) + "\n")
                hyp = [r["pred_text"] for r in recs]
                metrics[f"{d}/num_samples"] = float(len(recs))
                metrics[f"{d}/empty_text_rate"] = sum(not (h or "").strip() for h in hyp) / max(1, len(hyp))
                if recs and all("target_text" in r for r in recs):
                    ref = [r["target_text"] for r in recs]
                    metrics[f"{d}/wer"] = float(word_error_rate(hyp, ref))
                    metrics[f"{d}/bleu"] = float(bleu(hyp, ref))
                if self.mcq is not None and os.path.exists(os.path.join(self.mcq.manifest_dir, f"{d}.jsonl")):
                    metrics.update({f"{d}/{k}": v for k, v in self.mcq.evaluate(d, recs).items()})
            with open(os.path.join(self.dir, "metrics.json"), "w") as f:
                json.dump(metrics, f, indent=1, sort_keys=True)
        if self.world > 1 and dist.is_available() and dist.is_initialized():
            box = [metrics]
            dist.broadcast_object_list(box, src=0)
            metrics = box[0]
        return metrics

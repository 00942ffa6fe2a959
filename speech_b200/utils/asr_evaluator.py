"""ASR evaluation driver and a static data-explorer report.

``ASREvaluator`` is the transcribe-then-score loop: it reads a manifest, transcribes the audio with a model (offline
``transcribe``, or any callable for buffered / streaming engines), writes a prediction manifest (``pred_text`` next to
``text``) and scores it — corpus WER / CER with insertion, deletion and substitution rates, per-utterance error rates, and
breakdowns over metadata fields (e.g. by duration bucket, gender, or any manifest key) (reference: ``tools/asr_evaluator``:
``asr_evaluator.py`` + ``utils.py`` ``cal_write_wer`` / ``target_metadata_wer``).

``write_explorer_report`` renders what the reference's web UI (``tools/speech_data_explorer``) shows on its statistics and
samples pages into ONE self-contained HTML file: corpus totals (hours, utterances, vocabulary, alphabet), duration and
characters-per-second histograms, the most frequent words and the most frequent word errors, and a sortable-by-WER table of
utterances with their reference / hypothesis word-level diffs.  No server and no plotting package is needed to look at it.
"""
from __future__ import annotations

import html
import json
import os
from collections import Counter
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from .metrics import word_error_rate, word_error_rate_detail


def _read(path: str) -> List[Dict[str, Any]]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(l) for l in f if l.strip()]


def _write(path: str, items: Sequence[Dict[str, Any]]) -> None:
    with open(path, "w", encoding="utf-8") as f:
        for it in items:
            f.write(json.dumps(it, ensure_ascii=False) + "\n")


def align_words(ref: Sequence[str], hyp: Sequence[str]) -> List[Tuple[str, Optional[str], Optional[str]]]:
    """Levenshtein alignment: list of (op, ref_word, hyp_word) with op in {"ok", "sub", "del", "ins"}."""
    R, H = len(ref), len(hyp)
    d = [[0] * (H + 1) for _ in range(R + 1)]
    for i in range(R + 1):
        d[i][0] = i
    for j in range(H + 1):
        d[0][j] = j
    for i in range(1, R + 1):
        for j in range(1, H + 1):
            d[i][j] = min(d[i - 1][j - 1] + (ref[i - 1] != hyp[j - 1]), d[i - 1][j] + 1, d[i][j - 1] + 1)
    out, i, j = [], R, H
    while i > 0 or j > 0:
        if i > 0 and j > 0 and d[i][j] == d[i - 1][j - 1] + (ref[i - 1] != hyp[j - 1]):
            out.append(("ok" if ref[i - 1] == hyp[j - 1] else "sub", ref[i - 1], hyp[j - 1]))
            i, j = i - 1, j - 1
        elif i > 0 and d[i][j] == d[i - 1][j] + 1:
            out.append(("del", ref[i - 1], None))
            i -= 1
        else:
            out.append(("ins", None, hyp[j - 1]))
            j -= 1
    return out[::-1]


class ASREvaluator:
    def __init__(self, model=None, transcribe_fn: Optional[Callable[[List[str]], List[Any]]] = None, batch_size: int = 16,
                 text_processing: Optional[Callable[[str], str]] = None, use_cer: bool = False):
        if model is None and transcribe_fn is None:
            raise ValueError("give a model with .transcribe() or a transcribe_fn")
        self.fn = transcribe_fn or (lambda paths: model.transcribe(paths, batch_size=batch_size))
        self.norm = text_processing or (lambda s: " ".join(s.lower().split()))
        self.use_cer = use_cer

    def transcribe_manifest(self, manifest: str, out_manifest: str) -> List[Dict[str, Any]]:
        items = _read(manifest)
        hyps = self.fn([it["audio_filepath"] for it in items])
        for it, h in zip(items, hyps):
            it["pred_text"] = h.text if hasattr(h, "text") else str(h)
        _write(out_manifest, items)
        return items

    def score(self, items: Sequence[Dict[str, Any]], metadata_keys: Sequence[str] = (), duration_buckets: Sequence[float] = ()) -> Dict[str, Any]:
        ref = [self.norm(it.get("text", "")) for it in items]
        hyp = [self.norm(it.get("pred_text", "")) for it in items]
        wer, words, ins, dele, sub = word_error_rate_detail(hyp, ref, use_cer=self.use_cer)
        res: Dict[str, Any] = {"wer": wer, "cer": word_error_rate(hyp, ref, use_cer=True), "tokens": words, "ins_rate": ins, "del_rate": dele,
                               "sub_rate": sub, "utterances": len(items)}
        per = [word_error_rate([h], [r], use_cer=self.use_cer) if r else float(bool(h)) for h, r in zip(hyp, ref)]
        for it, w in zip(items, per):
            it["wer"] = w
        groups: Dict[str, Dict[str, List[int]]] = {}
        for k in metadata_keys:
            for i, it in enumerate(items):
                groups.setdefault(k, {}).setdefault(str(it.get(k, "unknown")), []).append(i)
        if duration_buckets:
            edges = list(duration_buckets)
            for i, it in enumerate(items):
                d = float(it.get("duration", 0.0))
                b = sum(d >= e for e in edges)
                name = f"<{edges[0]:g}s" if b == 0 else (f">={edges[-1]:g}s" if b == len(edges) else f"{edges[b - 1]:g}-{edges[b]:g}s")
                groups.setdefault("duration", {}).setdefault(name, []).append(i)
        res["breakdown"] = {k: {v: {"wer": word_error_rate([hyp[i] for i in idx], [ref[i] for i in idx], use_cer=self.use_cer), "utterances": len(idx)}
                                for v, idx in vals.items()} for k, vals in groups.items()}
        return res

    def run(self, manifest: str, out_dir: str, **score_kw) -> Dict[str, Any]:
        os.makedirs(out_dir, exist_ok=True)
        items = self.transcribe_manifest(manifest, os.path.join(out_dir, "predictions.json"))
        res = self.score(items, **score_kw)
        _write(os.path.join(out_dir, "predictions.json"), items)
        with open(os.path.join(out_dir, "scores.json"), "w") as f:
            json.dump(res, f, indent=1)
        return res


def _hist(values: Sequence[float], bins: int = 20) -> List[Tuple[float, float, int]]:
    if not values:
        return []
    lo, hi = min(values), max(values)
    w = (hi - lo) / bins or 1.0
    counts = [0] * bins
    for v in values:
        counts[min(bins - 1, int((v - lo) / w))] += 1
    return [(lo + i * w, lo + (i + 1) * w, c) for i, c in enumerate(counts)]


def _svg_bars(hist, width=560, height=140, unit="") -> str:
    if not hist:
        return ""
    top = max(c for _, _, c in hist) or 1
    bw = width / len(hist)
    bars = "".join(f'<rect x="{i * bw + 1:.1f}" y="{height - 20 - (height - 30) * c / top:.1f}" width="{bw - 2:.1f}" '
                   f'height="{(height - 30) * c / top:.1f}" fill="#4a7"><title>{a:.2f}-{b:.2f}{unit}: {c}</title></rect>'
                   for i, (a, b, c) in enumerate(hist))
    return (f'<svg width="{width}" height="{height}">{bars}<text x="0" y="{height - 4}" font-size="11">{hist[0][0]:.2f}{unit}</text>'
            f'<text x="{width - 60}" y="{height - 4}" font-size="11">{hist[-1][1]:.2f}{unit}</text></svg>')


def write_explorer_report(manifest_or_items, out_html: str, max_rows: int = 500) -> Dict[str, Any]:
    items = _read(manifest_or_items) if isinstance(manifest_or_items, str) else list(manifest_or_items)
    durs = [float(it.get("duration", 0.0)) for it in items]
    texts = [str(it.get("text", "")) for it in items]
    words = Counter(w for t in texts for w in t.split())
    alphabet = sorted(set("".join(texts)))
    cps = [len(t) / d for t, d in zip(texts, durs) if d > 0]
    has_pred = any("pred_text" in it for it in items)
    stats: Dict[str, Any] = {"utterances": len(items), "hours": sum(durs) / 3600.0, "vocabulary": len(words), "alphabet": len(alphabet)}
    errs: Counter = Counter()
    rows = []
    if has_pred:
        hyp = [str(it.get("pred_text", "")) for it in items]
        stats["wer"] = word_error_rate(hyp, texts)
        stats["cer"] = word_error_rate(hyp, texts, use_cer=True)
    for it, t in zip(items, texts):
        w = None
        diff = html.escape(t)
        if has_pred:
            al = align_words(t.split(), str(it.get("pred_text", "")).split())
            nerr = sum(op != "ok" for op, _, _ in al)
            w = nerr / max(1, len(t.split()))
            for op, r, h in al:
                if op != "ok":
                    errs[(op, r or "", h or "")] += 1
            colour = {"ok": "", "sub": "background:#fd8", "del": "background:#f99;text-decoration:line-through", "ins": "background:#9cf"}
            diff = " ".join(f'<span style="{colour[op]}">{html.escape(r if op == "del" else (h if op == "ins" else (r if op == "ok" else f"{r}→{h}")))}</span>'
                            for op, r, h in al)
        rows.append((w if w is not None else 0.0, it.get("audio_filepath", ""), float(it.get("duration", 0.0)), diff))
    rows.sort(key=lambda r: -r[0])
    top_words = "".join(f"<tr><td>{html.escape(w)}</td><td>{c}</td></tr>" for w, c in words.most_common(30))
    top_errs = "".join(f"<tr><td>{op}</td><td>{html.escape(r)}</td><td>{html.escape(h)}</td><td>{c}</td></tr>" for (op, r, h), c in errs.most_common(30))
    table = "".join(f"<tr><td>{w:.2%}</td><td>{html.escape(os.path.basename(str(p)))}</td><td>{d:.2f}</td><td>{diff}</td></tr>" for w, p, d, diff in rows[:max_rows])
    doc = f"""<!doctype html><html><head><meta charset="utf-8"><title>Speech data report</title>
<style>body{{font-family:sans-serif;margin:1.5em}}table{{border-collapse:collapse}}td,th{{border:1px solid #ccc;padding:2px 6px;font-size:13px}}</style></head><body>
<h1>Speech data report</h1><p>{' | '.join(f'<b>{k}</b>: {v:.4g}' if isinstance(v, float) else f'<b>{k}</b>: {v}' for k, v in stats.items())}</p>
<h2>Duration (s)</h2>{_svg_bars(_hist(durs), unit='s')}<h2>Characters per second</h2>{_svg_bars(_hist(cps))}
<h2>Alphabet</h2><p>{html.escape(' '.join(alphabet))}</p>
<h2>Most frequent words</h2><table><tr><th>word</th><th>count</th></tr>{top_words}</table>
{'<h2>Most frequent word errors</h2><table><tr><th>type</th><th>reference</th><th>hypothesis</th><th>count</th></tr>' + top_errs + '</table>' if has_pred else ''}
<h2>Utterances{' (highest WER first)' if has_pred else ''}</h2><table><tr><th>WER</th><th>file</th><th>duration</th><th>text</th></tr>{table}</table></body></html>"""
    with open(out_html, "w", encoding="utf-8") as f:
        f.write(doc)
    stats["top_errors"] = [(op, r, h, c) for (op, r, h), c in errs.most_common(10)]
    return stats

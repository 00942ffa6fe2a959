"""Text post-processing for streaming transcripts: inverse text normalisation (spoken → written form) and a translation hook.

Reference: ``asr/inference/itn`` (batched ITN of finished segments through ``nemo_text_processing`` — an optional WFST package) and
``asr/inference/nmt`` (optional machine translation of finished segments through a vLLM-served model).  Here ITN is a small
rule set for English cardinals, ordinals, decimals, percentages, currency amounts and o'clock times (good enough for captions; a
caller can plug any callable with the same signature), and translation is a hook around any ``translate(list[str]) -> list[str]``.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, List, Optional, Sequence

_UNITS = {w: i for i, w in enumerate("zero one two three four five six seven eight nine ten eleven twelve thirteen fourteen fifteen sixteen "
                                     "seventeen eighteen nineteen".split())}
_TENS = {w: 10 * (i + 2) for i, w in enumerate("twenty thirty forty fifty sixty seventy eighty ninety".split())}
_SCALES = {"hundred": 100, "thousand": 1000, "million": 10 ** 6, "billion": 10 ** 9}
_ORD = {"first": 1, "second": 2, "third": 3, "fifth": 5, "eighth": 8, "ninth": 9, "twelfth": 12}
_ORD_TENS = {w[:-1] + "ieth": v for w, v in _TENS.items()}


def _is_num(w: str) -> bool:
    return w in _UNITS or w in _TENS or w in _SCALES or "-" in w and all(_is_num(p) for p in w.split("-"))


def _value(words: Sequence[str]) -> int:
    total = cur = 0
    for w in words:
        for p in w.split("-"):
            if p in _UNITS:
                cur += _UNITS[p]
            elif p in _TENS:
                cur += _TENS[p]
            elif p == "hundred":
                cur = max(cur, 1) * 100
            else:
                total += max(cur, 1) * _SCALES[p]
                cur = 0
    return total + cur


def _ordinal(w: str) -> Optional[int]:
    if w in _ORD:
        return _ORD[w]
    if w in _ORD_TENS:
        return _ORD_TENS[w]
    if w.endswith("th") and _is_num(w[:-2]):
        return _value([w[:-2]])
    if "-" in w:
        head, tail = w.rsplit("-", 1)
        t = _ordinal(tail)
        if t is not None and _is_num(head):
            return _value([head]) + t
    return None


def _suffix(n: int) -> str:
    return "th" if 10 <= n % 100 <= 20 else {1: "st", 2: "nd", 3: "rd"}.get(n % 10, "th")


class InverseTextNormalizer:
    def __init__(self, lang: str = "en", extra_rules: Optional[Dict[str, str]] = None):
        if lang != "en":
            raise ValueError("the built-in rule set covers English; pass a callable for other languages")
        self.extra = dict(extra_rules or {})

    def normalize(self, text: str) -> str:
        words = text.split()
        out: List[str] = []
        i = 0
        while i < len(words):
            w = words[i].lower()
            if w in self.extra:
                out.append(self.extra[w])
                i += 1
                continue
            nxt_w = words[i + 1].lower() if i + 1 < len(words) else ""
            lone_one = w == "one" and not (_is_num(nxt_w) or nxt_w in ("point", "percent", "dollar", "dollars", "euro", "euros", "o'clock"))
            if _is_num(w) and not lone_one:
                j = i
                while j < len(words) and (_is_num(words[j].lower()) or (words[j].lower() == "and" and j + 1 < len(words) and
                                                                        _is_num(words[j + 1].lower()) and j > i)):
                    j += 1
                nums = [x.lower() for x in words[i:j] if x.lower() != "and"]
                val = str(_value(nums))
                if j < len(words) and words[j].lower() == "point":
                    k, digits = j + 1, ""
                    while k < len(words) and words[k].lower() in _UNITS and _UNITS[words[k].lower()] < 10:
                        digits += str(_UNITS[words[k].lower()])
                        k += 1
                    if digits:
                        val, j = val + "." + digits, k
                nxt = words[j].lower() if j < len(words) else ""
                if j < len(words) and _ordinal(nxt) is not None and nxt not in _UNITS and _value(nums) % 10 == 0 and _ordinal(nxt) < 10 and _value(nums) >= 20:
                    n = _value(nums) + _ordinal(nxt)
                    out.append(f"{n}{_suffix(n)}")
                    j += 1
                elif nxt in ("percent", "per cent"):
                    out.append(val + "%")
                    j += 1
                elif nxt in ("dollars", "dollar"):
                    out.append("$" + val)
                    j += 1
                elif nxt in ("euros", "euro"):
                    out.append("€" + val)
                    j += 1
                elif nxt == "o'clock":
                    out.append(val + ":00")
                    j += 1
                else:
                    out.append(val)
                i = j
                continue
            o = _ordinal(w)
            if o is not None:
                out.append(f"{o}{_suffix(o)}")
            else:
                out.append(words[i])
            i += 1
        return " ".join(out)

    __call__ = normalize

    def normalize_list(self, texts: Sequence[str]) -> List[str]:
        return [self.normalize(t) for t in texts]


class TranslationHook:
    """Wraps a batch translator (e.g. a served LLM); finished segments are translated in batches of ``batch_size``."""

    def __init__(self, translate: Callable[[List[str]], List[str]], source_lang: str = "en", target_lang: str = "de", batch_size: int = 16):
        self.translate, self.source_lang, self.target_lang, self.batch_size = translate, source_lang, target_lang, batch_size

    def __call__(self, texts: Sequence[str]) -> List[str]:
        out: List[str] = []
        texts = list(texts)
        for s in range(0, len(texts), self.batch_size):
            chunk = texts[s:s + self.batch_size]
            res = self.translate(chunk)
            if len(res) != len(chunk):
                raise RuntimeError(f"translator returned {len(res)} outputs for {len(chunk)} inputs")
            out += list(res)
        return out

"""Text post-processing for streaming transcripts: inverse text normalisation (spoken → written form) and a translation hook.

Reference: ``asr/inference/itn`` (batched ITN of finished segments through ``nemo_text_processing`` — an optional WFST package) and
``asr/inference/nmt`` (optional machine translation of finished segments through a vLLM-served model).  Here ITN is a small
rule set for English cardinals, ordinals, decimals, percentages, currency amounts and o'clock times (good enough for captions; a
caller can plug any callable with the same signature), and translation is a hook around any ``translate(list[str]) -> list[str]``.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

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


# ---------------------------------------------------------------------------------------------- alignment-preserving ITN
class AlignmentPreservingInverseNormalizer:
    """Inverse text normalisation that also says which input words each output word came from, so that word timestamps and
    confidences survive the rewrite ("twenty five dollars" at 1.2-2.0 s becomes "$25" at 1.2-2.0 s).

    ``get_word_alignment(words)`` returns ``(input words, output words, spans)`` where ``spans[k] = (i0, i1, o0, o1)`` maps input
    words ``[i0, i1)`` onto output words ``[o0, o1)``; every input and every output word belongs to exactly one span.  The rules
    are those of ``InverseTextNormalizer`` (or any ``normalize(str) -> str`` passed in); spans are found by normalising growing
    windows, which works for any normaliser whose rewrites are local.
    Reference: ``inference/itn/inverse_normalizer.py`` ``AlignmentPreservingInverseNormalizer``.
    """

    def __init__(self, normalizer: Optional[Callable[[str], str]] = None, max_span: int = 12, cache_size: int = 4096):
        self.normalize = normalizer or InverseTextNormalizer()
        self.max_span = max_span
        self._cache: Dict[str, str] = {}
        self._cache_size = cache_size

    def _norm(self, text: str) -> str:
        got = self._cache.get(text)
        if got is None:
            got = self.normalize(text)
            if len(self._cache) < self._cache_size:
                self._cache[text] = got
        return got

    def get_word_alignment(self, words: Sequence[str]) -> Tuple[List[str], List[str], List[Tuple[int, int, int, int]]]:
        words = list(words)
        whole = self._norm(" ".join(words)).split()
        spans: List[Tuple[int, int, int, int]] = []
        i = o = 0
        while i < len(words):
            # the shortest window [i, j) whose own normalisation is what the whole sentence shows at this place, and after which
            # the rest normalises to the rest: that is a unit the rules rewrote together
            done = False
            for j in range(i + 1, min(len(words), i + self.max_span) + 1):
                head = self._norm(" ".join(words[i:j])).split()
                if whole[o:o + len(head)] != head:
                    continue
                tail = self._norm(" ".join(words[j:])).split() if j < len(words) else []
                if whole[o + len(head):] == tail:
                    spans.append((i, j, o, o + len(head)))
                    i, o = j, o + len(head)
                    done = True
                    break
            if not done:                                        # a rewrite longer than max_span: close everything in one span
                spans.append((i, len(words), o, len(whole)))
                i, o = len(words), len(whole)
        if o < len(whole) and spans:
            i0, i1, o0, _ = spans[-1]
            spans[-1] = (i0, i1, o0, len(whole))
        return words, whole, spans

    def apply_to_words(self, words: Sequence["Word"]) -> List["Word"]:
        """``Word`` records (text, start, end, conf) in, rewritten records out; a span's time range is shared by its outputs."""
        from .state import Word

        texts = [w.text for w in words]
        _, out, spans = self.get_word_alignment(texts)
        res: List[Word] = []
        for i0, i1, o0, o1 in spans:
            src = list(words[i0:i1])
            if not src or o1 == o0:
                continue
            start, end = src[0].start, src[-1].end
            conf = min(w.conf for w in src)
            n = o1 - o0
            for k in range(n):                                   # several outputs from one span split its time evenly
                a = start + (end - start) * k / n
                b = start + (end - start) * (k + 1) / n
                res.append(Word(text=out[o0 + k], start=a, end=b, conf=conf))
        return res


def merge_punctuation_and_itn(words_pnc: Sequence[str], words_itn: Sequence[str], spans: Sequence[Tuple[int, int, int, int]],
                              punctuation: str = ".,?!;:") -> List[str]:
    """Combines a punctuated / capitalised transcript with its inverse-normalised form: rewritten spans take the ITN text, keep the
    trailing punctuation of the last word they replace and the capitalisation of the first; untouched words stay as punctuated.
    Reference: ``inference/itn/batch_inverse_normalizer.py`` ``merge_punctuation_and_itn_tags``."""
    out: List[str] = []
    for i0, i1, o0, o1 in spans:
        src = list(words_pnc[i0:i1])
        new = list(words_itn[o0:o1])
        if not new:
            continue
        plain = [w.strip(punctuation).lower() for w in src]
        if [w.lower() for w in new] == plain:
            out += src
            continue
        tail = ""
        last = src[-1] if src else ""
        while last and last[-1] in punctuation:
            tail, last = last[-1] + tail, last[:-1]
        if src and src[0][:1].isupper() and new[0][:1].isalpha():
            new[0] = new[0][:1].upper() + new[0][1:]
        new[-1] = new[-1] + tail
        out += new
    return out


class BatchAlignmentPreservingInverseNormalizer:
    """Applies the aligner to many segments at once (a thread pool: the rules are pure Python and release nothing, but segments are
    independent and a served normaliser may block on IO) and merges with punctuation when a punctuated variant is given."""

    def __init__(self, itn: Optional[AlignmentPreservingInverseNormalizer] = None, n_jobs: int = 1):
        self.itn = itn or AlignmentPreservingInverseNormalizer()
        self.n_jobs = n_jobs

    def _one(self, args):
        words, words_pnc = args
        texts = [w.text for w in words]
        _, out, spans = self.itn.get_word_alignment([t.strip(".,?!;:").lower() for t in texts] if words_pnc is None else texts)
        new_words = self.itn.apply_to_words(words)
        if words_pnc is not None:
            merged = merge_punctuation_and_itn(words_pnc, out, spans)
            if len(merged) == len(new_words):
                for w, t in zip(new_words, merged):
                    w.text = t
        return new_words

    def __call__(self, batch_words: Sequence[Sequence["Word"]], batch_words_pnc: Optional[Sequence[Optional[Sequence[str]]]] = None):
        pnc = list(batch_words_pnc) if batch_words_pnc is not None else [None] * len(batch_words)
        items = list(zip(batch_words, pnc))
        if self.n_jobs > 1 and len(items) > 1:
            from concurrent.futures import ThreadPoolExecutor

            with ThreadPoolExecutor(self.n_jobs) as ex:
                return list(ex.map(self._one, items))
        return [self._one(it) for it in items]


# ---------------------------------------------------------------------------------------------- streaming LLM translation
_LANG_NAMES = {"en": "English", "de": "German", "es": "Spanish", "fr": "French", "it": "Italian", "pt": "Portuguese", "nl": "Dutch", "pl": "Polish",
               "ru": "Russian", "uk": "Ukrainian", "zh": "Chinese", "ja": "Japanese", "ko": "Korean", "hi": "Hindi", "ar": "Arabic", "tr": "Turkish"}


class TranslationPrompt:
    """Chat-style prompt of an instruction-tuned LLM asked to translate; the target side ends open so that the model continues a
    given ``tgt_prefix``.  ``extract`` cuts the answer at the first line break or end-of-turn marker."""

    end_markers = ("<|im_end|>", "</s>", "<|eot_id|>", "\n")

    @classmethod
    def format(cls, src_lang: str, tgt_lang: str, src_text: str, tgt_prefix: str = "", src_context: str = "", tgt_context: str = "") -> str:
        s, t = _LANG_NAMES.get(src_lang, src_lang), _LANG_NAMES.get(tgt_lang, tgt_lang)
        ctx = f"Earlier {s} text: {src_context}\nIts {t} translation: {tgt_context}\n" if src_context else ""
        return (f"<|im_start|>system\n<|im_end|>\n<|im_start|>user\n{ctx}Translate the following {s} source text to {t}:\n{s}: {src_text}\n"
                f"{t}: <|im_end|>\n<|im_start|>assistant\n{tgt_prefix}")

    @classmethod
    def extract(cls, response: str) -> str:
        cut = len(response)
        for m in cls.end_markers:
            k = response.find(m)
            if k >= 0:
                cut = min(cut, k)
        return response[:cut]


class LLMTranslator:
    """Simultaneous translation of a growing transcript with an LLM.  Every step re-translates the current transcript but forces
    the model to continue a *prefix* — the part of the translation that has stopped changing — so what was shown stays shown.

    ``generate(prompts: list[str]) -> list[str]`` is the engine (a served model, or ``NativeLMGenerator`` below).
    ``get_prefixes`` implements the stability rule: the new prefix is the longest common prefix of this step's and the previous
    step's translation cut back to a word boundary; when it lags the transcript by more than ``waitk`` words it is forced forward
    from the current translation; an empty transcript empties it.
    Reference: ``inference/nmt/llm_translator.py`` ``LLMTranslator``.
    """

    def __init__(self, generate: Callable[[List[str]], List[str]], prompt=TranslationPrompt, waitk: int = -1, batch_size: int = -1):
        self.generate, self.prompt, self.waitk, self.batch_size = generate, prompt, waitk, batch_size

    def translate_batch(self, asr_transcripts, prefixes, src_langs, tgt_langs, src_contexts=None, tgt_contexts=None) -> List[str]:
        n = len(asr_transcripts)
        src_contexts = src_contexts or [""] * n
        tgt_contexts = tgt_contexts or [""] * n
        prompts = [self.prompt.format(sl, tl, a, p, sc, tc) for a, p, sl, tl, sc, tc in
                   zip(asr_transcripts, prefixes, src_langs, tgt_langs, src_contexts, tgt_contexts)]
        outs = self.generate(prompts)
        if len(outs) != n:
            raise RuntimeError(f"the engine returned {len(outs)} outputs for {n} prompts")
        return [f"{p}{self.prompt.extract(o)}" for p, o in zip(prefixes, outs)]

    def translate(self, asr_transcripts, prefixes, src_langs, tgt_langs, src_contexts=None, tgt_contexts=None) -> List[str]:
        n = len(asr_transcripts)
        bs = self.batch_size if self.batch_size and self.batch_size > 0 else max(n, 1)
        out: List[str] = []
        for i in range(0, n, bs):
            sl = slice(i, i + bs)
            out += self.translate_batch(asr_transcripts[sl], prefixes[sl], src_langs[sl], tgt_langs[sl],
                                        None if src_contexts is None else src_contexts[sl], None if tgt_contexts is None else tgt_contexts[sl])
        return out

    def get_prefixes(self, asr_transcripts: Sequence[str], translations: Sequence[str], prev_translations: Sequence[str]) -> List[str]:
        import string

        res = []
        for asr, cur, prev in zip(asr_transcripts, translations, prev_translations):
            k = 0
            while k < min(len(cur), len(prev)) and cur[k] == prev[k]:
                k += 1
            lcp = cur[:k]
            lead = lcp.startswith(" ")
            if lcp and lcp[-1] not in string.punctuation + " " and k < max(len(cur), len(prev)):
                lcp = " ".join(lcp.split()[:-1])                 # the agreement ended inside a word
            lcp = lcp.strip()
            if not asr:
                lcp = ""
            n_src, n_pre = len(asr.split()), len(lcp.split())
            new = " ".join(cur.split()[: n_src - self.waitk]) if self.waitk > 0 and n_src - n_pre > self.waitk else lcp
            if new and lead and not new.startswith(" "):
                new = " " + new
            res.append(new)
        return res


class NativeLMGenerator:
    """``generate`` for ``LLMTranslator`` on this package's own causal LM (``speechlm.llm``) and a tokenizer: greedy decoding with
    the KV cache, one prompt at a time (prompts of a translation step differ in length; the LM is small next to the ASR encoder)."""

    def __init__(self, llm, tokenizer, max_new_tokens: int = 64, eos_id: Optional[int] = None):
        self.llm, self.tok, self.max_new, self.eos = llm, tokenizer, max_new_tokens, eos_id

    @torch.no_grad()
    def __call__(self, prompts: List[str]) -> List[str]:
        outs = []
        dev = next(self.llm.parameters()).device
        eos = self.eos if self.eos is not None else getattr(self.tok, "eos_id", None)
        for p in prompts:
            ids = torch.tensor([self.tok.text_to_ids(p)], device=dev)
            gen = self.llm.generate(input_ids=ids, max_new_tokens=self.max_new, eos_token_id=eos)
            new = gen[0].tolist()                               # the LM returns only the new ids
            if eos is not None and eos in new:
                new = new[: new.index(eos)]
            outs.append(self.tok.ids_to_text(new))
        return outs

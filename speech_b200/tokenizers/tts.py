"""Text tokenizers of the TTS models: text -> ids over a fixed symbol inventory (characters or phonemes), with the bookkeeping
TTS needs — a pad symbol, an optional blank, an out-of-vocabulary symbol, punctuation handling, optional padding of the utterance
with spaces, text normalisation per locale — and an aggregate that gives several tokenizers disjoint id ranges.

* ``BaseCharsTokenizer`` and the locale classes (English, German, Spanish, French, Italian, Vietnamese, Hindi, Arabic)
* ``EnglishPhonemesTokenizer`` (ARPABET from a G2P callable, stress marks optional, graphemes for unknown words)
* ``IPATokenizer`` (any locale: IPA symbols from an ``IpaG2p``, graphemes prefixed so they never collide with phonemes)
* ``ChinesePhonemesTokenizer`` / ``JapanesePhonemeTokenizer`` (through the G2P classes of ``tts/g2p.py``)
* ``AggregatedTTSTokenizer``; ``get_grapheme_character_set`` / ``get_ipa_punctuation_list`` / text preprocessing helpers

Reference: ``common/tokenizers/text_to_speech/{tts_tokenizers,ipa_lexicon,tokenizer_utils}.py``.
"""
from __future__ import annotations

import re
import string
import unicodedata
from typing import Callable, Dict, List, Optional, Sequence

__all__ = ["AggregatedTTSTokenizer", "ArabicCharsTokenizer", "BaseCharsTokenizer", "BaseTokenizer", "ChinesePhonemesTokenizer", "EnglishCharsTokenizer",
           "EnglishPhonemesTokenizer", "FrenchCharsTokenizer", "GermanCharsTokenizer", "HindiCharsTokenizer", "IPATokenizer", "ItalianCharsTokenizer",
           "JapanesePhonemeTokenizer", "SpanishCharsTokenizer", "VietnameseCharsTokenizer", "any_locale_text_preprocessing", "english_text_preprocessing",
           "get_grapheme_character_set", "get_ipa_punctuation_list", "normalize_unicode_text"]

# ------------------------------------------------------------------------------------------------ lexicon
_GRAPHEMES = {
    "en-US": string.ascii_uppercase + "'",
    "en-GB": string.ascii_uppercase + "'",
    "es-ES": string.ascii_uppercase + "ÁÉÍÑÓÚÜ",
    "es-US": string.ascii_uppercase + "ÁÉÍÑÓÚÜ",
    "it-IT": string.ascii_uppercase + "ÀÈÉÌÒÙ",
    "fr-FR": string.ascii_uppercase + "ÀÂÄÆÇÈÉÊËÍÎÏÑÔÖÙÛÜŌŒ",
    "de-DE": string.ascii_uppercase + "ÄÖÜẞ",
    "pt-BR": string.ascii_uppercase + "ÁÂÃÀÇÉÊÍÓÔÕÚÜ",
    "nl-NL": string.ascii_uppercase + "ÁÄÉËÍÏÓÖÚÜ",
    "pl-PL": string.ascii_uppercase + "ĄĆĘŁŃÓŚŹŻ",
    "vi-VN": string.ascii_uppercase + "ÀÁẢÃẠĂẰẮẲẴẶÂẦẤẨẪẬĐÈÉẺẼẸÊỀẾỂỄỆÌÍỈĨỊÒÓỎÕỌÔỒỐỔỖỘƠỜỚỞỠỢÙÚỦŨỤƯỪỨỬỮỰỲÝỶỸỴ",
}
_PUNCT_COMMON = list(",.!?-:;/\"()[]{}")
_PUNCT_EXTRA = {"es-ES": ["¿", "¡"], "es-US": ["¿", "¡"], "fr-FR": ["«", "»", "–", "—", "‹", "›"], "de-DE": ["„", "“", "‚", "‘", "–", "—"],
                "it-IT": ["«", "»", "–", "—", "’"], "en-GB": ["‘", "’", "“", "”"]}


def validate_locale(locale: str) -> None:
    if locale not in _GRAPHEMES:
        raise ValueError(f"unsupported locale {locale!r}; supported: {sorted(_GRAPHEMES)}")


def get_grapheme_character_set(locale: str, case: str = "upper") -> str:
    validate_locale(locale)
    g = _GRAPHEMES[locale]
    if case == "upper":
        return g
    if case == "lower":
        return g.lower()
    if case == "mixed":
        return "".join(dict.fromkeys(g + g.lower()))
    raise ValueError(f"case must be upper, lower or mixed, got {case!r}")


def get_ipa_punctuation_list(locale: Optional[str]) -> List[str]:
    if locale is None:
        return sorted(_PUNCT_COMMON)
    validate_locale(locale)
    return sorted(set(_PUNCT_COMMON + _PUNCT_EXTRA.get(locale, [])))


# ------------------------------------------------------------------------------------------------ text preprocessing
_SYNONYMS = {"“": '"', "”": '"', "‘": "'", "’": "'", "`": "'", "´": "'", "–": "-", "—": "-", "…": "...", " ": " "}


def normalize_unicode_text(text: str) -> str:
    """Canonical composition (one code point per accented letter where it exists)."""
    return unicodedata.normalize("NFC", text)


def any_locale_text_preprocessing(text: str) -> str:
    text = normalize_unicode_text(text)
    for a, b in _SYNONYMS.items():
        text = text.replace(a, b)
    return re.sub(r"\s+", " ", text).strip()


def english_text_preprocessing(text: str, lower: bool = True) -> str:
    """Accents stripped to ASCII, typographic quotes and dashes replaced, optional lower case."""
    text = any_locale_text_preprocessing(text)
    text = "".join(c for c in unicodedata.normalize("NFD", text) if unicodedata.category(c) != "Mn")
    return text.lower() if lower else text


# ------------------------------------------------------------------------------------------------ base classes
class BaseTokenizer:
    PAD, BLANK, OOV = "<pad>", "<blank>", "<oov>"

    def __init__(self, tokens: Sequence[str], pad: str = PAD, blank: str = BLANK, oov: str = OOV, sep: str = "|", add_blank_at: Optional[str] = None):
        """``add_blank_at``: ``None`` (no blank symbol), ``"last"`` or ``"last_but_one"`` (before the OOV symbol)."""
        tokens = list(dict.fromkeys(tokens))
        self.pad, tokens = len(tokens), tokens + [pad]
        if add_blank_at is not None:
            self.blank, tokens = len(tokens), tokens + [blank]
        else:
            self.blank = None
        self.oov, tokens = len(tokens), tokens + [oov]
        if add_blank_at == "last":
            tokens[-1], tokens[-2] = tokens[-2], tokens[-1]
            self.oov, self.blank = self.blank, self.oov
        self.tokens, self.sep = tokens, sep
        self._token2id = {t: i for i, t in enumerate(tokens)}
        self._util_ids = {self.pad, self.blank, self.oov} - {None}
        self.pad_id = self.pad

    @property
    def vocab_size(self) -> int:
        return len(self.tokens)

    def __call__(self, text: str) -> List[int]:
        return self.encode(text)

    text_to_ids = __call__

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def decode(self, tokens: Sequence[int]) -> str:
        return self.sep.join(self.tokens[int(t)] for t in tokens if int(t) not in self._util_ids)

    ids_to_text = decode


class BaseCharsTokenizer(BaseTokenizer):
    """Characters of ``chars`` (+ space, apostrophe and punctuation when asked).  Characters outside the inventory are dropped (with
    the OOV id when ``keep_oov``); runs of spaces collapse; ``pad_with_space`` surrounds the utterance with a space."""

    PUNCT_LIST = tuple(",.!?-:;/\"()[]{}")

    def __init__(self, chars: str, punct: bool = True, apostrophe: bool = True, add_blank_at: Optional[str] = None, pad_with_space: bool = False,
                 non_default_punct_list: Optional[Sequence[str]] = None, text_preprocessing_func: Callable[[str], str] = any_locale_text_preprocessing, keep_oov: bool = False):
        tokens = [" "] + list(chars)
        if apostrophe and "'" not in tokens:
            tokens.append("'")
        self.punct_list = list(non_default_punct_list) if non_default_punct_list is not None else list(self.PUNCT_LIST)
        if punct:
            tokens += [p for p in self.punct_list if p not in tokens]
        super().__init__(tokens, add_blank_at=add_blank_at, sep="")
        self.punct, self.pad_with_space, self.prep, self.keep_oov = punct, pad_with_space, text_preprocessing_func, keep_oov

    def encode(self, text: str) -> List[int]:
        text = self.prep(text)
        space = self._token2id[" "]
        out: List[int] = []
        for c in text:
            if c in self._token2id and (self.punct or c not in self.punct_list):
                if c == " " and out and out[-1] == space:
                    continue
                out.append(self._token2id[c])
            elif self.keep_oov:
                out.append(self.oov)
        while out and out[-1] == space:
            out.pop()
        while out and out[0] == space:
            out.pop(0)
        return [space] + out + [space] if self.pad_with_space else out


def _locale_chars(locale: str, lower: bool = True):
    return get_grapheme_character_set(locale, "lower" if lower else "mixed")


class EnglishCharsTokenizer(BaseCharsTokenizer):
    def __init__(self, punct=True, apostrophe=True, add_blank_at=None, pad_with_space=False, non_default_punct_list=None, text_preprocessing_func=english_text_preprocessing):
        super().__init__(string.ascii_lowercase, punct, apostrophe, add_blank_at, pad_with_space, non_default_punct_list, text_preprocessing_func)


class _LowerLocaleChars(BaseCharsTokenizer):
    LOCALE = "en-US"

    def __init__(self, punct=True, apostrophe=True, add_blank_at=None, pad_with_space=False, non_default_punct_list=None, text_preprocessing_func=None):
        prep = text_preprocessing_func or (lambda t: any_locale_text_preprocessing(t).lower())
        punct_list = non_default_punct_list if non_default_punct_list is not None else get_ipa_punctuation_list(self.LOCALE)
        super().__init__(_locale_chars(self.LOCALE).replace("'", ""), punct, apostrophe, add_blank_at, pad_with_space, punct_list, prep)


class GermanCharsTokenizer(BaseCharsTokenizer):
    """German keeps case: nouns are capitalised and the case carries meaning for pronunciation models."""

    def __init__(self, punct=True, apostrophe=True, add_blank_at=None, pad_with_space=False, non_default_punct_list=None, text_preprocessing_func=any_locale_text_preprocessing):
        punct_list = non_default_punct_list if non_default_punct_list is not None else get_ipa_punctuation_list("de-DE")
        super().__init__(get_grapheme_character_set("de-DE", "mixed"), punct, apostrophe, add_blank_at, pad_with_space, punct_list, text_preprocessing_func)


class SpanishCharsTokenizer(_LowerLocaleChars):
    LOCALE = "es-ES"


class FrenchCharsTokenizer(_LowerLocaleChars):
    LOCALE = "fr-FR"


class ItalianCharsTokenizer(_LowerLocaleChars):
    LOCALE = "it-IT"


class VietnameseCharsTokenizer(_LowerLocaleChars):
    LOCALE = "vi-VN"


class HindiCharsTokenizer(BaseCharsTokenizer):
    def __init__(self, punct=True, apostrophe=True, add_blank_at=None, pad_with_space=False, non_default_punct_list=None, text_preprocessing_func=any_locale_text_preprocessing):
        deva = "".join(chr(c) for c in range(0x0900, 0x0980) if unicodedata.category(chr(c))[0] in "LMN")
        super().__init__(deva + string.ascii_lowercase, punct, apostrophe, add_blank_at, pad_with_space, (non_default_punct_list or list(self.PUNCT_LIST) + ["।"]),
                         text_preprocessing_func)


class ArabicCharsTokenizer(BaseCharsTokenizer):
    def __init__(self, punct=True, apostrophe=True, add_blank_at=None, pad_with_space=False, non_default_punct_list=None, text_preprocessing_func=any_locale_text_preprocessing):
        letters = "".join(chr(c) for c in range(0x0621, 0x064B)) + "".join(chr(c) for c in range(0x064B, 0x0653))      # letters and short-vowel marks
        super().__init__(letters + string.ascii_lowercase, punct, apostrophe, add_blank_at, pad_with_space, (non_default_punct_list or list(self.PUNCT_LIST) + ["،", "؛", "؟"]),
                         text_preprocessing_func)


# ------------------------------------------------------------------------------------------------ phoneme tokenizers
_ARPABET_VOWELS = ("AA", "AE", "AH", "AO", "AW", "AY", "EH", "ER", "EY", "IH", "IY", "OW", "OY", "UH", "UW")
_ARPABET_CONSONANTS = ("B", "CH", "D", "DH", "F", "G", "HH", "JH", "K", "L", "M", "N", "NG", "P", "R", "S", "SH", "T", "TH", "V", "W", "Y", "Z", "ZH")


class EnglishPhonemesTokenizer(BaseTokenizer):
    """``g2p(text) -> symbols`` (ARPABET phonemes, characters for words it does not convert, punctuation, spaces).  With ``stresses``
    the vowels carry their stress digit (``AH0``), without it the digit is removed; ``chars`` adds the lower-case letters so that
    mixed grapheme / phoneme input is representable."""

    PUNCT_LIST = BaseCharsTokenizer.PUNCT_LIST

    def __init__(self, g2p: Callable[[str], List[str]], punct: bool = True, non_default_punct_list=None, stresses: bool = False, chars: bool = False, space: str = " ",
                 silence: Optional[str] = None, apostrophe: bool = True, add_blank_at: Optional[str] = None, pad_with_space: bool = False,
                 text_preprocessing_func: Callable[[str], str] = lambda t: english_text_preprocessing(t, lower=False)):
        self.phoneme_probability = getattr(g2p, "phoneme_probability", None)
        tokens = [space] + ([silence] if silence else [])
        tokens += list(_ARPABET_CONSONANTS)
        tokens += [f"{v}{s}" for v in _ARPABET_VOWELS for s in range(3)] if stresses else list(_ARPABET_VOWELS)
        if chars:
            tokens += list(string.ascii_lowercase)
        if apostrophe:
            tokens.append("'")
        self.punct_list = list(non_default_punct_list) if non_default_punct_list is not None else list(self.PUNCT_LIST)
        if punct:
            tokens += self.punct_list
        super().__init__(tokens, add_blank_at=add_blank_at)
        self.g2p, self.punct, self.stresses, self.space, self.pad_with_space, self.prep = g2p, punct, stresses, space, pad_with_space, text_preprocessing_func

    def encode(self, text: str) -> List[int]:
        return self.encode_from_g2p(self.g2p(self.prep(text)))

    def encode_from_g2p(self, symbols: Sequence[str]) -> List[int]:
        sp = self._token2id[self.space]
        out: List[int] = []
        for p in symbols:
            if p == " " or p == self.space:
                if out and out[-1] != sp:
                    out.append(sp)
                continue
            if not self.stresses and len(p) == 3 and p[-1].isdigit() and p[:2] in _ARPABET_VOWELS:
                p = p[:2]
            if p in self._token2id and (self.punct or p not in self.punct_list):
                out.append(self._token2id[p])
            elif p.lower() in self._token2id and len(p) == 1:
                out.append(self._token2id[p.lower()])
        while out and out[-1] == sp:
            out.pop()
        return [sp] + out + [sp] if self.pad_with_space else out


class IPATokenizer(BaseTokenizer):
    """Symbols come from ``g2p`` (an ``IpaG2p``): its phoneme inventory plus, when it can emit graphemes, the (prefixed) grapheme set
    of the locale.  ``fixed_vocab`` pins the inventory (for compatibility with a trained model): symbols outside it are removed
    from the G2P dictionary so that they cannot be produced."""

    def __init__(self, g2p, locale: Optional[str] = "en-US", punct: bool = True, non_default_punct_list=None, fixed_vocab: Optional[Sequence[str]] = None, space: str = " ",
                 silence: Optional[str] = None, apostrophe: bool = False, add_blank_at: Optional[str] = None, pad_with_space: bool = False):
        if not hasattr(g2p, "symbols"):
            raise ValueError("g2p must expose its symbol inventory (.symbols)")
        if fixed_vocab is not None:
            g2p.replace_symbols(set(fixed_vocab), keep_alternate=True)
            symbols = set(fixed_vocab)
        else:
            symbols = set(g2p.symbols)
            prefix = getattr(g2p, "prefix", "")
            if locale is not None and (getattr(g2p, "use_chars", False) or getattr(g2p, "p", None) is not None):
                case = {"upper": "upper", "lower": "lower", None: "mixed"}.get(getattr(g2p, "case", "upper"), "upper")
                symbols |= {prefix + c for c in get_grapheme_character_set(locale, case)}
        tokens = [space] + ([silence] if silence else []) + sorted(symbols - {space})
        if apostrophe and "'" not in tokens:
            tokens.append("'")
        self.punct_list = list(non_default_punct_list) if non_default_punct_list is not None else get_ipa_punctuation_list(locale)
        if punct:
            tokens += [p for p in self.punct_list if p not in tokens]
        super().__init__(tokens, add_blank_at=add_blank_at, sep="")
        self.g2p, self.punct, self.space, self.pad_with_space, self.locale = g2p, punct, space, pad_with_space, locale
        self.phoneme_probability = getattr(g2p, "p", None)

    def encode(self, text: str) -> List[int]:
        return self.encode_from_g2p(self.g2p(any_locale_text_preprocessing(text)))

    def encode_from_g2p(self, symbols: Sequence[str]) -> List[int]:
        sp = self._token2id[self.space]
        out: List[int] = []
        for p in symbols:
            if p == " ":
                if out and out[-1] != sp:
                    out.append(sp)
            elif p in self._token2id and (self.punct or p not in self.punct_list):
                out.append(self._token2id[p])
        while out and out[-1] == sp:
            out.pop()
        return [sp] + out + [sp] if self.pad_with_space else out


class ChinesePhonemesTokenizer(BaseTokenizer):
    """Pinyin initials / finals / tone marks from a ``ChineseG2p`` plus upper-case Latin letters and Chinese punctuation."""

    PUNCT = list("，。？！；：、‘’“”（）【】「」《》") + list(",.?!;:'\"()")

    def __init__(self, g2p, symbols: Sequence[str], punct: bool = True, add_blank_at: Optional[str] = None, pad_with_space: bool = False, space: str = " "):
        tokens = [space] + list(symbols) + list(string.ascii_uppercase)
        if punct:
            tokens += [p for p in self.PUNCT if p not in tokens]
        super().__init__(tokens, add_blank_at=add_blank_at)
        self.g2p, self.space, self.pad_with_space = g2p, space, pad_with_space

    def encode(self, text: str) -> List[int]:
        sp = self._token2id[self.space]
        out = [self._token2id[s] for s in self.g2p(text) if s in self._token2id]
        return [sp] + out + [sp] if self.pad_with_space else out


class JapanesePhonemeTokenizer(ChinesePhonemesTokenizer):
    PUNCT = list("、。？！・「」『』（）") + list(",.?!;:'\"()")


class AggregatedTTSTokenizer:
    """Several tokenizers side by side: tokenizer k's ids are shifted by the sizes of the ones before it, so that one embedding
    table serves them all; ``encode(text, tokenizer_name)`` picks one."""

    def __init__(self, tokenizers: Sequence, tokenizer_names: Sequence[str]):
        if len(tokenizers) != len(tokenizer_names):
            raise ValueError("one name per tokenizer")
        self.tokenizers = dict(zip(tokenizer_names, tokenizers))
        self.offsets, off = {}, 0
        self.tokens: List[str] = []
        for n, t in self.tokenizers.items():
            self.offsets[n] = off
            size = getattr(t, "vocab_size", None) or len(t.tokens)
            toks = list(getattr(t, "tokens", [f"{n}_{i}" for i in range(size)]))
            self.tokens += toks
            off += size
        self.num_tokens = off
        first = next(iter(self.tokenizers))
        self.pad = self.offsets[first] + self.tokenizers[first].pad
        self.first_tokenizer = self.tokenizers[first]

    @property
    def vocab_size(self) -> int:
        return self.num_tokens

    def encode(self, text: str, tokenizer_name: str) -> List[int]:
        t = self.tokenizers[tokenizer_name]
        off = self.offsets[tokenizer_name]
        return [off + i for i in (t.encode(text) if hasattr(t, "encode") else t.text_to_ids(text))]

    def decode(self, tokens: Sequence[int], tokenizer_name: Optional[str] = None) -> str:
        if tokenizer_name is not None:
            off = self.offsets[tokenizer_name]
            return self.tokenizers[tokenizer_name].decode([int(t) - off for t in tokens])
        return "".join(self.tokens[int(t)] for t in tokens)

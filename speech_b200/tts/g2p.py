"""Grapheme-to-phoneme conversion beyond a plain dictionary lookup.

* ``IpaG2p`` — dictionary G2P for any locale with IPA symbols: several pronunciations per word, heteronyms left as graphemes,
  possessive / hyphen handling, optional grapheme prefix so that graphemes and phonemes share no symbols, stress removal,
  mixing of graphemes and phonemes during training.
* ``ChineseG2p`` (pinyin syllables → initials / finals + tone), ``JapaneseG2p`` (kana → IPA mora table) — both take the
  word segmenter / reader as an injected callable, because those come from optional packages.
* ``CTCG2PModel`` — character encoder trained with CTC on phoneme targets (the input is up-sampled so that phoneme strings
  longer than the spelling are reachable); ``Seq2SeqG2PModel`` — byte-level encoder-decoder Transformer (the role the
  reference gives to a pre-trained ByT5).
* ``G2PModel.convert_graphemes_to_phonemes`` for manifests, phoneme error rate.

References: ``tts/g2p/models/i18n_ipa.py`` (``IpaG2p``), ``zh_cn_pinyin.py``, ``ja_jp_ipa.py``, ``ctc.py`` (``CTCG2PModel``), ``t5.py``
(``T5G2PModel``), ``base.py``.
"""
from __future__ import annotations

import json
import re
import unicodedata
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from ..core.config import DictConfig, cfg_get
from ..core.modelpt import ModelPT

__all__ = ["ChineseG2p", "CTCG2PModel", "G2PModel", "IpaG2p", "JapaneseG2p", "Seq2SeqG2PModel", "T5G2PModel", "phoneme_error_rate"]

_STRESS = "ˈˌ"
_PUNCT = ",.!?;:\"()¿¡«»—-…"


def _edit_distance(a: Sequence, b: Sequence) -> int:
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


def phoneme_error_rate(hyps: Sequence[Sequence[str]], refs: Sequence[Sequence[str]]) -> float:
    errs = sum(_edit_distance(h, r) for h, r in zip(hyps, refs))
    return errs / max(1, sum(len(r) for r in refs))


# ------------------------------------------------------------------------------------------------ IPA dictionary G2P
class IpaG2p:
    """``phoneme_dict``: a path (lines ``word<TAB or two spaces>ipa[, ipa2...]``) or ``{word: [ipa, ...]}`` where an ipa entry
    is a string (split into characters, combining marks attached to their base) or a list of symbols."""

    def __init__(self, phoneme_dict, locale: str = "en-US", apply_to_oov_word: Optional[Callable[[str], List[str]]] = None,
                 ignore_ambiguous_words: bool = True, heteronyms: Optional[Iterable[str]] = None, use_chars: bool = False,
                 phoneme_probability: Optional[float] = None, use_stresses: bool = True, grapheme_case: Optional[str] = "upper",
                 grapheme_prefix: str = "", mapping_file: Optional[str] = None, seed: int = 0):
        self.locale, self.oov_fn, self.ignore_ambiguous = locale, apply_to_oov_word, ignore_ambiguous_words
        self.use_chars, self.p, self.use_stresses = use_chars, phoneme_probability, use_stresses
        self.case, self.prefix = grapheme_case, grapheme_prefix
        self.rng = np.random.default_rng(seed)
        self.heteronyms: Set[str] = set()
        if heteronyms is not None:
            src = open(heteronyms, encoding="utf-8").read().split() if isinstance(heteronyms, str) else heteronyms
            self.heteronyms = {self._case(w) for w in src}
        self.mapping: Dict[str, str] = json.load(open(mapping_file, encoding="utf-8")) if mapping_file else {}
        self.phoneme_dict: Dict[str, List[List[str]]] = {}
        self.symbols: Set[str] = set()
        self.replace_dict(phoneme_dict)

    # .............................................................. dictionary
    def _case(self, w: str) -> str:
        return w.upper() if self.case == "upper" else w.lower() if self.case == "lower" else w

    @staticmethod
    def split_ipa(s: str) -> List[str]:
        """Characters of an IPA string, combining marks and length / tie marks attached to the preceding symbol."""
        out: List[str] = []
        for ch in unicodedata.normalize("NFC", s):
            if out and (unicodedata.combining(ch) or ch in "ːˑ͡"):
                out[-1] += ch
            elif out and out[-1].endswith("͡"):
                out[-1] += ch
            elif not ch.isspace():
                out.append(ch)
        return out

    def replace_dict(self, phoneme_dict):
        entries: Dict[str, List] = {}
        if isinstance(phoneme_dict, dict):
            entries = {w: (p if isinstance(p, (list, tuple)) and not (p and isinstance(p[0], str) and len(p[0]) == 1 and all(len(x) == 1 for x in p)) else [p])
                       for w, p in phoneme_dict.items()}
        else:
            with open(phoneme_dict, encoding="utf-8") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if not line.strip() or line.startswith(";;;"):
                        continue
                    if line[0] != "'" and not line[0].isalnum() and not unicodedata.category(line[0]).startswith("L"):
                        continue                                     # symbol entries of pronunciation lexicons
                    w, _, rest = line.partition("\t") if "\t" in line else line.partition("  ")
                    entries.setdefault(w.strip(), []).extend(x.strip() for x in rest.split(",") if x.strip())
        self.phoneme_dict, self.symbols = {}, set()
        for w, prons in entries.items():
            plist = []
            for p in prons:
                syms = list(p) if isinstance(p, (list, tuple)) else self.split_ipa(p)
                if not self.use_stresses:
                    syms = [s for s in syms if s not in _STRESS]
                syms = [self.mapping.get(s, s) for s in syms]
                plist.append(syms)
                self.symbols.update(syms)
            self.phoneme_dict[self._case(w)] = plist

    def replace_symbols(self, symbols: Iterable[str], keep_alternate: bool = True):
        """Keeps only pronunciations spelled with ``symbols``; words left without any are dropped (``keep_alternate=False`` also
        drops a word as soon as one of its pronunciations uses a foreign symbol)."""
        allowed = set(symbols)
        new = {}
        for w, prons in self.phoneme_dict.items():
            ok = [p for p in prons if set(p) <= allowed]
            if ok and (keep_alternate or len(ok) == len(prons)):
                new[w] = ok
        self.phoneme_dict, self.symbols = new, allowed & self.symbols

    def is_unique_in_phoneme_dict(self, word: str) -> bool:
        return len(self.phoneme_dict[word]) == 1

    # .............................................................. one word
    def _graphemes(self, word: str) -> List[str]:
        return [self.prefix + ch for ch in word]

    def parse_one_word(self, word: str) -> Tuple[List[str], bool]:
        """``(symbols, handled)``; ``handled`` False means the word is unknown and the caller applies its OOV rule."""
        w = self._case(word)
        if self.p is not None and self.rng.random() > self.p:
            return self._graphemes(w), True
        if w in self.heteronyms:
            return self._graphemes(w), True
        d = self.phoneme_dict

        def lookup(x):
            if x in d and (not self.ignore_ambiguous or self.is_unique_in_phoneme_dict(x)):
                return d[x][0]
            return None

        got = lookup(w)
        if got is not None:
            return list(got), True
        if w in d:                                                   # ambiguous and not allowed to pick: spell it
            return self._graphemes(w), True
        if self.locale.startswith("en"):
            s_up, s = self._case("'S"), self._case("S")
            if len(w) > 2 and w.endswith(s_up) and lookup(w[:-2]) is not None:
                base = lookup(w[:-2])
                return base + (["s"] if base[-1] in "ptkfθ" else ["ɪ", "z"] if base[-1] in "szʃʒ" or base[-1].endswith("ʃ") or base[-1].endswith("ʒ") else ["z"]), True
            if len(w) > 1 and w.endswith(s) and lookup(w[:-1]) is not None:
                base = lookup(w[:-1])
                return base + (["s"] if base[-1] in "ptkfθ" else ["z"]), True
        if self.locale.startswith("fr") and "'" in w:                # elided article: l'ami -> l + ami
            head, _, rest = w.partition("'")
            if lookup(rest) is not None and head:
                h = lookup(head + "'") or lookup(head) or self._graphemes(head)
                return list(h) + lookup(rest), True
        if "-" in w:
            parts = [self.parse_one_word(p) for p in w.split("-") if p]
            if parts and all(ok for _, ok in parts):
                out: List[str] = []
                for k, (syms, _) in enumerate(parts):
                    out += (["-"] if k else []) + syms
                return out, True
        if self.use_chars:
            return self._graphemes(w), True
        return [], False

    def __call__(self, text: str) -> List[str]:
        text = unicodedata.normalize("NFC", text)
        out: List[str] = []
        for tok in re.findall(r"[^\W\d_]+(?:['’\-][^\W\d_]+)*|\d+|\s+|[^\w\s]", text, flags=re.UNICODE):
            if tok.isspace():
                out.append(" ")
            elif tok[0].isalpha():
                syms, ok = self.parse_one_word(tok.replace("’", "'"))
                if not ok:
                    syms = self.oov_fn(tok) if self.oov_fn is not None else self._graphemes(self._case(tok))
                out += syms
            else:
                out.append(tok)
        return out


# ------------------------------------------------------------------------------------------------ Mandarin / Japanese
_PINYIN_INITIALS = ("zh", "ch", "sh", "b", "p", "m", "f", "d", "t", "n", "l", "g", "k", "h", "j", "q", "x", "r", "z", "c", "s", "y", "w")


class ChineseG2p:
    """Mandarin text → pinyin units.  ``word_segmenter(text) -> words`` and ``pinyin_reader(word) -> ["ni3", "hao3"]`` come from
    the caller (dictionary-backed defaults: a ``phoneme_dict`` of ``{word or character: "ni3 hao3"}`` with longest-match
    segmentation).  Each syllable is split into initial, final and tone (``#3``); Latin words are spelled in upper case."""

    def __init__(self, phoneme_dict: Optional[Dict[str, str]] = None, word_segmenter: Optional[Callable[[str], List[str]]] = None,
                 pinyin_reader: Optional[Callable[[str], List[str]]] = None, tone_prefix: str = "#", ascii_letter_prefix: str = "",
                 ascii_letter_case: str = "upper"):
        if isinstance(phoneme_dict, str):
            d = {}
            for line in open(phoneme_dict, encoding="utf-8"):
                if line.strip():
                    w, _, p = line.strip().partition("\t")
                    d[w] = p
            phoneme_dict = d
        self.dict = dict(phoneme_dict or {})
        self.max_word = max((len(w) for w in self.dict), default=1)
        self.segment = word_segmenter or self._longest_match
        self.read = pinyin_reader or self._dict_read
        self.tone_prefix, self.ascii_prefix, self.ascii_case = tone_prefix, ascii_letter_prefix, ascii_letter_case

    def _longest_match(self, text: str) -> List[str]:
        out, i = [], 0
        while i < len(text):
            if text[i].isascii():
                m = re.match(r"[A-Za-z]+|\s+|.", text[i:])
                out.append(m.group(0))
                i += len(m.group(0))
                continue
            for n in range(min(self.max_word, len(text) - i), 0, -1):
                if text[i:i + n] in self.dict or n == 1:
                    out.append(text[i:i + n])
                    i += n
                    break
        return out

    def _dict_read(self, word: str) -> List[str]:
        if word in self.dict:
            return self.dict[word].split()
        out = []
        for ch in word:
            out += self.dict[ch].split() if ch in self.dict else [ch]
        return out

    @staticmethod
    def split_syllable(syl: str) -> Tuple[str, str, str]:
        m = re.fullmatch(r"([a-zü:]+?)([1-5]?)", syl.lower())
        if not m:
            return "", syl, ""
        body, tone = m.group(1).replace("u:", "ü"), m.group(2) or "5"
        for ini in _PINYIN_INITIALS:
            if body.startswith(ini) and len(body) > len(ini):
                return ini, body[len(ini):], tone
        return "", body, tone

    def __call__(self, text: str) -> List[str]:
        out: List[str] = []
        for w in self.segment(text):
            if w.isspace():
                out.append(" ")
            elif w.isascii() and w.isalpha():
                w = w.upper() if self.ascii_case == "upper" else w.lower()
                out += [self.ascii_prefix + c for c in w]
            elif w.isascii():
                out.append(w)
            else:
                for syl in self.read(w):
                    ini, fin, tone = self.split_syllable(syl)
                    if not tone:
                        out.append(syl)                               # punctuation or an unknown character
                        continue
                    out += ([ini] if ini else []) + [fin, f"{self.tone_prefix}{tone}"]
        return out


_KANA_IPA = {
    "ア": "a", "イ": "i", "ウ": "ɯ", "エ": "e", "オ": "o", "カ": "ka", "キ": "ki", "ク": "kɯ", "ケ": "ke", "コ": "ko", "サ": "sa", "シ": "ɕi", "ス": "sɯ",
    "セ": "se", "ソ": "so", "タ": "ta", "チ": "tɕi", "ツ": "tsɯ", "テ": "te", "ト": "to", "ナ": "na", "ニ": "ni", "ヌ": "nɯ", "ネ": "ne", "ノ": "no",
    "ハ": "ha", "ヒ": "çi", "フ": "ɸɯ", "ヘ": "he", "ホ": "ho", "マ": "ma", "ミ": "mi", "ム": "mɯ", "メ": "me", "モ": "mo", "ヤ": "ja", "ユ": "jɯ",
    "ヨ": "jo", "ラ": "ɾa", "リ": "ɾi", "ル": "ɾɯ", "レ": "ɾe", "ロ": "ɾo", "ワ": "wa", "ヲ": "o", "ン": "ɴ", "ガ": "ga", "ギ": "gi", "グ": "gɯ",
    "ゲ": "ge", "ゴ": "go", "ザ": "za", "ジ": "dʑi", "ズ": "zɯ", "ゼ": "ze", "ゾ": "zo", "ダ": "da", "ヂ": "dʑi", "ヅ": "zɯ", "デ": "de", "ド": "do",
    "バ": "ba", "ビ": "bi", "ブ": "bɯ", "ベ": "be", "ボ": "bo", "パ": "pa", "ピ": "pi", "プ": "pɯ", "ペ": "pe", "ポ": "po",
}
_SMALL_Y = {"ャ": "a", "ュ": "ɯ", "ョ": "o"}


class JapaneseG2p:
    """Japanese text → IPA through katakana readings.  ``kana_reader(text) -> katakana`` (a morphological analyser) is supplied by
    the caller; kana input needs none.  Handles palatalised morae (キャ), the geminate mark (ッ doubles the next consonant) and
    the long-vowel mark (ー lengthens the previous vowel)."""

    def __init__(self, kana_reader: Optional[Callable[[str], str]] = None, word_sep: str = " "):
        self.read = kana_reader
        self.word_sep = word_sep

    @staticmethod
    def _to_katakana(s: str) -> str:
        return "".join(chr(ord(c) + 0x60) if "ぁ" <= c <= "ゖ" else c for c in s)

    def kana_to_ipa(self, kana: str) -> List[str]:
        kana = self._to_katakana(kana)
        out: List[str] = []
        geminate = False
        i = 0
        while i < len(kana):
            c = kana[i]
            if c == "ッ":
                geminate = True
            elif c == "ー":
                if out:
                    out[-1] += "ː"
            elif c in _KANA_IPA:
                ipa = _KANA_IPA[c]
                if i + 1 < len(kana) and kana[i + 1] in _SMALL_Y and ipa.endswith("i"):
                    stem = ipa[:-1]
                    ipa = stem + ("" if stem[-1] in "ɕʑç" else "j") + _SMALL_Y[kana[i + 1]]
                    i += 1
                syms = IpaG2p.split_ipa(ipa)
                if geminate and syms and syms[0][0] not in "aiɯeo":
                    syms = [syms[0]] + syms
                geminate = False
                out += syms
            elif c.isspace():
                out.append(self.word_sep)
            else:
                out.append(c)
            i += 1
        return out

    def __call__(self, text: str) -> List[str]:
        if self.read is not None:
            text = self.read(text)
        elif any("一" <= c <= "鿿" for c in text):
            raise ValueError("kanji need a reader: pass kana_reader (a morphological analyser returning katakana)")
        return self.kana_to_ipa(text)


# ------------------------------------------------------------------------------------------------ neural G2P
class _SymbolTable:
    def __init__(self, symbols: Sequence[str], specials: Sequence[str] = ("<pad>", "<bos>", "<eos>", "<unk>")):
        self.tokens = list(specials) + [s for s in dict.fromkeys(symbols) if s not in specials]
        self.t2i = {t: i for i, t in enumerate(self.tokens)}
        self.pad, self.bos, self.eos, self.unk = 0, 1, 2, 3

    def __len__(self):
        return len(self.tokens)

    def encode(self, syms: Sequence[str]) -> List[int]:
        return [self.t2i.get(s, self.unk) for s in syms]

    def decode(self, ids: Sequence[int]) -> List[str]:
        return [self.tokens[int(i)] for i in ids if int(i) > 3]


class G2PModel(ModelPT):
    """Shared by the neural G2P models: ``(graphemes, phonemes)`` example lists as data, batch collation, manifest conversion."""

    def _examples_from(self, config) -> List[Tuple[str, List[str]]]:
        ex = []
        if config is None:
            return ex
        for item in config.get("examples", []) or []:
            ex.append((item[0], list(item[1]) if not isinstance(item[1], str) else item[1].split()))
        path = config.get("manifest_filepath", None)
        if path:
            gf, pf = config.get("grapheme_field", "text_graphemes"), config.get("phoneme_field", "text")
            for line in open(path, encoding="utf-8"):
                if line.strip():
                    d = json.loads(line)
                    ex.append((d[gf], d[pf].split() if " " in d[pf] else IpaG2p.split_ipa(d[pf])))
        return ex

    def _loader(self, config, shuffle=False):
        ex = self._examples_from(config)
        if not ex:
            return None
        bs = int(config.get("batch_size", 8))
        return torch.utils.data.DataLoader(ex, batch_size=bs, shuffle=shuffle and bool(config.get("shuffle", True)), collate_fn=self._collate)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c, shuffle=True)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def setup_test_data(self, c):
        self._test_dl = self._loader(c)

    def _encode_text(self, texts: Sequence[str]) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = [self.graphemes.encode(list(t.lower() if self.lower else t)) for t in texts]
        lens = torch.tensor([len(i) for i in ids])
        x = torch.zeros(len(ids), int(lens.max()), dtype=torch.long)
        for b, i in enumerate(ids):
            x[b, : len(i)] = torch.tensor(i)
        return x, lens

    def _collate(self, items):
        x, xl = self._encode_text([g for g, _ in items])
        ys = [self.phonemes.encode(p) for _, p in items]
        yl = torch.tensor([len(y) for y in ys])
        y = torch.zeros(len(ys), int(yl.max()), dtype=torch.long)
        for b, v in enumerate(ys):
            y[b, : len(v)] = torch.tensor(v)
        return x, xl, y, yl

    @torch.no_grad()
    def convert_graphemes_to_phonemes(self, manifest_filepath: str, output_manifest_filepath: str, grapheme_field: str = "text_graphemes",
                                      batch_size: int = 32, pred_field: str = "pred_text") -> List[str]:
        """Adds ``pred_field`` (space-joined phonemes) to every line of a JSON-lines manifest."""
        rows = [json.loads(l) for l in open(manifest_filepath, encoding="utf-8") if l.strip()]
        preds: List[str] = []
        for s in range(0, len(rows), batch_size):
            preds += [" ".join(p) for p in self.predict([r[grapheme_field] for r in rows[s:s + batch_size]])]
        with open(output_manifest_filepath, "w", encoding="utf-8") as f:
            for r, p in zip(rows, preds):
                r[pred_field] = p
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        return preds

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        x, xl, y, yl = batch
        hyps = self._predict_ids(x, xl)
        refs = [self.phonemes.decode(y[b, : int(yl[b])].tolist()) for b in range(y.shape[0])]
        return {"val_per": torch.tensor(phoneme_error_rate(hyps, refs)), "val_loss": self._loss(batch).detach()}

    def training_step(self, batch, batch_idx):
        loss = self._loss(batch)
        self.log("train_loss", loss.detach())
        return {"loss": loss}

    @torch.no_grad()
    def predict(self, texts: Sequence[str]) -> List[List[str]]:
        was = self.training
        self.eval()
        x, xl = self._encode_text(texts)
        dev = next(self.parameters()).device
        out = self._predict_ids(x.to(dev), xl.to(dev))
        self.train(was)
        return out


class CTCG2PModel(G2PModel):
    """Characters → embedding → each position repeated ``upsample`` times (+ a learned phase embedding) → Transformer encoder →
    CTC over the phoneme inventory."""

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        from ..modules.transformer import TransformerEncoder

        cfg = self._cfg
        self.lower = bool(cfg_get(cfg, "lowercase", True))
        self.graphemes = _SymbolTable(list(cfg_get(cfg, "graphemes", "abcdefghijklmnopqrstuvwxyz' -")))
        self.phonemes = _SymbolTable(list(cfg_get(cfg, "phonemes")))
        d, self.up = int(cfg_get(cfg, "d_model", 128)), int(cfg_get(cfg, "upsample", 2))
        self.embed = nn.Embedding(len(self.graphemes), d, padding_idx=0)
        self.phase = nn.Embedding(self.up, d)
        self.pos = nn.Embedding(int(cfg_get(cfg, "max_len", 512)) * self.up, d)
        self.encoder = TransformerEncoder(int(cfg_get(cfg, "n_layers", 2)), d, 4 * d, num_attention_heads=int(cfg_get(cfg, "n_heads", 4)), pre_ln=True)
        self.head = nn.Linear(d, len(self.phonemes) + 1)
        self.blank = len(self.phonemes)
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def forward(self, input_ids, input_len):
        B, T = input_ids.shape
        h = self.embed(input_ids).repeat_interleave(self.up, dim=1)
        idx = torch.arange(T * self.up, device=h.device)
        h = h + self.phase(idx % self.up)[None] + self.pos(idx)[None]
        lens = input_len * self.up
        mask = (idx[None, :] < lens[:, None]).to(h.dtype)
        return F.log_softmax(self.head(self.encoder(h, mask)).float(), dim=-1), lens

    def _loss(self, batch):
        x, xl, y, yl = batch
        lp, lens = self(x, xl)
        return F.ctc_loss(lp.transpose(0, 1), y, lens, yl, blank=self.blank, zero_infinity=True)

    def _predict_ids(self, x, xl):
        lp, lens = self(x, xl)
        best = lp.argmax(-1)
        out = []
        for b in range(best.shape[0]):
            seq, prev = [], self.blank
            for t in best[b, : int(lens[b])].tolist():
                if t != prev and t != self.blank:
                    seq.append(t)
                prev = t
            out.append(self.phonemes.decode(seq))
        return out


class Seq2SeqG2PModel(G2PModel):
    """Byte-level encoder-decoder Transformer: UTF-8 bytes of the spelling in, phoneme symbols out, greedy or beam decoding."""

    def __init__(self, cfg: DictConfig, trainer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        from ..modules.transformer_nm import GreedySequenceGenerator, TokenClassifier, TransformerDecoderNM, TransformerEncoderNM

        cfg = self._cfg
        self.lower = bool(cfg_get(cfg, "lowercase", True))
        self.graphemes = _SymbolTable([bytes([b]).decode("latin-1") for b in range(256)])
        self.phonemes = _SymbolTable(list(cfg_get(cfg, "phonemes")))
        d, L, H = int(cfg_get(cfg, "d_model", 128)), int(cfg_get(cfg, "n_layers", 2)), int(cfg_get(cfg, "n_heads", 4))
        self.max_len = int(cfg_get(cfg, "max_len", 256))
        self.encoder = TransformerEncoderNM(len(self.graphemes), d, L, 4 * d, H, max_sequence_length=self.max_len, pre_ln=True)
        self.decoder = TransformerDecoderNM(len(self.phonemes), d, L, 4 * d, H, max_sequence_length=self.max_len, pre_ln=True)
        self.classifier = TokenClassifier(d, len(self.phonemes))
        self.generator = GreedySequenceGenerator(self.decoder.embedding, self.decoder.decoder, self.classifier, pad=0, bos=1, eos=2,
                                                 max_sequence_length=self.max_len, max_delta_length=int(cfg_get(cfg, "max_delta_length", 24)))
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _encode_text(self, texts):
        ids = [[4 + b for b in (t.lower() if self.lower else t).encode("utf-8")] for t in texts]      # 4 specials in front of the 256 bytes
        lens = torch.tensor([len(i) for i in ids])
        x = torch.zeros(len(ids), int(lens.max()), dtype=torch.long)
        for b, i in enumerate(ids):
            x[b, : len(i)] = torch.tensor(i)
        return x, lens

    def _encode(self, x, xl):
        mask = (torch.arange(x.shape[1], device=x.device)[None, :] < xl[:, None]).long()
        return self.encoder(x, mask), mask

    def _loss(self, batch):
        x, xl, y, yl = batch
        enc, emask = self._encode(x, xl)
        B, T = y.shape
        tgt_in = torch.cat([torch.full((B, 1), 1, dtype=torch.long, device=y.device), y], dim=1)
        tgt_out = torch.cat([y, torch.zeros(B, 1, dtype=torch.long, device=y.device)], dim=1)
        tgt_out[torch.arange(B, device=y.device), yl] = 2
        dmask = (torch.arange(T + 1, device=y.device)[None, :] <= yl[:, None]).long()
        logp = self.classifier(self.decoder(tgt_in, dmask, enc, emask))
        nll = F.nll_loss(logp.float().transpose(1, 2), tgt_out, reduction="none")
        return (nll * dmask).sum() / dmask.sum()

    def _predict_ids(self, x, xl):
        enc, emask = self._encode(x, xl)
        out = self.generator(encoder_hidden_states=enc, encoder_input_mask=emask)
        res = []
        for row in out[:, 1:].tolist():
            if 2 in row:
                row = row[: row.index(2)]
            res.append(self.phonemes.decode(row))
        return res


T5G2PModel = Seq2SeqG2PModel

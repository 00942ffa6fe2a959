"""Further tokenizers: word / regex / null / Chinese-character / English-Japanese / Moses-style / tiktoken, and chat templates.

Reference: ``common/tokenizers/word_tokenizer.py``, ``regex_tokenizer.py`` (regex-split tokens with a vocabulary file,
``<PAD> <UNK> ^ & <MASK> <SEP>`` specials), ``null_tokenizer.py`` (ids are their own text), ``chinese_tokenizers.py`` (per-character
with optional word segmenter), ``en_ja_tokenizers.py`` / ``moses_tokenizers.py`` (punctuation splitting / detokenisation),
``tiktoken_tokenizer.py`` (BPE ranks file + special tokens; needs the optional ``tiktoken`` package),
``chat_template_mixin.py`` (roles → one prompt string).
"""
from __future__ import annotations

import json
import re
from typing import Dict, Iterable, List, Optional, Sequence

from . import TokenizerSpec


class WordTokenizer(TokenizerSpec):
    """Whitespace words against a vocabulary file (one word per line); unknown words map to ``<UNK>``."""

    def __init__(self, vocab_file: Optional[str] = None, vocab: Optional[Sequence[str]] = None, pad_token="<PAD>", unk_token="<UNK>",
                 bos_token: Optional[str] = None, eos_token: Optional[str] = None):
        words = list(vocab) if vocab is not None else [l.rstrip("\n") for l in open(vocab_file, encoding="utf-8") if l.strip()]
        specials = [t for t in (pad_token, unk_token, bos_token, eos_token) if t]
        self.vocab = list(dict.fromkeys(specials + words))
        self._t2i = {t: i for i, t in enumerate(self.vocab)}
        self.pad_id, self.unk_id = self._t2i[pad_token], self._t2i[unk_token]
        self.bos_id = self._t2i.get(bos_token) if bos_token else None
        self.eos_id = self._t2i.get(eos_token) if eos_token else None

    def text_to_tokens(self, text):
        return text.split()

    def tokens_to_text(self, tokens):
        return " ".join(tokens)

    def tokens_to_ids(self, tokens):
        return [self._t2i.get(t, self.unk_id) for t in tokens]

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids]

    def text_to_ids(self, text):
        return self.tokens_to_ids(self.text_to_tokens(text))

    def ids_to_text(self, ids):
        return self.tokens_to_text([t for t in self.ids_to_tokens(ids) if t not in (self.vocab[self.pad_id],)])


class RegExTokenizer(WordTokenizer):
    """Tokens are the matches of a regular expression (default: a SMILES-style chemistry pattern in the reference; any pattern
    here); ``build_vocab_from_text`` collects the vocabulary."""

    DEFAULT_REGEX = r"\[[^\]]+\]|[A-Za-z][a-z]?|\d+|\S"

    def __init__(self, regex: Optional[str] = None, vocab: Optional[Sequence[str]] = None, vocab_file: Optional[str] = None, **kw):
        self.regex = re.compile(regex or self.DEFAULT_REGEX)
        super().__init__(vocab_file=vocab_file, vocab=vocab if vocab is not None or vocab_file else [], bos_token="^", eos_token="&", **kw)

    def text_to_tokens(self, text):
        return self.regex.findall(text)

    def tokens_to_text(self, tokens):
        return "".join(t for t in tokens if t not in ("^", "&"))

    def build_vocab_from_text(self, texts: Iterable[str]) -> None:
        for t in texts:
            for tok in self.text_to_tokens(t):
                if tok not in self._t2i:
                    self._t2i[tok] = len(self.vocab)
                    self.vocab.append(tok)


class NullTokenizer(TokenizerSpec):
    """For pre-tokenised data: text is a space-separated list of ids."""

    def __init__(self, vocab_size: int):
        self._vocab_size = vocab_size
        self.eos_id, self.pad_id, self.bos_id = vocab_size - 1, -1, -1

    vocab_size = property(lambda self: self._vocab_size)

    def text_to_ids(self, text):
        return [int(x) for x in text.split()]

    def ids_to_text(self, ids):
        return " ".join(str(int(i)) for i in ids)

    def text_to_tokens(self, text):
        return text.split()

    def tokens_to_text(self, tokens):
        return " ".join(tokens)

    def tokens_to_ids(self, tokens):
        return [int(t) for t in tokens]

    def ids_to_tokens(self, ids):
        return [str(int(i)) for i in ids]


class ChineseCharsTokenizer(WordTokenizer):
    """One token per CJK character; Latin runs stay whole words."""

    def text_to_tokens(self, text):
        return re.findall(r"[一-鿿぀-ヿ]|[^\s一-鿿぀-ヿ]+", text)

    def tokens_to_text(self, tokens):
        out = ""
        for t in tokens:
            cjk = bool(re.match(r"[一-鿿぀-ヿ]", t))
            out += t if cjk or not out or re.match(r"[一-鿿぀-ヿ]", out[-1]) else " " + t
        return out


class EnJaProcessor:
    """Pre / post-processing for English and Japanese text (punctuation split off for English, characters for Japanese)."""

    def __init__(self, lang_id: str):
        if lang_id not in ("en", "ja"):
            raise ValueError("lang_id must be 'en' or 'ja'")
        self.lang_id = lang_id

    def tokenize(self, text: str) -> str:
        if self.lang_id == "ja":
            return " ".join(ChineseCharsTokenizer(vocab=[]).text_to_tokens(text))
        return MosesProcessor("en").tokenize(text)

    def detokenize(self, tokens: List[str]) -> str:
        if self.lang_id == "ja":
            return "".join(tokens)
        return MosesProcessor("en").detokenize(tokens)

    def normalize(self, text: str) -> str:
        return re.sub(r"\s+", " ", text).strip()


class MosesProcessor:
    """Rule-based tokenisation / detokenisation in the manner of the Moses scripts (punctuation separated, contractions kept)."""

    def __init__(self, lang_id: str = "en"):
        self.lang_id = lang_id

    def tokenize(self, text: str) -> str:
        text = re.sub(r"([.,!?;:()\"«»“”])", r" \1 ", text)
        text = re.sub(r"(\w)'(\w)", r"\1 '\2", text) if self.lang_id == "en" else text
        return re.sub(r"\s+", " ", text).strip()

    def detokenize(self, tokens: List[str]) -> str:
        s = " ".join(tokens)
        s = re.sub(r" ([.,!?;:)»”])", r"\1", s)
        s = re.sub(r"([(«“]) ", r"\1", s)
        return re.sub(r" '(\w)", r"'\1", s)

    def normalize(self, text: str) -> str:
        return text.replace("’", "'").replace("“", '"').replace("”", '"').strip()


class TiktokenTokenizer(TokenizerSpec):
    """Byte-pair encoding from a ranks file (JSON list of ``{"token_bytes": base64, "rank": n}``) through ``tiktoken``; special
    tokens occupy the first ``num_special_tokens`` ids."""

    def __init__(self, vocab_file: str, pattern: str = r"[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+", vocab_size: Optional[int] = None,
                 num_special_tokens: int = 1000, special_tokens: Optional[List[str]] = None):
        try:
            import tiktoken
        except ImportError as e:
            raise ImportError("TiktokenTokenizer needs the optional `tiktoken` package") from e
        import base64

        entries = json.load(open(vocab_file, encoding="utf-8"))
        if vocab_size is not None:
            entries = entries[: vocab_size - num_special_tokens]
        specials = list(special_tokens or ["<unk>", "<s>", "</s>"])
        specials += [f"<SPECIAL_{i}>" for i in range(len(specials), num_special_tokens)]
        self.special = {t: i for i, t in enumerate(specials)}
        ranks = {base64.b64decode(e["token_bytes"]): e["rank"] for e in entries}
        self.enc = tiktoken.Encoding(name="speech_b200", pat_str=pattern, mergeable_ranks=ranks, special_tokens={})
        self.shift, self._vocab_size = num_special_tokens, len(ranks) + num_special_tokens
        self.unk_id, self.bos_id, self.eos_id = 0, 1, 2

    vocab_size = property(lambda self: self._vocab_size)

    def text_to_ids(self, text):
        return [t + self.shift for t in self.enc.encode(text)]

    def ids_to_text(self, ids):
        return self.enc.decode([int(i) - self.shift for i in ids if int(i) >= self.shift])

    def text_to_tokens(self, text):
        return [self.enc.decode_single_token_bytes(t).decode("utf-8", errors="replace") for t in self.enc.encode(text)]

    def tokens_to_ids(self, tokens):
        return [self.special[t] if t in self.special else self.enc.encode_single_token(t.encode()) + self.shift for t in tokens]

    def ids_to_tokens(self, ids):
        inv = {v: k for k, v in self.special.items()}
        return [inv[int(i)] if int(i) < self.shift else self.enc.decode_single_token_bytes(int(i) - self.shift).decode("utf-8", errors="replace") for i in ids]

    def tokens_to_text(self, tokens):
        return "".join(tokens)


class ChatTemplateMixin:
    """``apply_chat_template(messages)``: turns ``[{"role": ..., "content": ...}]`` into the prompt string of a chat format and
    (optionally) token ids plus a mask of the assistant tokens, which is what supervised fine-tuning trains on."""

    TEMPLATES: Dict[str, Dict[str, str]] = {
        "chatml": {"turn": "<|im_start|>{role}\n{content}<|im_end|>\n", "gen": "<|im_start|>assistant\n"},
        "llama3": {"turn": "<|start_header_id|>{role}<|end_header_id|>\n\n{content}<|eot_id|>", "gen": "<|start_header_id|>assistant<|end_header_id|>\n\n",
                   "bos": "<|begin_of_text|>"},
        "plain": {"turn": "{role}: {content}\n", "gen": "assistant: "},
    }

    def apply_chat_template(self, messages: List[Dict[str, str]], template: str = "chatml", add_generation_prompt: bool = False,
                            tokenize: bool = False):
        t = self.TEMPLATES[template]
        pieces = [(None, t.get("bos", ""))] if t.get("bos") else []
        for m in messages:
            pieces.append((m["role"], t["turn"].format(role=m["role"], content=m["content"])))
        if add_generation_prompt:
            pieces.append((None, t["gen"]))
        text = "".join(p for _, p in pieces)
        if not tokenize:
            return text
        ids, mask = [], []
        for role, p in pieces:
            pid = list(self.text_to_ids(p))
            ids += pid
            mask += [role == "assistant"] * len(pid)
        return {"input_ids": ids, "assistant_mask": mask, "text": text}

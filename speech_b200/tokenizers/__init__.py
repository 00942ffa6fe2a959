"""Tokenizers: SentencePiece, character, byte-level, word-piece vocab, Hugging Face, aggregate and Canary.

Interfaces (``text_to_ids``, ``ids_to_text``, ``ids_to_tokens``, ``tokens_to_ids``, ``vocab_size``, ``vocab``)
follow ``nemo/collections/common/tokenizers/tokenizer_spec.py``.  ``AggregateTokenizer`` offsets the ids of
per-language tokenizers into one id space (``aggregate_tokenizer.py``); ``CanaryTokenizer`` adds the
``spl_tokens`` sub-tokenizer that holds the ``<|...|>`` prompt specials
(``canary_tokenizer.py:30-70``).
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, List, Optional, Union

__all__ = ["TokenizerSpec", "SentencePieceTokenizer", "CharTokenizer", "ByteLevelTokenizer", "WordPieceVocabTokenizer",
           "AutoTokenizer", "AggregateTokenizer", "CanaryTokenizer", "create_spt_model", "SyntheticTokenizer"]


class TokenizerSpec:
    def text_to_tokens(self, text: str) -> List[str]:
        raise NotImplementedError

    def tokens_to_text(self, tokens: List[str]) -> str:
        raise NotImplementedError

    def tokens_to_ids(self, tokens: List[str]) -> List[int]:
        raise NotImplementedError

    def ids_to_tokens(self, ids: List[int]) -> List[str]:
        raise NotImplementedError

    def text_to_ids(self, text: str) -> List[int]:
        raise NotImplementedError

    def ids_to_text(self, ids: List[int]) -> str:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    @property
    def name(self) -> str:
        return type(self).__name__


class SentencePieceTokenizer(TokenizerSpec):
    def __init__(self, model_path: str, special_tokens: Optional[Union[Dict[str, str], List[str]]] = None,
                 legacy: bool = False, **_):
        import sentencepiece

        if not model_path or not os.path.exists(model_path):
            raise ValueError(f"model_path: {model_path} is invalid")
        self.tokenizer = sentencepiece.SentencePieceProcessor()
        self.tokenizer.Load(model_path)
        self.original_vocab_size = self.tokenizer.get_piece_size()
        self._vocab_size = self.original_vocab_size
        self.legacy = legacy
        self.special_token_to_id: Dict[str, int] = {}
        self.id_to_special_token: Dict[int, str] = {}
        if special_tokens:
            if not legacy:
                raise ValueError("Special tokens must be None when legacy is set to False. Provide special tokens at "
                                 "train time.")
            self.add_special_tokens(special_tokens)
        self.vocab = [self.tokenizer.id_to_piece(i) for i in range(self.original_vocab_size)]

    def add_special_tokens(self, special_tokens):
        toks = special_tokens.values() if isinstance(special_tokens, dict) else special_tokens
        for t in toks:
            if self.tokenizer.piece_to_id(t) == self.tokenizer.unk_id() and t not in self.special_token_to_id:
                self.special_token_to_id[t] = self._vocab_size
                self.id_to_special_token[self._vocab_size] = t
                self._vocab_size += 1

    @property
    def vocab_size(self):
        return self._vocab_size

    def text_to_tokens(self, text):
        return self.tokenizer.encode_as_pieces(text)

    def text_to_ids(self, text, sample_alpha=None):
        if sample_alpha is not None:
            return self.tokenizer.encode(text, enable_sampling=True, alpha=sample_alpha, nbest_size=-1)
        return self.tokenizer.encode_as_ids(text)

    def tokens_to_text(self, tokens):
        return self.tokenizer.decode_pieces(tokens)

    def ids_to_text(self, ids):
        ids = [int(i) for i in ids]
        if not self.legacy:
            return self.tokenizer.decode_ids([i for i in ids if i < self.original_vocab_size])
        text, last = "", 0
        for i, idx in enumerate(ids):
            if idx in self.id_to_special_token:
                text += self.tokenizer.decode_ids(ids[last:i]) + " " + self.id_to_special_token[idx] + " "
                last = i + 1
        return (text + self.tokenizer.decode_ids(ids[last:])).strip()

    def token_to_id(self, token):
        return self.special_token_to_id.get(token, self.tokenizer.piece_to_id(token))

    def tokens_to_ids(self, tokens):
        return [self.token_to_id(t) for t in ([tokens] if isinstance(tokens, str) else tokens)]

    def ids_to_tokens(self, ids):
        return [self.id_to_special_token[i] if i in self.id_to_special_token else self.tokenizer.id_to_piece(int(i)) for i in ids]

    @property
    def pad_id(self):
        return self.tokenizer.pad_id()

    @property
    def bos_id(self):
        return self.tokenizer.bos_id()

    @property
    def eos_id(self):
        return self.tokenizer.eos_id()

    @property
    def unk_id(self):
        return self.tokenizer.unk_id()


def create_spt_model(data_file: str, vocab_size: int, sample_size: int = -1, do_lower_case: bool = True,
                     tokenizer_type: str = "unigram", output_dir: Optional[str] = None, character_coverage: float = 1.0,
                     user_defined_symbols: Optional[List[str]] = None, bos: bool = False, eos: bool = False,
                     pad: bool = False, **kw):
    """Train a SentencePiece model; returns (model_path, vocab_path)."""
    import sentencepiece

    output_dir = output_dir or f"{os.path.dirname(data_file)}/spt"
    os.makedirs(output_dir, exist_ok=True)
    prefix = os.path.join(output_dir, "tokenizer")
    cmd = (f"--input={data_file} --model_prefix={prefix} --vocab_size={vocab_size} --shuffle_input_sentence=true "
           f"--hard_vocab_limit=false --model_type={tokenizer_type} --character_coverage={character_coverage}")
    cmd += f" --bos_id={'1' if bos else '-1'} --eos_id={'2' if eos else '-1'} --pad_id={'3' if pad else '-1'}"
    if do_lower_case:
        cmd += " --normalization_rule_name=nmt_nfkc_cf"
    if sample_size > 0:
        cmd += f" --input_sentence_size={sample_size}"
    if user_defined_symbols:
        cmd += " --user_defined_symbols=" + ",".join(user_defined_symbols)
    sentencepiece.SentencePieceTrainer.Train(cmd)
    vocab_file = os.path.join(output_dir, "vocab.txt")
    with open(prefix + ".vocab") as f, open(vocab_file, "w") as g:
        for line in f:
            piece = line.split("\t")[0]
            if piece not in ("<unk>", "<s>", "</s>", "<pad>"):
                g.write(("##" + piece if not piece.startswith("▁") else piece[1:]) + "\n")
    return prefix + ".model", vocab_file


class CharTokenizer(TokenizerSpec):
    def __init__(self, vocab: Union[str, Iterable[str]], unk_token: Optional[str] = None, **_):
        if isinstance(vocab, str) and os.path.exists(vocab):
            with open(vocab, encoding="utf-8") as f:
                vocab = [l.rstrip("\n") for l in f if l.rstrip("\n") != ""]
        self.vocab = list(vocab)
        self.unk_token = unk_token
        if unk_token is not None and unk_token not in self.vocab:
            self.vocab.append(unk_token)
        self._t2i = {t: i for i, t in enumerate(self.vocab)}

    def text_to_tokens(self, text):
        return [c if c in self._t2i else self.unk_token for c in text if c in self._t2i or self.unk_token is not None]

    def tokens_to_ids(self, tokens):
        return [self._t2i[t] for t in tokens]

    def text_to_ids(self, text):
        return self.tokens_to_ids(self.text_to_tokens(text))

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids if 0 <= int(i) < len(self.vocab)]

    def ids_to_text(self, ids):
        return "".join(self.ids_to_tokens(ids))

    def tokens_to_text(self, tokens):
        return "".join(tokens)


class ByteLevelTokenizer(TokenizerSpec):
    def __init__(self, special_tokens: Optional[List[str]] = None, **_):
        self.vocab = [chr(i) for i in range(256)] + list(special_tokens or [])
        self._special = {t: 256 + i for i, t in enumerate(special_tokens or [])}

    @property
    def vocab_size(self):
        return len(self.vocab)

    def add_special_tokens(self, special_tokens) -> int:
        toks = special_tokens.get("additional_special_tokens", []) if isinstance(special_tokens, dict) else list(special_tokens)
        n = 0
        for t in toks:
            if t not in self._special:
                self._special[t] = len(self.vocab)
                self.vocab.append(t)
                n += 1
        return n

    def token_to_id(self, token):
        return self._special.get(token, ord(token) if len(token) == 1 and ord(token) < 256 else -1)

    def _special_id(self, name):
        return self._special.get(name, -1)

    @property
    def pad_id(self):
        return self._special_id("<pad>")

    @property
    def bos_id(self):
        return self._special_id("<s>")

    @property
    def eos_id(self):
        return self._special_id("</s>")

    def text_to_ids(self, text):
        """Special tokens that occur verbatim in the text map to their single id, everything else to UTF-8 bytes."""
        if not self._special:
            return list(text.encode("utf-8"))
        import re

        pat = "(" + "|".join(re.escape(t) for t in sorted(self._special, key=len, reverse=True)) + ")"
        out: List[int] = []
        for piece in re.split(pat, text):
            if piece in self._special:
                out.append(self._special[piece])
            elif piece:
                out.extend(piece.encode("utf-8"))
        return out

    def ids_to_text(self, ids):
        return bytes(int(i) for i in ids if int(i) < 256).decode("utf-8", errors="ignore")

    def text_to_tokens(self, text):
        return [self.vocab[i] for i in self.text_to_ids(text)]

    def tokens_to_ids(self, tokens):
        return [self._special.get(t, ord(t)) for t in tokens]

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids]

    def tokens_to_text(self, tokens):
        return self.ids_to_text(self.tokens_to_ids(tokens))


class WordPieceVocabTokenizer(TokenizerSpec):
    """Greedy longest-match word-piece tokenizer over a ``vocab.txt`` (``##`` continuation marks)."""

    def __init__(self, vocab_file: str, lower_case: bool = True, unk_token: str = "[UNK]", **_):
        with open(vocab_file, encoding="utf-8") as f:
            self.vocab = [l.rstrip("\n") for l in f]
        self._t2i = {t: i for i, t in enumerate(self.vocab)}
        self.lower_case, self.unk_token = lower_case, unk_token

    def text_to_tokens(self, text):
        out = []
        for word in (text.lower() if self.lower_case else text).split():
            start, pieces, bad = 0, [], False
            while start < len(word):
                end, cur = len(word), None
                while start < end:
                    sub = ("##" if start > 0 else "") + word[start:end]
                    if sub in self._t2i:
                        cur = sub
                        break
                    end -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(cur)
                start = end
            out.extend([self.unk_token] if bad else pieces)
        return out

    def tokens_to_ids(self, tokens):
        unk = self._t2i.get(self.unk_token, 0)
        return [self._t2i.get(t, unk) for t in tokens]

    def text_to_ids(self, text):
        return self.tokens_to_ids(self.text_to_tokens(text))

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids]

    def tokens_to_text(self, tokens):
        return " ".join(tokens).replace(" ##", "")

    def ids_to_text(self, ids):
        return self.tokens_to_text(self.ids_to_tokens(ids))


class AutoTokenizer(TokenizerSpec):
    """Hugging Face tokenizer behind the common interface (local files only in this build)."""

    def __init__(self, pretrained_model_name: str, use_fast: bool = True, additional_special_tokens=None, **kw):
        from transformers import AutoTokenizer as _HF

        self.tokenizer = _HF.from_pretrained(pretrained_model_name, use_fast=use_fast, local_files_only=True, **kw)
        if additional_special_tokens:
            self.tokenizer.add_special_tokens({"additional_special_tokens": list(additional_special_tokens)})

    @property
    def vocab(self):
        return [t for t, _ in sorted(self.tokenizer.get_vocab().items(), key=lambda kv: kv[1])]

    @property
    def vocab_size(self):
        return len(self.tokenizer)

    def text_to_tokens(self, text):
        return self.tokenizer.tokenize(text)

    def text_to_ids(self, text):
        return self.tokenizer.encode(text, add_special_tokens=False)

    def ids_to_text(self, ids):
        return self.tokenizer.decode([int(i) for i in ids], skip_special_tokens=True)

    def ids_to_tokens(self, ids):
        return self.tokenizer.convert_ids_to_tokens([int(i) for i in ids])

    def tokens_to_ids(self, tokens):
        return self.tokenizer.convert_tokens_to_ids(tokens)

    def tokens_to_text(self, tokens):
        return self.tokenizer.convert_tokens_to_string(tokens)

    def token_to_id(self, token):
        return self.tokenizer.convert_tokens_to_ids(token)

    @property
    def pad_id(self):
        return self.tokenizer.pad_token_id

    @property
    def bos_id(self):
        return self.tokenizer.bos_token_id

    @property
    def eos_id(self):
        return self.tokenizer.eos_token_id


class AggregateTokenizer(TokenizerSpec):
    def __init__(self, tokenizers: Dict[str, TokenizerSpec]):
        self.tokenizers_dict = tokenizers
        self.langs = list(tokenizers.keys())
        self.vocabulary: List[str] = []
        self.token_id_offset: Dict[str, int] = {}
        self.offset_token_ids_by_token_id: Dict[int, int] = {}
        self.tokenizers_by_token_id: Dict[int, TokenizerSpec] = {}
        self.langs_by_token_id: Dict[int, str] = {}
        off = 0
        for lang, tok in tokenizers.items():
            self.token_id_offset[lang] = off
            for i in range(tok.vocab_size):
                self.offset_token_ids_by_token_id[off + i] = i
                self.tokenizers_by_token_id[off + i] = tok
                self.langs_by_token_id[off + i] = lang
            self.vocabulary.extend(tok.vocab if hasattr(tok, "vocab") else [str(i) for i in range(tok.vocab_size)])
            off += tok.vocab_size
        self._vocab_size = off

    @property
    def vocab(self):
        return self.vocabulary

    @property
    def vocab_size(self):
        return self._vocab_size

    def text_to_tokens(self, text, lang_id):
        return self.tokenizers_dict[lang_id].text_to_tokens(text)

    def text_to_ids(self, text, lang_id):
        off = self.token_id_offset[lang_id]
        return [i + off for i in self.tokenizers_dict[lang_id].text_to_ids(text)]

    def ids_to_text(self, ids):
        out, cur_tok, cur_ids = [], None, []
        for i in ids:
            i = int(i)
            tok = self.tokenizers_by_token_id[i]
            if tok is not cur_tok and cur_ids:
                out.append(cur_tok.ids_to_text(cur_ids))
                cur_ids = []
            cur_tok = tok
            cur_ids.append(self.offset_token_ids_by_token_id[i])
        if cur_ids:
            out.append(cur_tok.ids_to_text(cur_ids))
        return " ".join(o for o in out if o != "") if len(out) > 1 else (out[0] if out else "")

    def ids_to_tokens(self, ids):
        return [self.tokenizers_by_token_id[int(i)].ids_to_tokens([self.offset_token_ids_by_token_id[int(i)]])[0] for i in ids]

    def ids_to_lang(self, ids):
        counts: Dict[str, int] = {}
        for i in ids:
            l = self.langs_by_token_id[int(i)]
            counts[l] = counts.get(l, 0) + 1
        return max(counts, key=counts.get) if counts else ""

    def ids_to_text_and_langs(self, ids):
        return [{"char": self.ids_to_tokens([i])[0], "lang": self.langs_by_token_id[int(i)]} for i in ids]

    def tokens_to_ids(self, tokens, langs):
        if isinstance(langs, str):
            langs = [langs] * len(tokens)
        return [self.tokenizers_dict[l].tokens_to_ids([t])[0] + self.token_id_offset[l] for t, l in zip(tokens, langs)]

    def token_to_id(self, token, lang_id):
        return self.tokenizers_dict[lang_id].tokens_to_ids([token])[0] + self.token_id_offset[lang_id]


CANARY_BOS = "<|startoftranscript|>"
CANARY_EOS = "<|endoftext|>"
CANARY_PAD = "<pad>"
CANARY_NOSPEECH = "<|nospeech|>"
CANARY_PNC = "<|pnc|>"
CANARY_NOPNC = "<|nopnc|>"
CANARY2_BOCTX = "<|startofcontext|>"
CANARY_SPECIAL_TOKENIZER = "spl_tokens"
DEFAULT_TOKENS = [CANARY_NOSPEECH, CANARY_PAD, CANARY_EOS, CANARY_BOS, CANARY_PNC, CANARY_NOPNC]


class CanaryTokenizer(AggregateTokenizer):
    def __init__(self, tokenizers: Dict[str, TokenizerSpec]):
        super().__init__(tokenizers)
        self.special_tokens: Dict[str, int] = {}
        if CANARY_SPECIAL_TOKENIZER in tokenizers:
            spl = tokenizers[CANARY_SPECIAL_TOKENIZER]
            off = self.token_id_offset[CANARY_SPECIAL_TOKENIZER]
            for i, tok in enumerate(spl.vocab):
                if tok.startswith("<|") or tok == CANARY_PAD:
                    self.special_tokens[tok] = i + off

    def spl_token_to_id(self, token):
        token = token if token.startswith("<") else f"<|{token}|>"
        if token not in self.special_tokens:
            raise KeyError(f"Token {token} not found in tokenizer.")
        return self.special_tokens[token]

    @property
    def eos_id(self):
        return self.special_tokens[CANARY_EOS]

    @property
    def bos_id(self):
        return self.special_tokens[CANARY_BOS]

    @property
    def nospeech_id(self):
        return self.special_tokens[CANARY_NOSPEECH]

    @property
    def pad_id(self):
        return self.special_tokens[CANARY_PAD]

    def text_to_ids(self, text, lang_id):
        if lang_id == CANARY_SPECIAL_TOKENIZER:
            return [self.spl_token_to_id(t) for t in _split_specials(text)]
        if text.endswith(CANARY_EOS):
            return super().text_to_ids(text[: -len(CANARY_EOS)], lang_id) + [self.eos_id]
        return super().text_to_ids(text, lang_id)

    @staticmethod
    def build_special_tokenizer(tokens: Iterable[str], model_dir: str, force_rebuild: bool = False) -> "CharTokenizer":
        """The special-token tokenizer is a plain lookup table stored as ``tokenizer.vocab`` in ``model_dir``."""
        os.makedirs(model_dir, exist_ok=True)
        path = os.path.join(model_dir, "tokenizer.vocab")
        toks = list(DEFAULT_TOKENS) + [t if t.startswith("<") else f"<|{t}|>" for t in tokens
                                       if (t if t.startswith("<") else f"<|{t}|>") not in DEFAULT_TOKENS]
        if force_rebuild or not os.path.exists(path):
            with open(path, "w", encoding="utf-8") as f:
                f.write("\n".join(toks) + "\n")
        return SpecialTokenTable(path)


class SpecialTokenTable(TokenizerSpec):
    def __init__(self, vocab_path_or_list):
        if isinstance(vocab_path_or_list, str):
            with open(vocab_path_or_list, encoding="utf-8") as f:
                self.vocab = [l.rstrip("\n") for l in f if l.strip()]
        else:
            self.vocab = list(vocab_path_or_list)
        self._t2i = {t: i for i, t in enumerate(self.vocab)}

    def text_to_tokens(self, text):
        return _split_specials(text)

    def tokens_to_ids(self, tokens):
        return [self._t2i[t] for t in tokens]

    def text_to_ids(self, text):
        return self.tokens_to_ids(self.text_to_tokens(text))

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids]

    def ids_to_text(self, ids):
        return "".join(self.ids_to_tokens(ids))


def _split_specials(text: str) -> List[str]:
    import re

    return re.findall(r"<\|[^|]*\|>|<pad>", text)


class SyntheticTokenizer(TokenizerSpec):
    """Id <-> pseudo-word table of a given size; lets models with a BPE head run on synthetic token ids."""

    def __init__(self, vocab_size: int):
        self.vocab = [f"▁w{i}" for i in range(vocab_size)]
        self.pad_id, self.bos_id, self.eos_id = 0, 1, 2          # the first three ids double as control tokens for decoders that need them

    def text_to_ids(self, text):
        return [int(w[1:]) for w in text.split() if w.startswith("w") and w[1:].isdigit()]

    def ids_to_text(self, ids):
        return " ".join(f"w{int(i)}" for i in ids if 0 <= int(i) < len(self.vocab))

    def ids_to_tokens(self, ids):
        return [self.vocab[int(i)] for i in ids if 0 <= int(i) < len(self.vocab)]

    def tokens_to_ids(self, tokens):
        return [int(t.lstrip("▁")[1:]) for t in tokens]

    def text_to_tokens(self, text):
        return ["▁" + w for w in text.split()]

    def tokens_to_text(self, tokens):
        return " ".join(t.lstrip("▁") for t in tokens)


def build_tokenizer(cfg) -> TokenizerSpec:
    """``cfg.type`` ∈ {bpe, spe, wpe, char, byte, hf, auto, synthetic}; mirrors the tokenizer block of model configs
    (``dir`` holding ``tokenizer.model`` / ``vocab.txt``, or ``model_path`` / ``pretrained_model_name``)."""
    import os

    get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
    kind = str(get("type", "bpe")).lower()
    if kind in ("bpe", "spe", "sentencepiece"):
        path = get("model_path", None) or os.path.join(get("dir"), "tokenizer.model")
        return SentencePieceTokenizer(path, special_tokens=get("special_tokens", None))
    if kind == "wpe":
        return WordPieceVocabTokenizer(get("vocab_file", None) or os.path.join(get("dir"), "vocab.txt"))
    if kind == "char":
        return CharTokenizer(get("vocab", None) or get("vocab_file"))
    if kind == "byte":
        return ByteLevelTokenizer(special_tokens=list(get("special_tokens", None) or []))
    if kind in ("hf", "auto", "huggingface"):
        return AutoTokenizer(get("pretrained_model_name", None) or get("dir"), use_fast=get("use_fast", True))
    if kind == "synthetic":
        return SyntheticTokenizer(int(get("vocab_size")))
    raise ValueError(f"unknown tokenizer type {kind}")

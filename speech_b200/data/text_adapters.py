"""Typed examples for text and conversation data, the iterable adapters that produce them, and a writer for tarred
conversation shards.  The adapters read through the data-type parsers of :mod:`speech_b200.data.sources` (so sharding, shuffling
and tar pairing behave the same as in the dataloader) and turn each cut into a typed example with prompt-format hooks and
length properties that token-based samplers use.
Reference: ``common/data/lhotse/text_adapters.py`` (``TextExample``, ``SourceTargetTextExample``, ``NeMoSFTExample``,
``NeMoMultimodalConversation`` with ``TextTurn`` / ``AudioTurn``, the JSONL / ShareGPT adapters, ``NeMoMultimodalConversationTarWriter``).
"""
from __future__ import annotations

import io
import json
import math
import os
import tarfile
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .audio_to_text import expand_sharded_filepaths
from .cuts import Cut

_PROMPT_FORMAT_FNS: Dict[type, Callable] = {}


def registered_prompt_format_fn(example_type: type):
    """Decorator: the function ``(example, prompt_formatter) -> dict of id tensors`` used for examples of this type."""
    def deco(fn):
        _PROMPT_FORMAT_FNS[example_type] = fn
        return fn
    return deco


def get_prompt_format_fn(example) -> Callable:
    for t in type(example).__mro__:
        if t in _PROMPT_FORMAT_FNS:
            return _PROMPT_FORMAT_FNS[t]
    raise KeyError(f"no prompt format function is registered for {type(example).__name__}")


class Formattable:
    """After ``apply_prompt_format`` the example carries ``input_ids`` (whole sequence), ``context_ids`` (the part the model is given),
    ``answer_ids`` (the part it must produce) and ``mask`` (True on trained positions); the length properties read them."""

    input_ids: Optional[torch.Tensor] = None
    context_ids: Optional[torch.Tensor] = None
    answer_ids: Optional[torch.Tensor] = None
    mask: Optional[torch.Tensor] = None

    @property
    def input_length(self) -> Optional[int]:
        return None if self.context_ids is None else int(len(self.context_ids))

    @property
    def output_length(self) -> Optional[int]:
        return None if self.answer_ids is None else int(len(self.answer_ids))

    @property
    def total_length(self) -> Optional[int]:
        return None if self.input_ids is None else int(len(self.input_ids))

    def apply_prompt_format(self, prompt, **kw) -> "Formattable":
        ans = get_prompt_format_fn(self)(self, prompt, **kw)
        self.input_ids, self.context_ids = ans["input_ids"], ans["context_ids"]
        self.answer_ids, self.mask = ans.get("answer_ids"), ans.get("mask")
        return self


def _ids(x) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(list(x), dtype=torch.long)


# ---------------------------------------------------------------------------------------------------------------- plain text
@dataclass
class TextExample(Formattable):
    text: str
    language: Optional[str] = None
    tokens: Optional[np.ndarray] = None
    custom: Dict[str, Any] = field(default_factory=dict)

    @property
    def num_tokens(self) -> Optional[int]:
        return None if self.tokens is None else len(self.tokens)

    def tokenize(self, tokenizer) -> "TextExample":
        self.tokens = np.asarray(_tok(tokenizer, self.text, self.language))
        return self


def _tok(tokenizer, text, lang=None):
    if lang is not None and hasattr(tokenizer, "langs"):
        return tokenizer.text_to_ids(text, lang)
    return tokenizer.text_to_ids(text) if hasattr(tokenizer, "text_to_ids") else tokenizer(text)


@registered_prompt_format_fn(TextExample)
def default_text_example_prompt_format_fn(example: TextExample, prompt, **_):
    """Language-model data: the whole text (plus end-of-sequence) is both input and answer."""
    tok = prompt.tokenizer if hasattr(prompt, "tokenizer") else prompt
    ids = list(_tok(tok, example.text, example.language))
    eos = getattr(tok, "eos_id", getattr(tok, "eos", None))
    if eos is not None and eos >= 0:
        ids = ids + [eos]
    t = _ids(ids)
    return {"input_ids": t, "context_ids": t[:0], "answer_ids": t, "mask": torch.ones(len(t), dtype=torch.bool)}


def _from_source(kind: str, entry: Dict[str, Any], seed: int = 0, rank: int = 0, world: int = 1):
    from .sources import get_parser

    return get_parser(kind)(entry, {"seed": seed, "rank": rank, "world": world})


@dataclass
class LhotseTextAdapter:
    """Lines of text files (optionally sharded ``_OP_..._CL_`` patterns; shards are shuffled with ``shuffle_shards``)."""

    paths: Union[str, Sequence[str]]
    language: Optional[str] = None
    shuffle_shards: bool = False
    shard_seed: Union[int, str] = "trng"

    def __iter__(self) -> Iterator[TextExample]:
        e = {"paths": self.paths, "language": self.language, "shuffle": self.shuffle_shards, "shard_seed": self.shard_seed}
        for c in _from_source("txt", e):
            yield TextExample(c.text, c.lang)


@dataclass
class LhotseTextJsonlAdapter:
    paths: Union[str, Sequence[str]]
    language: Optional[str] = None
    text_field: str = "text"
    shuffle_shards: bool = False
    shard_seed: Union[int, str] = "trng"

    def __iter__(self) -> Iterator[TextExample]:
        e = {"paths": self.paths, "language": self.language, "text_field": self.text_field, "shuffle": self.shuffle_shards, "shard_seed": self.shard_seed}
        for c in _from_source("txt_jsonl", e):
            yield TextExample(c.text, c.lang, custom={k: v for k, v in c.custom.items() if k != "kind"})


# --------------------------------------------------------------------------------------------------------------- text pairs
@dataclass
class SourceTargetTextExample(Formattable):
    source: TextExample
    target: TextExample
    question: Optional[TextExample] = None
    custom: Dict[str, Any] = field(default_factory=dict)

    def tokenize(self, tokenizer) -> "SourceTargetTextExample":
        self.source.tokenize(tokenizer)
        self.target.tokenize(tokenizer)
        if self.question is not None:
            self.question.tokenize(tokenizer)
        return self


@registered_prompt_format_fn(SourceTargetTextExample)
def default_src_tgt_prompt_format_fn(example: SourceTargetTextExample, prompt, **_):
    """The question (if any) and the source form the user turn, the target the assistant turn."""
    ctx = f"{example.question.text} {example.source.text}" if example.question is not None else example.source.text
    return _encode_turns(prompt, [{"role": "user", "slots": {"message": ctx}}, {"role": prompt.OUTPUT_ROLE, "slots": {"message": example.target.text}}])


def _encode_turns(prompt, turns) -> Dict[str, torch.Tensor]:
    out = prompt.encode_dialog(turns)
    return {k: _ids(v) if not isinstance(v, torch.Tensor) else v for k, v in out.items()}


@dataclass
class LhotseTextPairAdapter:
    source_paths: Union[str, Sequence[str]]
    target_paths: Union[str, Sequence[str]]
    source_language: Optional[str] = None
    target_language: Optional[str] = None
    questions_path: Optional[str] = None
    questions_language: Optional[str] = None
    shuffle_shards: bool = False
    shard_seed: Union[int, str] = "trng"

    def __post_init__(self):
        ns, nt = len(expand_sharded_filepaths(self.source_paths)), len(expand_sharded_filepaths(self.target_paths))
        if ns != nt:
            raise ValueError(f"{ns} source files but {nt} target files")

    def __iter__(self) -> Iterator[SourceTargetTextExample]:
        e = dict(source_paths=self.source_paths, target_paths=self.target_paths, source_language=self.source_language, target_language=self.target_language,
                 questions_path=self.questions_path, questions_language=self.questions_language, shuffle=self.shuffle_shards, shard_seed=self.shard_seed)
        for c in _from_source("txt_pair", e):
            p = c.custom
            q = TextExample(p["question"], p.get("question_language")) if p.get("question") else None
            yield SourceTargetTextExample(TextExample(p["source"], p.get("source_language")), TextExample(p["target"], p.get("target_language")), q)


# ---------------------------------------------------------------------------------------------------------------- SFT chats
@dataclass
class NeMoSFTExample(Formattable):
    """``data``: ``{"system": str, "mask": "User" | "Assistant" (the role that is NOT trained), "conversations": [{"from", "value"}]}``."""

    data: Dict[str, Any]
    language: Optional[str] = None
    metadata: Optional[Dict[str, Any]] = None
    custom: Dict[str, Any] = field(default_factory=dict)


@registered_prompt_format_fn(NeMoSFTExample)
def default_sft_prompt_format_fn(example: NeMoSFTExample, prompt, **_):
    masked = (example.data.get("mask") or "User").lower()
    turns = []
    if example.data.get("system"):
        turns.append({"role": "system", "slots": {"message": example.data["system"]}})
    for t in example.data["conversations"]:
        role = "user" if t["from"].lower() == masked else prompt.OUTPUT_ROLE
        turns.append({"role": role, "slots": {"message": t["value"]}})
    return _encode_turns(prompt, turns)


@dataclass
class NeMoSFTJsonlAdapter:
    paths: Union[str, Sequence[str]]
    language: Optional[str] = None
    shuffle_shards: bool = False
    shard_seed: Union[int, str] = "trng"

    def __iter__(self) -> Iterator[NeMoSFTExample]:
        e = {"paths": self.paths, "language": self.language, "shuffle": self.shuffle_shards, "shard_seed": self.shard_seed}
        for c in _from_source("nemo_sft_jsonl", e):
            conv = [{"from": t["role"].title(), "value": t["value"]} for t in c.custom["turns"]]
            yield NeMoSFTExample({"system": c.custom.get("system", ""), "mask": c.custom.get("mask", "user").title(), "conversations": conv}, self.language)


# ------------------------------------------------------------------------------------------------ multimodal conversations
@dataclass
class TextTurn:
    value: str
    role: str

    def to_dict(self):
        return {"type": "text", "from": self.role.title(), "value": self.value}


@dataclass
class AudioTurn:
    cut: Cut
    role: str
    audio_locator_tag: str = "<|audioplaceholder|>"
    text: Optional[str] = None

    def to_dict(self):
        c = self.cut
        val = c.audio if isinstance(c.audio, str) else f"{c.id}.wav"
        d = {"type": "audio", "from": self.role.title(), "duration": c.duration, "value": val}
        if c.offset:
            d["offset"] = c.offset
        if self.text is not None:
            d["text"] = self.text
        return d


@dataclass
class NeMoMultimodalConversation(Formattable):
    id: str
    turns: List[Union[TextTurn, AudioTurn]]
    token_equivalent_duration: Optional[float] = None
    custom: Dict[str, Any] = field(default_factory=dict)

    def _audio_tokens(self, which: str) -> int:
        if self.token_equivalent_duration is None:
            raise ValueError("token_equivalent_duration must be set to count the tokens of audio turns")
        out_role = self.custom.get("output_role", "assistant")
        turns = [t for t in self.turns if isinstance(t, AudioTurn) and (which == "all" or (t.role == out_role) == (which == "answer"))]
        return sum(int(math.ceil(t.cut.duration / self.token_equivalent_duration)) - 1 for t in turns)     # the placeholder token is already counted once

    @property
    def input_length(self) -> Optional[int]:
        n = Formattable.input_length.fget(self)
        return None if n is None else n + self._audio_tokens("context")

    @property
    def output_length(self) -> Optional[int]:
        n = Formattable.output_length.fget(self)
        return None if n is None else n + self._audio_tokens("answer")

    @property
    def total_length(self) -> Optional[int]:
        n = Formattable.total_length.fget(self)
        return None if n is None else n + self._audio_tokens("all")

    @property
    def has_audio_turns(self) -> bool:
        return any(isinstance(t, AudioTurn) for t in self.turns)

    @property
    def has_text_turns(self) -> bool:
        return any(isinstance(t, TextTurn) for t in self.turns)

    @property
    def is_text_only(self) -> bool:
        return not self.has_audio_turns

    def list_cuts(self) -> List[Cut]:
        return [t.cut for t in self.turns if isinstance(t, AudioTurn)]

    def to_dict(self):
        d = {"id": self.id, "conversations": [t.to_dict() for t in self.turns]}
        if self.custom:
            d["custom"] = {k: v for k, v in self.custom.items() if isinstance(v, (str, int, float, bool, list, dict, type(None)))}
        return d

    @staticmethod
    def from_cut(cut: Cut, audio_locator_tag: str = "<|audioplaceholder|>") -> "NeMoMultimodalConversation":
        turns: List[Union[TextTurn, AudioTurn]] = []
        for k, t in enumerate(cut.custom["turns"]):
            if t["type"] == "audio":
                src = t["audio"] if t.get("audio") is not None else t["value"]
                cid = os.path.splitext(os.path.basename(t["value"]))[0] if isinstance(t["value"], str) else f"{cut.id}_turn{k}"
                turns.append(AudioTurn(Cut(cid, src, float(t.get("duration") or 0.0), float(t.get("offset") or 0.0)), t["role"], audio_locator_tag, t.get("text")))
            else:
                turns.append(TextTurn(t["value"], t["role"]))
        extra = {k: v for k, v in cut.custom.items() if k not in ("kind", "turns", "conversation", "token_equivalent_duration")}
        return NeMoMultimodalConversation(cut.id, turns, cut.custom.get("token_equivalent_duration"), extra)


@registered_prompt_format_fn(NeMoMultimodalConversation)
def default_multimodal_conversation_prompt_format_fn(example: NeMoMultimodalConversation, prompt, **_):
    """Consecutive turns of one role merge into one message; an audio turn contributes its locator tag."""
    merged: List[Tuple[str, List[str]]] = []
    for t in example.turns:
        piece = t.value if isinstance(t, TextTurn) else t.audio_locator_tag
        role = t.role if t.role in ("system", "user") else prompt.OUTPUT_ROLE if t.role == "assistant" else t.role
        if merged and merged[-1][0] == role:
            merged[-1][1].append(piece)
        else:
            merged.append((role, [piece]))
    if hasattr(prompt, "OUTPUT_ROLE"):
        example.custom.setdefault("output_role", "assistant")
    return _encode_turns(prompt, [{"role": r, "slots": {"message": " ".join(p)}} for r, p in merged])


def collate_conversation_audio_fault_tolerant(conversations: Sequence[NeMoMultimodalConversation], sample_rate: int = 16000):
    """Load and pad the audio of every audio turn: ``(audio [N, T], lengths [N], kept conversations)``.  A conversation with an
    unreadable audio turn is dropped as a whole (with a warning) and the rest of the batch goes on."""
    from ..utils.logging import logging

    audios, kept = [], []
    for conv in conversations:
        try:
            xs = [torch.from_numpy(np.ascontiguousarray(c.load_audio(sample_rate))) for c in conv.list_cuts()]
        except Exception as ex:                                         # unreadable file, missing tar member, bad header
            logging.warning("conversation %s skipped: %s", conv.id, ex)
            continue
        audios.extend(xs)
        kept.append(conv)
    if not audios:
        return torch.zeros(0, 0), torch.zeros(0, dtype=torch.long), kept
    lens = torch.tensor([len(x) for x in audios])
    out = torch.zeros(len(audios), int(lens.max()))
    for k, x in enumerate(audios):
        out[k, :len(x)] = x
    return out, lens, kept


@dataclass
class NeMoMultimodalConversationJsonlAdapter:
    """Conversations from JSONL manifests, optionally with tar shards that hold the audio (manifest shard k pairs with tar k)."""

    manifest_filepath: Union[str, Sequence[str]]
    audio_locator_tag: str = "<|audioplaceholder|>"
    tarred_audio_filepaths: Union[str, Sequence[str], None] = None
    token_equivalent_duration: Optional[float] = None
    shuffle_shards: bool = False
    shard_seed: Union[int, str] = "trng"
    system_prompt: Optional[str] = None
    context: Optional[str] = None
    slice_length: Optional[float] = None
    audio_root: Optional[str] = None
    kind: str = "multimodal_conversation"
    extra: Dict[str, Any] = field(default_factory=dict)

    def _entry(self) -> Dict[str, Any]:
        tags = {k: v for k, v in (("system_prompt", self.system_prompt), ("context", self.context)) if v}
        return dict(manifest_filepath=self.manifest_filepath, tarred_audio_filepaths=self.tarred_audio_filepaths, shuffle=self.shuffle_shards,
                    shard_seed=self.shard_seed, token_equivalent_duration=self.token_equivalent_duration, slice_length=self.slice_length,
                    audio_root=self.audio_root, tags=tags, **self.extra)

    def __iter__(self) -> Iterator[NeMoMultimodalConversation]:
        for c in _from_source(self.kind, self._entry()):
            yield NeMoMultimodalConversation.from_cut(c, self.audio_locator_tag)


@dataclass
class NeMoMultimodalConversationShareGPTJsonlAdapter(NeMoMultimodalConversationJsonlAdapter):
    """ShareGPT records (``conversations: [{from: human|gpt, value}]`` with ``<sound>`` / ``<speech>`` placeholders and a ``sound`` path)."""

    audio_placeholders: Union[str, Sequence[str], None] = None
    kind: str = "share_gpt"

    def _entry(self):
        e = super()._entry()
        if self.audio_placeholders:
            e["audio_placeholders"] = [self.audio_placeholders] if isinstance(self.audio_placeholders, str) else list(self.audio_placeholders)
        return e


class TarIterator:
    """``(member name, bytes)`` pairs of a tar archive in stored order."""

    def __init__(self, source: str):
        self.source = source

    def __iter__(self):
        with tarfile.open(self.source) as tf:
            for m in tf:
                if m.isfile():
                    yield m.name, tf.extractfile(m).read()


@dataclass
class NeMoMultimodalConversationShareGPTWebdatasetAdapter:
    """WebDataset-style shards: every sample is a ``<key>.json`` ShareGPT record followed by its ``<key>.<audio ext>`` member."""

    data_dir: Union[str, Sequence[str]]
    audio_locator_tag: str = "<|audioplaceholder|>"
    audio_placeholders: Union[str, Sequence[str], None] = None
    token_equivalent_duration: Optional[float] = None
    shuffle_shards: bool = False
    shard_seed: int = 0

    def _shards(self) -> List[str]:
        if isinstance(self.data_dir, str) and os.path.isdir(self.data_dir):
            return sorted(os.path.join(self.data_dir, f) for f in os.listdir(self.data_dir) if f.endswith(".tar"))
        return list(expand_sharded_filepaths(self.data_dir))

    def __iter__(self) -> Iterator[NeMoMultimodalConversation]:
        import random

        from .audio_to_text import load_audio
        from .sources import sharegpt_turns

        shards = self._shards()
        if self.shuffle_shards:
            random.Random(self.shard_seed).shuffle(shards)
        ph = [self.audio_placeholders] if isinstance(self.audio_placeholders, str) else list(self.audio_placeholders or ("<sound>", "<speech>"))
        for s in shards:
            pending: Optional[Tuple[str, Dict[str, Any]]] = None
            for name, data in TarIterator(s):
                stem, ext = os.path.splitext(os.path.basename(name))
                if ext == ".json":
                    if pending is not None:                                   # a text-only record (no audio member followed)
                        yield self._make(pending[0], pending[1], None, ph)
                    pending = (stem, json.loads(data))
                elif pending is not None and stem == pending[0]:
                    x = np.asarray(load_audio(io.BytesIO(data)), dtype=np.float32)
                    yield self._make(stem, pending[1], x, ph, name)
                    pending = None
            if pending is not None:
                yield self._make(pending[0], pending[1], None, ph)

    def _make(self, key, rec, audio, ph, name=None):
        from .sources import sharegpt_turns

        turns = sharegpt_turns(rec, ph, audio_fallback=name)
        out: List[Union[TextTurn, AudioTurn]] = []
        for t in turns:
            if t["type"] == "audio":
                if audio is None:
                    raise ValueError(f"record {key} refers to audio but its shard holds none for it")
                out.append(AudioTurn(Cut(key, audio, len(audio) / 16000.0), t["role"], self.audio_locator_tag))
            else:
                out.append(TextTurn(t["value"], t["role"]))
        return NeMoMultimodalConversation(rec.get("id", key), out, self.token_equivalent_duration)


class NeMoMultimodalConversationTarWriter:
    """Writes conversations as shards ``manifest_<k>.jsonl`` + ``audio_<k>.tar`` of at most ``shard_size`` conversations; the audio of
    every audio turn is stored as 16-bit WAV named ``<cut id>.wav`` in the order the manifest uses it (offsets are resolved: the stored
    clip is the turn's segment).  Use as a context manager or call ``close()``."""

    def __init__(self, output_dir: str, shard_size: int = 100, sample_rate: int = 16000):
        self.output_dir, self.shard_size, self.sample_rate = output_dir, int(shard_size), sample_rate
        os.makedirs(output_dir, exist_ok=True)
        self.shard, self.count, self.total = 0, 0, 0
        self._man = self._tar = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _open(self):
        self._man = open(os.path.join(self.output_dir, f"manifest_{self.shard}.jsonl"), "w", encoding="utf-8")
        self._tar = tarfile.open(os.path.join(self.output_dir, f"audio_{self.shard}.tar"), "w")

    def close(self):
        if self._man is not None:
            self._man.close()
            self._tar.close()
            self._man = self._tar = None

    def write(self, example: NeMoMultimodalConversation):
        import wave

        if self._man is None:
            self._open()
        elif self.count == self.shard_size:
            self.close()
            self.shard, self.count = self.shard + 1, 0
            self._open()
        rec = example.to_dict()
        k = 0
        for t, d in zip(example.turns, rec["conversations"]):
            if not isinstance(t, AudioTurn):
                continue
            x = np.asarray(t.cut.load_audio(self.sample_rate), dtype=np.float32)
            name = f"{t.cut.id}.wav" if k == 0 or not any(o.get("value") == f"{t.cut.id}.wav" for o in rec["conversations"][:rec["conversations"].index(d)]) else f"{t.cut.id}_{k}.wav"
            buf = io.BytesIO()
            with wave.open(buf, "wb") as w:
                w.setnchannels(1); w.setsampwidth(2); w.setframerate(self.sample_rate)
                w.writeframes((np.clip(x, -1.0, 1.0) * 32767.0).astype("<i2").tobytes())
            info = tarfile.TarInfo(name)
            info.size = buf.tell()
            buf.seek(0)
            self._tar.addfile(info, buf)
            d["value"], d["duration"] = name, len(x) / self.sample_rate
            d.pop("offset", None)
            k += 1
        self._man.write(json.dumps(rec, ensure_ascii=False) + "\n")
        self.count += 1
        self.total += 1

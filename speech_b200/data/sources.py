"""Input-source readers of the cut pipeline, selected by the ``type`` key of an ``input_cfg`` entry.

Every reader is registered under one or more type names with :func:`data_type_parser` (the reference keeps the same
registry, ``common/data/lhotse/cutset.py:153-209``) and maps an entry ``{type, ...}`` to a lazy :class:`CutSet`.  User code
can register further formats the same way.  Readers built here:

===========================  ==================================================================================
``nemo`` / ``nemo_tarred``    JSON-lines manifests, optionally with tar shards of audio (``cutset.py:1452``)
``lhotse``                    a Lhotse cut manifest, ``.jsonl`` or ``.jsonl.gz`` (``cutset.py:621``)
``lhotse_shar``               Lhotse Shar: ``cuts.NNNNNN.jsonl.gz`` + ``recording.NNNNNN.tar`` shards read in lockstep
``parquet``                   rows with ``audio`` bytes / ``text`` / ``duration`` columns (``cutset.py:722``)
``txt`` / ``txt_jsonl``       one text example per line / per JSON object (``text_adapters.py:109,135``)
``txt_pair``                  parallel source / target files, optional question pool (``text_adapters.py:201``)
``nemo_sft_jsonl``            chat SFT records (``text_adapters.py:299``)
``multimodal_conversation``   turns of text and audio, audio next to the manifest or in tar shards (``:599``)
``share_gpt``                 ShareGPT records with ``<sound>`` / ``<speech>`` placeholders (``:848``)
``lhotse_as_conversation``    audio cuts wrapped as (audio question, text answer) conversations (``cutset.py:1145``)
``nemo_tarred_to_duplex``     single-supervision cuts as two-channel user/agent cuts (``cutset.py:1721``)
``group``                     a nested ``input_cfg`` muxed by weight
===========================  ==================================================================================

Text-only examples are cuts without audio (``audio=None``, ``duration=0``) whose payload sits in ``custom``: ``kind`` is
one of ``text`` / ``text_pair`` / ``sft`` / ``conversation``.  :func:`measure_tokens` gives input / output / total token
counts of any example for the multimodal sampling constraints.
"""
from __future__ import annotations

import gzip
import io
import json
import os
import random
import tarfile
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Union

import numpy as np

from .audio_to_text import expand_sharded_filepaths, load_audio

_PARSERS: Dict[str, Callable] = {}


def data_type_parser(names: Union[str, Sequence[str]]):
    """Decorator: register ``fn(entry: dict, ctx: dict) -> CutSet`` as the reader of the given ``type`` names."""
    names = [names] if isinstance(names, str) else list(names)

    def deco(fn):
        for n in names:
            _PARSERS[n] = fn
        return fn
    return deco


def known_data_types() -> List[str]:
    return sorted(_PARSERS)


def get_parser(name: str) -> Callable:
    if name not in _PARSERS:
        raise ValueError(f"unsupported input_cfg type '{name}'; known types: {known_data_types()}")
    return _PARSERS[name]


def _seed(shard_seed, fallback: int = 0) -> int:
    if isinstance(shard_seed, int):
        return shard_seed
    if shard_seed == "randomized":
        return int.from_bytes(os.urandom(4), "little")
    return fallback          # "trng" resolves to the loader's base seed so that ranks differ only by the shard split


def _open_text(path: str):
    return gzip.open(path, "rt", encoding="utf-8") if str(path).endswith(".gz") else open(path, encoding="utf-8")


def _jsonl(path: str) -> Iterator[Dict[str, Any]]:
    with _open_text(path) as f:
        for line in f:
            line = line.strip()
            if line:
                yield json.loads(line)


def _shards(paths, entry, ctx) -> List[str]:
    ps = list(expand_sharded_filepaths(paths))
    if entry.get("shuffle", entry.get("shuffle_shards", False)):
        random.Random(_seed(entry.get("shard_seed", "trng"), ctx.get("seed", 0))).shuffle(ps)
    return ps


def _maybe_repeat(cs, entry):
    """Text sources repeat for ever unless ``force_finite`` (audio decides the epoch length in a mixed mux)."""
    from .cuts import CutSet

    if entry.get("force_finite", True):
        return cs

    def gen():
        while True:
            n = 0
            for c in cs:
                n += 1
                yield c
            if n == 0:
                return
    return CutSet(gen)


# ------------------------------------------------------------------------------------------ audio manifests
@data_type_parser(["nemo"])
def _read_nemo(e, ctx):
    from .cuts import read_nemo_manifest

    return read_nemo_manifest(e["manifest_filepath"], e.get("lang_field", "lang"), e.get("text_field", "text"), tags=e.get("tags"))


@data_type_parser(["nemo_tarred"])
def _read_nemo_tarred(e, ctx):
    from .cuts import read_nemo_tarred

    return read_nemo_tarred(e["manifest_filepath"], e["tarred_audio_filepaths"], e.get("tags"), ctx.get("rank", 0), ctx.get("world", 1))


def _cut_from_lhotse_dict(d: Dict[str, Any], base_dir: str, tags, audio=None):
    """One Lhotse ``MonoCut`` dict -> Cut.  Text / language come from the supervisions (joined in time order)."""
    from .cuts import Cut

    sups = sorted(d.get("supervisions", []), key=lambda s: s.get("start", 0.0))
    text = " ".join(s.get("text", "") for s in sups if s.get("text")).strip()
    lang = next((s.get("language") for s in sups if s.get("language")), None)
    rec = d.get("recording") or {}
    sr = int(rec.get("sampling_rate", 16000))
    if audio is None:
        src = (rec.get("sources") or [{}])[0]
        audio = src.get("source")
        if audio and src.get("type", "file") == "file" and not os.path.isabs(audio) and not os.path.exists(audio):
            audio = os.path.join(base_dir, audio)
    custom = dict(d.get("custom") or {})
    if sups:
        custom.setdefault("speaker", sups[0].get("speaker"))
        custom["supervisions"] = [{k: s.get(k) for k in ("start", "duration", "text", "speaker", "language")} for s in sups]
    custom.update(tags or {})
    return Cut(d["id"], audio, float(d.get("duration", 0.0)), float(d.get("start", 0.0)), text, lang, sr, custom)


@data_type_parser(["lhotse"])
def _read_lhotse(e, ctx):
    """``cuts_path``: a cut manifest.  With ``shar_path`` the entry is a Shar directory (see ``lhotse_shar``)."""
    from .cuts import CutSet

    if e.get("shar_path") is not None:
        return _read_lhotse_shar(e, ctx)
    paths = _shards(e["cuts_path"], e, ctx)

    def gen():
        for p in paths:
            base = os.path.dirname(os.path.abspath(p))
            for d in _jsonl(p):
                yield _cut_from_lhotse_dict(d, base, e.get("tags"))
    return CutSet(gen)


def _shar_fields(shar_path) -> Dict[str, List[str]]:
    """``shar_path`` is a directory, or a dict ``{field: [paths]}`` with at least ``cuts`` (and usually ``recording``)."""
    if isinstance(shar_path, dict):
        return {k: list(expand_sharded_filepaths(v)) for k, v in shar_path.items()}
    fields: Dict[str, List[str]] = {}
    for d in ([shar_path] if isinstance(shar_path, str) else list(shar_path)):
        for name in sorted(os.listdir(d)):
            fields.setdefault(name.split(".")[0], []).append(os.path.join(d, name))
    return fields


@data_type_parser(["lhotse_shar"])
def _read_lhotse_shar(e, ctx):
    """Lhotse Shar: shard ``k`` is ``cuts.k.jsonl.gz`` plus one tar per data field (``recording.k.tar``) whose members come
    in cut order as ``<cut_id>.<ext>`` (audio) and ``<cut_id>.json`` (its manifest); both files are streamed once, in
    lockstep, so a shard is read sequentially.  Shards are split over ranks."""
    from .cuts import CutSet

    fields = _shar_fields(e["shar_path"])
    if "cuts" not in fields:
        raise ValueError("a Shar source needs cuts.*.jsonl(.gz) shards")
    n = len(fields["cuts"])
    order = list(range(n))
    if e.get("shuffle", e.get("shuffle_shards", False)):
        random.Random(_seed(e.get("shard_seed", "trng"), ctx.get("seed", 0))).shuffle(order)
    order = order[ctx.get("rank", 0)::ctx.get("world", 1)] if n >= ctx.get("world", 1) else order
    recs = fields.get("recording")
    if recs is not None and len(recs) != n:
        raise ValueError(f"{len(recs)} recording shards for {n} cut shards")

    def gen():
        for k in order:
            base = os.path.dirname(os.path.abspath(fields["cuts"][k]))
            tf = tarfile.open(recs[k]) if recs is not None else None
            members = iter(tf) if tf is not None else None
            try:
                for d in _jsonl(fields["cuts"][k]):
                    audio = None
                    if members is not None:
                        data, seen_json = None, False
                        for m in members:                     # the members of one cut are adjacent: its audio and its .json
                            stem, ext = os.path.splitext(os.path.basename(m.name))
                            if stem != d["id"]:
                                raise ValueError(f"Shar shard {recs[k]}: member '{m.name}' where cut '{d['id']}' was expected")
                            if ext == ".json":
                                seen_json = True
                            else:
                                data = tf.extractfile(m).read()
                            if seen_json and data is not None:
                                break
                        if data is not None:
                            sr = int((d.get("recording") or {}).get("sampling_rate", 16000))
                            audio = np.asarray(load_audio(io.BytesIO(data), target_sr=sr), dtype=np.float32)
                            # the stored clip already starts at the cut's start
                            d = {**d, "start": 0.0}
                    yield _cut_from_lhotse_dict(d, base, e.get("tags"), audio=audio)
            finally:
                if tf is not None:
                    tf.close()
    return CutSet(gen)


@data_type_parser(["parquet"])
def _read_parquet(e, ctx):
    """Rows of ``.parquet`` files: ``audio`` (encoded bytes, or a struct with ``bytes``) or ``audio_filepath``, ``text``,
    ``duration``, optional ``lang`` / ``id``; other columns land in ``custom``.  Files are split over ranks."""
    import pyarrow.parquet as pq

    from .cuts import Cut, CutSet

    paths = _shards(e["manifest_filepath"], e, ctx)
    paths = paths[ctx.get("rank", 0)::ctx.get("world", 1)] if len(paths) >= ctx.get("world", 1) else paths
    audio_col, text_col = e.get("audio_field", "audio"), e.get("text_field", "text")

    def gen():
        for p in paths:
            pf = pq.ParquetFile(p)
            k = 0
            for rg in range(pf.num_row_groups):
                for row in pf.read_row_group(rg).to_pylist():
                    a = row.get(audio_col)
                    if isinstance(a, dict):
                        a = a.get("bytes") or a.get("path")
                    if isinstance(a, (bytes, bytearray)):
                        x = np.asarray(load_audio(io.BytesIO(a)), dtype=np.float32)
                        dur = float(row.get("duration") or len(x) / 16000.0)
                        audio = x
                    else:
                        audio, dur = a or row.get("audio_filepath"), float(row.get("duration") or 0.0)
                    custom = {c: v for c, v in row.items() if c not in (audio_col, text_col, "duration", "lang", "id", "audio_filepath")}
                    custom.update(e.get("tags") or {})
                    yield Cut(str(row.get("id", f"{os.path.basename(p)}-{k}")), audio, dur, 0.0, row.get(text_col) or "", row.get("lang"),
                              custom=custom)
                    k += 1
    return CutSet(gen)


# ------------------------------------------------------------------------------------------ text sources
def _text_cut(cid, kind, payload, text="", lang=None, tags=None):
    from .cuts import Cut

    return Cut(cid, None, 0.0, text=text, lang=lang, custom={"kind": kind, **payload, **(tags or {})})


@data_type_parser(["txt"])
def _read_txt(e, ctx):
    from .cuts import CutSet

    paths = _shards(e.get("paths", e.get("source_paths")), e, ctx)

    def gen():
        for p in paths:
            with _open_text(p) as f:
                for k, line in enumerate(f):
                    if line.strip():
                        yield _text_cut(f"{os.path.basename(p)}-{k}", "text", {}, line.strip(), e.get("language"), e.get("tags"))
    return _maybe_repeat(CutSet(gen), e)


@data_type_parser(["txt_jsonl"])
def _read_txt_jsonl(e, ctx):
    from .cuts import CutSet

    paths = _shards(e["paths"], e, ctx)
    field = e.get("text_field", "text")

    def gen():
        for p in paths:
            for k, d in enumerate(_jsonl(p)):
                extra = {a: b for a, b in d.items() if a != field}
                yield _text_cut(f"{os.path.basename(p)}-{k}", "text", extra, d[field], e.get("language"), e.get("tags"))
    return _maybe_repeat(CutSet(gen), e)


@data_type_parser(["txt_pair"])
def _read_txt_pair(e, ctx):
    """Line ``k`` of a source file pairs with line ``k`` of the target file; with ``questions_path`` each pair also draws a
    random question (the instruction of a translation prompt)."""
    from .cuts import CutSet

    src, tgt = list(expand_sharded_filepaths(e["source_paths"])), list(expand_sharded_filepaths(e["target_paths"]))
    if len(src) != len(tgt):
        raise ValueError(f"{len(src)} source files but {len(tgt)} target files")
    seed = _seed(e.get("shard_seed", "trng"), ctx.get("seed", 0))

    def gen():
        rng = random.Random(seed)
        pairs = list(zip(src, tgt))
        if e.get("shuffle", False):
            rng.shuffle(pairs)
        questions = None
        if e.get("questions_path"):
            with _open_text(e["questions_path"]) as f:
                questions = [q.strip() for q in f if q.strip()]
        for ps, pt in pairs:
            with _open_text(ps) as fs, _open_text(pt) as ft:
                for k, (ls, lt) in enumerate(zip(fs, ft)):
                    payload = {"source": ls.strip(), "target": lt.strip(), "source_language": e.get("source_language"),
                               "target_language": e.get("target_language")}
                    if questions:
                        payload["question"] = rng.choice(questions)
                        payload["question_language"] = e.get("questions_language")
                    yield _text_cut(f"{os.path.basename(ps)}-{k}", "text_pair", payload, lt.strip(), e.get("target_language"), e.get("tags"))
    return _maybe_repeat(CutSet(gen), e)


@data_type_parser(["nemo_sft_jsonl"])
def _read_sft(e, ctx):
    from .cuts import CutSet

    paths = _shards(e["paths"], e, ctx)

    def gen():
        for p in paths:
            for k, d in enumerate(_jsonl(p)):
                turns = [{"role": t["from"].lower(), "type": "text", "value": t["value"]} for t in d["conversations"]]
                payload = {"turns": turns, "mask": (d.get("mask") or "User").lower(), "system": d.get("system", "")}
                yield _text_cut(d.get("id", f"{os.path.basename(p)}-{k}"), "sft", payload, lang=e.get("language"), tags=e.get("tags"))
    return _maybe_repeat(CutSet(gen), e)


# ------------------------------------------------------------------------------------------ conversations
def _conversation_cut(cid, turns, tags, token_equivalent_duration=None, system_prompt=None, context=None):
    """``turns``: ``{"role", "type": "text" | "audio", "value", "duration", "offset", "audio"?}``.  The cut's duration is the
    total audio duration, so duration-based samplers and filters see the audio cost of the conversation."""
    from .cuts import Cut

    if system_prompt and not (turns and turns[0]["role"] == "system"):
        turns = [{"role": "system", "type": "text", "value": system_prompt}] + turns
    if context:
        # a default instruction put in front of the first user audio turn that no text precedes
        for i, t in enumerate(turns):
            if t["type"] == "audio" and t["role"] == "user":
                if i == 0 or turns[i - 1]["type"] != "text" or turns[i - 1]["role"] != "user":
                    turns = turns[:i] + [{"role": "user", "type": "text", "value": context}] + turns[i:]
                break
    dur = sum(float(t.get("duration") or 0.0) for t in turns if t["type"] == "audio")
    custom = {"kind": "conversation", "turns": turns, "token_equivalent_duration": token_equivalent_duration, **(tags or {})}
    # the record the conversation dataset consumes (same keys as a manifest line)
    custom["conversation"] = {"id": cid, "conversations": [
        {"from": t["role"].title(), "type": t["type"], "value": t["value"],
         **({"duration": t.get("duration"), "offset": t.get("offset", 0.0)} if t["type"] == "audio" else {}),
         **({"audio": t["audio"]} if t.get("audio") is not None else {})} for t in turns]}
    return Cut(cid, None, dur, custom=custom)


def _resolve_audio(path: str, base: str, audio_root: Optional[str] = None) -> str:
    if audio_root and not os.path.isabs(path):
        return os.path.join(audio_root, path)
    if not os.path.isabs(path) and not os.path.exists(path):
        return os.path.join(base, path)
    return path


def _slice_turns(turns, slice_length: Optional[float], rng: random.Random):
    """``slice_length``: audio turns longer than this many seconds are cut to a random window of that length."""
    if not slice_length:
        return turns
    out = []
    for t in turns:
        if t["type"] == "audio" and t.get("duration") and t["duration"] > slice_length:
            off = rng.uniform(0.0, t["duration"] - slice_length)
            t = {**t, "offset": float(t.get("offset", 0.0)) + off, "duration": float(slice_length)}
        out.append(t)
    return out


def _iter_conversation_records(e, ctx, to_turns: Callable[[Dict[str, Any]], List[Dict[str, Any]]]):
    """Manifest-only, or manifest + tar shards: with tars, shard ``k`` of the manifest pairs with tar ``k`` and the audio
    members appear in the order in which the conversations use them, so each tar is streamed once."""
    mans = list(expand_sharded_filepaths(e["manifest_filepath"]))
    tars = list(expand_sharded_filepaths(e["tarred_audio_filepaths"])) if e.get("tarred_audio_filepaths") else None
    if tars is not None and len(tars) != len(mans):
        raise ValueError(f"{len(mans)} manifest shards but {len(tars)} tar shards")
    order = list(range(len(mans)))
    seed = _seed(e.get("shard_seed", "trng"), ctx.get("seed", 0))
    rng = random.Random(seed)
    if e.get("shuffle", False):
        rng.shuffle(order)
    if tars is not None and len(order) >= ctx.get("world", 1):
        order = order[ctx.get("rank", 0)::ctx.get("world", 1)]
    for k in order:
        base = os.path.dirname(os.path.abspath(mans[k]))
        tf = tarfile.open(tars[k]) if tars is not None else None
        members = iter(tf) if tf is not None else None
        try:
            for j, d in enumerate(_jsonl(mans[k])):
                if d.get("_skipme"):
                    continue
                turns = to_turns(d)
                for t in turns:
                    if t["type"] != "audio":
                        continue
                    if members is not None:
                        want = os.path.basename(t["value"])
                        m = next(members, None)
                        while m is not None and not m.isfile():
                            m = next(members, None)
                        if m is None or os.path.basename(m.name) != want:
                            raise ValueError(f"tar shard {tars[k]}: expected member '{want}', found '{m.name if m else None}'")
                        x = np.asarray(load_audio(io.BytesIO(tf.extractfile(m).read())), dtype=np.float32)
                        t["audio"] = x
                        t["duration"] = float(t.get("duration") or len(x) / 16000.0)
                    else:
                        t["value"] = _resolve_audio(t["value"], base, e.get("audio_root"))
                turns = _slice_turns(turns, e.get("slice_length"), rng)
                yield d.get("id", f"{os.path.basename(mans[k])}-{j}"), turns, d
        finally:
            if tf is not None:
                tf.close()


@data_type_parser(["multimodal_conversation"])
def _read_conversations(e, ctx):
    from .cuts import CutSet

    tags = e.get("tags") or {}

    def to_turns(d):
        return [{"role": t["from"].lower(), "type": t.get("type", "text"), "value": t["value"],
                 "duration": t.get("duration"), "offset": t.get("offset", 0.0)} for t in d["conversations"]]

    def gen():
        for cid, turns, d in _iter_conversation_records(e, ctx, to_turns):
            extra = {k: v for k, v in tags.items() if k not in ("system_prompt", "context")}
            yield _conversation_cut(cid, turns, extra, e.get("token_equivalent_duration"), tags.get("system_prompt"), tags.get("context"))
    return _maybe_repeat(CutSet(gen), e)


def sharegpt_turns(d: Dict[str, Any], placeholders: Sequence[str] = ("<sound>", "<speech>"), audio_fallback: Optional[str] = None):
    """ShareGPT record -> flat turns.  A placeholder inside a ``value`` splits it into text / audio / text; the audio file
    is the record's ``sound`` (or ``ori_sound``) field."""
    out = []
    audio = d.get("sound") or d.get("ori_sound") or audio_fallback
    for t in d["conversations"]:
        role = "user" if t["from"].lower() in ("human", "user") else "assistant"
        tag = next((p for p in placeholders if p in t["value"]), None)
        if tag is None:
            out.append({"role": role, "type": "text", "value": t["value"]})
            continue
        if not audio:
            raise ValueError(f"record {d.get('id', '?')}: '{tag}' in a turn but no 'sound' / 'ori_sound' field")
        head, _, tail = t["value"].partition(tag)
        if head.strip():
            out.append({"role": role, "type": "text", "value": head.strip()})
        out.append({"role": role, "type": "audio", "value": audio, "duration": t.get("duration", d.get("duration")), "offset": t.get("offset", 0.0)})
        if tail.strip():
            out.append({"role": role, "type": "text", "value": tail.strip()})
    return out


@data_type_parser(["share_gpt"])
def _read_share_gpt(e, ctx):
    from .cuts import CutSet

    ph = e.get("audio_placeholders")
    ph = ["<sound>", "<speech>"] if ph is None else ([ph] if isinstance(ph, str) else list(ph))

    def gen():
        for cid, turns, d in _iter_conversation_records(e, ctx, lambda d: sharegpt_turns(d, ph)):
            yield _conversation_cut(cid, turns, e.get("tags"), e.get("token_equivalent_duration"))
    return _maybe_repeat(CutSet(gen), e)


@data_type_parser(["lhotse_as_conversation", "nemo_as_conversation"])
def _read_audio_as_conversation(e, ctx):
    """Audio cuts of any audio source as two-turn conversations: user = [context text,] audio; assistant = transcript.  The
    context is the entry's ``tags.context`` (one string, or a list to draw from)."""
    from .cuts import CutSet

    inner_type = "nemo" if ("manifest_filepath" in e and "cuts_path" not in e and "shar_path" not in e) else "lhotse"
    if e.get("tarred_audio_filepaths"):
        inner_type = "nemo_tarred"
    inner = get_parser(inner_type)({**e, "tags": None}, ctx)
    tags = e.get("tags") or {}
    ctxs = tags.get("context")
    seed = _seed(e.get("shard_seed", "trng"), ctx.get("seed", 0))

    def gen():
        rng = random.Random(seed)
        for c in inner:
            turns = []
            if ctxs:
                turns.append({"role": "user", "type": "text", "value": ctxs if isinstance(ctxs, str) else rng.choice(list(ctxs))})
            a = {"role": "user", "type": "audio", "value": c.audio if isinstance(c.audio, str) else c.id, "duration": c.duration,
                 "offset": c.offset}
            if not isinstance(c.audio, str):
                a["audio"] = c.load_audio()
            turns += [a, {"role": "assistant", "type": "text", "value": c.text}]
            extra = {k: v for k, v in tags.items() if k not in ("system_prompt", "context")}
            yield _conversation_cut(c.id, turns, extra, e.get("token_equivalent_duration"), tags.get("system_prompt"))
    return CutSet(gen)


@data_type_parser(["nemo_tarred_to_duplex"])
def _read_tarred_to_duplex(e, ctx):
    """Single-utterance cuts as duplex training cuts: the audio is the user channel, the transcript an agent turn that
    starts when the user stops; ``custom['duplex_turns']`` lists ``(role, start, duration, text)``."""
    from .cuts import Cut, CutSet

    inner = get_parser("nemo_tarred" if e.get("tarred_audio_filepaths") else "nemo")(e, ctx)
    agent_dur = float(e.get("agent_turn_duration", 0.0))

    def gen():
        for c in inner:
            ad = agent_dur or max(0.4, 0.08 * max(1, len(c.text.split())) * 4)
            turns = [("user", 0.0, c.duration, ""), ("agent", c.duration, ad, c.text)]
            yield Cut(c.id, c.audio, c.duration + ad, c.offset, c.text, c.lang, c.sampling_rate,
                      {**c.custom, "duplex_turns": turns, "source_duration": c.duration})
    return CutSet(gen)


# ------------------------------------------------------------------------------------------ token measurement
def measure_tokens(cut, tokenizer=None, token_equivalent_duration: Optional[float] = None):
    """``(input_len, output_len)`` of an example in tokens.  Audio counts ``ceil(duration / token_equivalent_duration)``;
    text counts tokenizer ids (whitespace words without a tokenizer).  For conversations the last assistant turn is the
    output and everything before it the input; for text pairs source (+ question) is input and target output."""
    import math

    def ntok(s: str) -> int:
        if not s:
            return 0
        return len(tokenizer.text_to_ids(s)) if tokenizer is not None else len(s.split())

    ted = token_equivalent_duration or cut.custom.get("token_equivalent_duration") or 0.08
    kind = cut.custom.get("kind")
    if kind == "text":
        return ntok(cut.text), 0
    if kind == "text_pair":
        return ntok(cut.custom["source"]) + ntok(cut.custom.get("question", "")), ntok(cut.custom["target"])
    if kind in ("conversation", "sft"):
        turns = cut.custom["turns"]
        last = max((i for i, t in enumerate(turns) if t["role"] == "assistant"), default=len(turns))
        def tl(t):
            return math.ceil(float(t.get("duration") or 0.0) / ted) if t["type"] == "audio" else ntok(t["value"])
        return sum(tl(t) for t in turns[:last]), sum(tl(t) for t in turns[last:])
    return math.ceil(cut.duration / ted), ntok(cut.text)

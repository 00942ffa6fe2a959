"""Task-specific datasets over cuts: prompted transcripts for multitask encoder-decoder models, prompt indices for prompt-
conditioned transducers, speaker targets, end-of-utterance frame labels and diarization activity matrices.

All of them extend :class:`speech_b200.data.cuts.CutsSpeechToTextDataset` (audio loading, augmentation, tokenisation) and are
passed to ``get_dataloader_from_cuts_config(..., dataset_cls=...)``.  References: ``asr/data/audio_to_text_lhotse_prompted.py``
(``PromptedAudioToTextLhotseDataset`` / ``PromptedAudioToTextMiniBatch``), ``audio_to_text_lhotse_prompt_index.py``,
``audio_to_text_lhotse_speaker.py``, ``audio_to_eou_label_lhotse.py``, ``audio_to_diar_label_lhotse.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .cuts import Cut, CutsSpeechToTextDataset


def _pad_1d(seqs: Sequence[torch.Tensor], value) -> Tuple[torch.Tensor, torch.Tensor]:
    lens = torch.tensor([int(s.numel()) for s in seqs], dtype=torch.long)
    out = torch.full((len(seqs), max(1, int(lens.max()) if len(seqs) else 1)), value, dtype=seqs[0].dtype if seqs else torch.long)
    for i, s in enumerate(seqs):
        out[i, : s.numel()] = s
    return out, lens


# ------------------------------------------------------------------------------------------------ prompted (Canary)
@dataclass
class PromptedAudioToTextMiniBatch:
    audio: torch.Tensor
    audio_lens: torch.Tensor
    transcript: torch.Tensor
    transcript_lens: torch.Tensor
    prompt: torch.Tensor
    prompt_lens: torch.Tensor
    prompted_transcript: torch.Tensor
    prompted_transcript_lens: torch.Tensor
    cuts: Optional[List[Cut]] = None

    def get_decoder_inputs_outputs(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Teacher forcing: input is the prompted transcript without its last token, output the same without its first."""
        return self.prompted_transcript[:, :-1], self.prompted_transcript[:, 1:]

    def as_tuple(self):
        """The positional layout the multitask model's loss reads: audio, audio lengths, full decoder sequence and lengths,
        prompt, prompt lengths."""
        return (self.audio, self.audio_lens, self.prompted_transcript, self.prompted_transcript_lens, self.prompt, self.prompt_lens)


class PromptedAudioToTextCutsDataset(CutsSpeechToTextDataset):
    """Every cut becomes ``prompt tokens + transcript + end token`` under a prompt format (``canary``, ``canary2``, ...).

    Slot values come from the cut: ``source_lang`` / ``target_lang`` (default: the cut's language), ``taskname`` / ``task``
    (``asr`` unless the languages differ, then ``ast``), ``pnc``, and for ``canary2`` ``itn`` / ``timestamp`` / ``diarize`` /
    ``emotion`` / ``decodercontext``; ``prompt_defaults`` fills what a cut does not carry.  Cuts whose text is split over several
    supervisions use the joined text."""

    def __init__(self, cuts, tokenizer=None, prompt=None, prompt_defaults: Optional[Dict[str, Any]] = None, return_minibatch: bool = False, **kw):
        super().__init__(cuts, tokenizer=tokenizer, **kw)
        if prompt is None:
            raise ValueError("a prompt formatter is required (PromptFormatter.resolve(name)(tokenizer))")
        self.prompt, self.defaults, self.return_minibatch = prompt, dict(prompt_defaults or {}), return_minibatch
        pad = getattr(tokenizer, "pad_id", 0)
        self.pad_id = 0 if pad is None or pad < 0 else pad

    def slots_for(self, c: Cut) -> Dict[str, str]:
        cu = c.custom
        src = cu.get("source_lang") or c.lang or self.defaults.get("source_lang", "en")
        tgt = cu.get("target_lang") or self.defaults.get("target_lang") or src
        task = cu.get("taskname") or cu.get("task") or self.defaults.get("task") or ("asr" if src == tgt else "ast")
        vals = {"source_lang": src, "target_lang": tgt, "task": task, "taskname": task,
                "pnc": str(cu.get("pnc", self.defaults.get("pnc", "yes"))), "itn": str(cu.get("itn", self.defaults.get("itn", "no"))),
                "timestamp": str(cu.get("timestamp", self.defaults.get("timestamp", "no"))),
                "diarize": str(cu.get("diarize", self.defaults.get("diarize", "no"))),
                "emotion": str(cu.get("emotion", self.defaults.get("emotion", "undefined"))),
                "decodercontext": str(cu.get("decodercontext", self.defaults.get("decodercontext", ""))), "prompt_language": tgt}
        need = self.prompt.get_slots("user")
        return {k: v for k, v in vals.items() if k in need or k == "prompt_language"}

    def encode(self, c: Cut) -> Dict[str, torch.Tensor]:
        return self.prompt.encode_dialog([{"role": "user", "slots": self.slots_for(c)},
                                          {"role": self.prompt.OUTPUT_ROLE, "slots": {"text": c.text, "prompt_language": c.custom.get("target_lang") or c.lang}}])

    def num_tokens(self, idx: int) -> int:
        return int(self.encode(self.cuts[idx])["input_ids"].numel())

    def __getitem__(self, idx):
        c = self.cuts[idx]
        x = c.load_audio(self.sr)
        for a in self.aug:
            x = a(x)
        enc = self.encode(c)
        return {"audio": torch.as_tensor(x), "full": enc["input_ids"], "prompt": enc["context_ids"], "answer": enc["answer_ids"], "cut": c}

    def collate_fn(self, batch):
        alen = torch.tensor([b["audio"].numel() for b in batch], dtype=torch.long)
        audio = torch.zeros(len(batch), int(alen.max()))
        for i, b in enumerate(batch):
            audio[i, : alen[i]] = b["audio"]
        full, fl = _pad_1d([b["full"] for b in batch], self.pad_id)
        prm, pl = _pad_1d([b["prompt"] for b in batch], self.pad_id)
        ans, al = _pad_1d([b["answer"] for b in batch], self.pad_id)
        mb = PromptedAudioToTextMiniBatch(audio, alen, ans, al, prm, pl, full, fl, [b["cut"] for b in batch])
        return mb if self.return_minibatch else mb.as_tuple()


# ------------------------------------------------------------------------------------------------ prompt index
class PromptIndexCutsDataset(CutsSpeechToTextDataset):
    """For transducers conditioned on a prompt vector: besides audio and tokens, each item carries the index of its prompt
    (``prompt_field`` of the cut, e.g. the target language) in ``prompt_dictionary``; the collate adds a one-hot ``[B, P]``."""

    def __init__(self, cuts, tokenizer=None, prompt_dictionary: Optional[Dict[str, int]] = None, prompt_field: str = "target_lang",
                 num_prompts: Optional[int] = None, **kw):
        super().__init__(cuts, tokenizer=tokenizer, **kw)
        if not prompt_dictionary:
            raise ValueError("prompt_dictionary {value: index} is required")
        self.pd, self.field = dict(prompt_dictionary), prompt_field
        self.P = int(num_prompts or (max(self.pd.values()) + 1))

    def prompt_index(self, c: Cut) -> int:
        v = c.custom.get(self.field) or (c.lang if self.field in ("lang", "target_lang", "source_lang") else None)
        if v not in self.pd:
            raise KeyError(f"cut {c.id}: prompt value '{v}' (field '{self.field}') is not in the prompt dictionary")
        return self.pd[v]

    def __getitem__(self, idx):
        a, al, t, tl = super().__getitem__(idx)
        return a, al, t, tl, torch.tensor(self.prompt_index(self.cuts[idx]))

    def collate_fn(self, batch):
        from .audio_to_text import speech_collate

        A, al, T, tl = speech_collate([b[:4] for b in batch], pad_id=self.pad_id)
        idx = torch.stack([b[4] for b in batch])
        return A, al, T, tl, torch.nn.functional.one_hot(idx, self.P).float()


# ------------------------------------------------------------------------------------------------ speaker
class SpeakerCutsDataset(CutsSpeechToTextDataset):
    """Audio, tokens and the speaker id of each cut (``custom['speaker']`` mapped through ``speaker_to_id``; built from the cuts
    in sorted order when not given).  For speaker-aware recognition with several supervisions per cut, ``spk_targets`` gives the
    frame-level activity ``[T_frames, S]`` of up to ``max_speakers`` speakers in order of first appearance."""

    def __init__(self, cuts, tokenizer=None, speaker_to_id: Optional[Dict[str, int]] = None, frame_shift: float = 0.08, max_speakers: int = 4, **kw):
        super().__init__(cuts, tokenizer=tokenizer, **kw)
        spk = sorted({str(c.custom.get("speaker")) for c in self.cuts if c.custom.get("speaker") is not None})
        self.s2i = dict(speaker_to_id) if speaker_to_id else {s: i for i, s in enumerate(spk)}
        self.shift, self.S = frame_shift, max_speakers

    def activity(self, c: Cut) -> torch.Tensor:
        n = max(1, int(np.ceil(c.duration / self.shift)))
        out = torch.zeros(n, self.S)
        order: List[str] = []
        for s in sorted(c.custom.get("supervisions") or [], key=lambda s: s.get("start") or 0.0):
            name = str(s.get("speaker"))
            if name not in order:
                if len(order) == self.S:
                    continue
                order.append(name)
            a = int(round((s.get("start") or 0.0) / self.shift))
            b = int(round(((s.get("start") or 0.0) + (s.get("duration") or 0.0)) / self.shift))
            out[max(0, a):min(n, b), order.index(name)] = 1.0
        if not order:
            out[:, 0] = 1.0
        return out

    def __getitem__(self, idx):
        a, al, t, tl = super().__getitem__(idx)
        c = self.cuts[idx]
        sid = self.s2i.get(str(c.custom.get("speaker")), -1)
        return a, al, t, tl, torch.tensor(sid), self.activity(c)

    def collate_fn(self, batch):
        from .audio_to_text import speech_collate

        A, al, T, tl = speech_collate([b[:4] for b in batch], pad_id=self.pad_id)
        n = max(b[5].shape[0] for b in batch)
        act = torch.zeros(len(batch), n, self.S)
        for i, b in enumerate(batch):
            act[i, : b[5].shape[0]] = b[5]
        return A, al, T, tl, torch.stack([b[4] for b in batch]), act


# ------------------------------------------------------------------------------------------------ end of utterance
class EOUCutsDataset(CutsSpeechToTextDataset):
    """End-of-utterance training data.  Tokens get the ``<EOU>`` id appended (``<EOB>`` for back-channels, ``custom['is_backchannel']``)
    unless the cut says the utterance is cut short (``custom['eou_time']`` beyond the audio); frame labels ``[T_frames]`` are 0
    before speech, 1 during speech and 2 from the end of the utterance on (``sou_time`` / ``eou_time`` in seconds, default: the whole
    cut is speech).  Random silence of ``[pad_min, pad_max]`` seconds may be added on both sides so that the model sees the
    transition; labels are extended accordingly."""

    def __init__(self, cuts, tokenizer=None, eou_id: Optional[int] = None, eob_id: Optional[int] = None, frame_shift: float = 0.08,
                 pad_min: float = 0.0, pad_max: float = 0.0, seed: int = 0, **kw):
        super().__init__(cuts, tokenizer=tokenizer, **kw)
        v = getattr(tokenizer, "vocab_size", None)
        self.eou = int(eou_id) if eou_id is not None else (int(v) if v is not None else 0)
        self.eob = int(eob_id) if eob_id is not None else self.eou
        self.shift, self.pad = frame_shift, (pad_min, pad_max)
        self.rng = np.random.default_rng(seed)

    def __getitem__(self, idx):
        a, _, t, _ = super().__getitem__(idx)
        c = self.cuts[idx]
        sou = float(c.custom.get("sou_time", 0.0) or 0.0)
        eou = float(c.custom.get("eou_time", c.duration) or c.duration)
        lead = float(self.rng.uniform(*self.pad)) if self.pad[1] > 0 else 0.0
        tail = float(self.rng.uniform(*self.pad)) if self.pad[1] > 0 else 0.0
        if lead or tail:
            a = torch.cat([torch.zeros(int(lead * self.sr)), a, torch.zeros(int(tail * self.sr))])
        total = a.numel() / self.sr
        n = max(1, int(np.ceil(total / self.shift)))
        lab = torch.zeros(n, dtype=torch.long)
        s, e = int(round((lead + sou) / self.shift)), int(round((lead + eou) / self.shift))
        lab[max(0, s):min(n, e)] = 1
        complete = eou <= c.duration + 1e-6
        if complete:
            lab[min(n, e):] = 2
            t = torch.cat([t, torch.tensor([self.eob if c.custom.get("is_backchannel") else self.eou])])
        return a, torch.tensor(a.numel()), t, torch.tensor(t.numel()), lab

    def collate_fn(self, batch):
        from .audio_to_text import speech_collate

        A, al, T, tl = speech_collate([b[:4] for b in batch], pad_id=self.pad_id)
        lab, ll = _pad_1d([b[4] for b in batch], 0)
        return A, al, T, tl, lab, ll


# ------------------------------------------------------------------------------------------------ diarization
class DiarLabelCutsDataset(SpeakerCutsDataset):
    """End-to-end diarization: audio and the speaker-activity matrix ``[T_frames, S]`` (speakers in order of first appearance),
    no text.  ``frame_shift`` is the model's output frame period (0.08 s for 8x sub-sampled 10 ms features)."""

    def __getitem__(self, idx):
        c = self.cuts[idx]
        x = c.load_audio(self.sr)
        for a in self.aug:
            x = a(x)
        return torch.as_tensor(x), torch.tensor(len(x)), self.activity(c)

    def collate_fn(self, batch):
        alen = torch.tensor([int(b[1]) for b in batch], dtype=torch.long)
        audio = torch.zeros(len(batch), int(alen.max()))
        n = max(b[2].shape[0] for b in batch)
        act = torch.zeros(len(batch), n, self.S)
        tl = torch.zeros(len(batch), dtype=torch.long)
        for i, b in enumerate(batch):
            audio[i, : alen[i]] = b[0]
            act[i, : b[2].shape[0]] = b[2]
            tl[i] = b[2].shape[0]
        return audio, alen, act, tl

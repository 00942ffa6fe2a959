"""Data for the duplex (listen-while-speaking) models and the remaining helpers of the speech-LM collection.

A training example is a two-channel conversation: the user's audio (source), the agent's audio (target, speech-to-speech only) and
the turns ``{"role", "start", "end", "text"}``.  The text of every turn becomes a *token channel*: one token per perception frame,
laid out from the frame of the turn's start (``BOS``, then the tokens on consecutive frames, ``EOS`` where the turn ends), padding
elsewhere — this is what the LLM predicts frame by frame.  With word timestamps in the text (``<|0.48|> word``) every word starts
at its own frame instead.

* ``build_token_channel`` / ``text_with_timestamps_to_ids`` / ``collate_token_channel`` / ``delay_eos``
* ``DuplexConversationDataset`` (+ ``synthetic_duplex_conversations``, ``build_duplex_dataloader``)
* ``AudioAugmenter`` — user-channel augmentation (background noise at a random SNR, room response, gain, band limit)
* ``encode_audio_with_optional_chunking`` — long recordings through the perception module in chunks
* ``configure_optimizers_exclude_norm_from_wd``, ``tokens_to_str``, ``build_speaker_tokens``, ``ForceAligner``

References: ``speechlm2/data/{s2s_dataset,duplex_stt_dataset,force_align}.py``, ``speechlm2/parts/{label_prep,augmentation,
encoder_chunking,optim_setup,text_utils,multispeaker}.py``.
"""
from __future__ import annotations

import json
import math
import re
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

__all__ = ["AudioAugmenter", "DuplexConversationDataset", "ForceAligner", "build_duplex_dataloader", "build_speaker_tokens", "build_token_channel",
           "collate_token_channel", "configure_optimizers_exclude_norm_from_wd", "delay_eos", "encode_audio_with_optional_chunking",
           "synthetic_duplex_conversations", "text_with_timestamps_to_ids", "tokens_to_str"]

_TS = re.compile(r"<\|(\d+(?:\.\d+)?)\|>")


# ------------------------------------------------------------------------------------------------ token channels
def text_with_timestamps_to_ids(text: str, tokenizer, frame_sec: float, turn_start: float = 0.0) -> List[Tuple[int, List[int]]]:
    """``"<|0.00|> hello <|0.40|> world"`` -> ``[(frame offset, token ids of the word), ...]``; times are relative to the turn
    start unless they exceed it (absolute times are accepted too).  Text without marks gives one entry at offset 0."""
    parts = _TS.split(text)
    if len(parts) == 1:
        return [(0, list(tokenizer.text_to_ids(text.strip())))] if text.strip() else []
    out = []
    lead = parts[0].strip()
    if lead:
        out.append((0, list(tokenizer.text_to_ids(lead))))
    for t, w in zip(parts[1::2], parts[2::2]):
        w = w.strip()
        if not w:
            continue
        sec = float(t)
        sec = sec - turn_start if sec >= turn_start > 0 else sec
        out.append((max(0, int(round(sec / frame_sec))), list(tokenizer.text_to_ids(w))))
    return out


def build_token_channel(turns: Sequence[Dict[str, Any]], roles: Sequence[str], tokenizer, frame_sec: float, num_frames: int, bos_id: int, eos_id: int,
                        pad_id: int, truncate_to_turn: bool = True) -> torch.Tensor:
    """The channel of the speakers in ``roles``.  A turn's tokens that do not fit before its end are cut (``truncate_to_turn``) so
    that ``EOS`` stays aligned with the end of the audio of the turn; a later turn overwrites the tail of an overlapping earlier one."""
    ch = torch.full((num_frames,), pad_id, dtype=torch.long)
    for turn in sorted(turns, key=lambda t: t["start"]):
        if turn["role"] not in roles:
            continue
        s = int(round(turn["start"] / frame_sec))
        e = min(num_frames - 1, int(round(turn["end"] / frame_sec)))
        if s >= num_frames:
            continue
        ch[s] = bos_id
        pos = s + 1
        for off, ids in text_with_timestamps_to_ids(turn["text"], tokenizer, frame_sec, turn["start"]):
            pos = max(pos, s + 1 + off)
            for tok in ids:
                limit = e if truncate_to_turn else num_frames
                if pos >= limit:
                    break
                ch[pos] = tok
                pos += 1
        end = e if truncate_to_turn else min(num_frames - 1, max(pos, e))
        if end > s:
            ch[end] = eos_id
    return ch


def collate_token_channel(channels: Sequence[torch.Tensor], pad_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
    lens = torch.tensor([len(c) for c in channels])
    out = torch.full((len(channels), int(lens.max())), pad_id, dtype=torch.long)
    for i, c in enumerate(channels):
        out[i, : len(c)] = c
    return out, lens


def delay_eos(tokens: torch.Tensor, eos_token_id: int, pad_token_id: int, shift: int = 10) -> torch.Tensor:
    """Moves every ``EOS`` ``shift`` frames later (the frames in between become padding) unless another non-pad token lies on the
    way, in which case it moves as far as it can: gives the agent a little time before it must declare its turn finished."""
    out = tokens.clone()
    B, T = tokens.shape
    for b in range(B):
        for t in (tokens[b] == eos_token_id).nonzero().flatten().tolist():
            new = t
            for k in range(1, shift + 1):
                if t + k >= T or int(tokens[b, t + k]) != pad_token_id:
                    break
                new = t + k
            if new != t:
                out[b, t] = pad_token_id
                out[b, new] = eos_token_id
    return out


# ------------------------------------------------------------------------------------------------ dataset
class DuplexConversationDataset(Dataset):
    """Items: ``{"source_audio": path or array, "target_audio": path or array (optional), "turns": [...], "system_prompt": str (optional)}``
    (a JSON-lines manifest with the same keys, audio as paths, is read by ``from_manifest``).  Returns / collates to
    ``source_audio, source_audio_lens, target_audio?, target_audio_lens?, target_tokens, source_tokens, token_lens, prompt_tokens?``."""

    def __init__(self, items: Sequence[Dict[str, Any]], tokenizer, frame_sec: float = 0.08, sample_rate: int = 16000, target_sample_rate: Optional[int] = None,
                 input_roles: Sequence[str] = ("user", "User"), output_roles: Sequence[str] = ("agent", "Assistant", "assistant"), bos_id: int = 1, eos_id: int = 2,
                 pad_id: int = 0, eos_delay: int = 0, augmenter: Optional["AudioAugmenter"] = None, audio_codes_fn: Optional[Callable] = None):
        self.items, self.tok, self.frame_sec, self.sr, self.tsr = list(items), tokenizer, frame_sec, sample_rate, target_sample_rate or sample_rate
        self.in_roles, self.out_roles = set(input_roles), set(output_roles)
        self.bos, self.eos, self.pad, self.eos_delay, self.aug, self.codes_fn = bos_id, eos_id, pad_id, eos_delay, augmenter, audio_codes_fn

    @classmethod
    def from_manifest(cls, path: str, tokenizer, **kw) -> "DuplexConversationDataset":
        return cls([json.loads(l) for l in open(path, encoding="utf-8") if l.strip()], tokenizer, **kw)

    def __len__(self):
        return len(self.items)

    def _audio(self, a, sr) -> torch.Tensor:
        if isinstance(a, str):
            from ..data.audio_to_text import load_audio

            a = load_audio(a, target_sr=sr)
        return torch.as_tensor(np.asarray(a), dtype=torch.float32).reshape(-1)

    def __getitem__(self, i) -> Dict[str, Any]:
        it = self.items[i]
        src = self._audio(it["source_audio"], self.sr)
        if self.aug is not None:
            src = self.aug(src, self.sr)
        n = int(math.ceil(src.numel() / self.sr / self.frame_sec))
        kw = dict(tokenizer=self.tok, frame_sec=self.frame_sec, num_frames=n, bos_id=self.bos, eos_id=self.eos, pad_id=self.pad)
        tgt = build_token_channel(it["turns"], self.out_roles, **kw)
        usr = build_token_channel(it["turns"], self.in_roles, **kw)
        if self.eos_delay:
            tgt = delay_eos(tgt[None], self.eos, self.pad, self.eos_delay)[0]
        ex: Dict[str, Any] = {"source_audio": src, "target_tokens": tgt, "source_tokens": usr}
        if it.get("target_audio") is not None:
            ex["target_audio"] = self._audio(it["target_audio"], self.tsr)
            if self.codes_fn is not None:
                ex["target_codes"] = self.codes_fn(ex["target_audio"])           # [T, K]
        if it.get("target_codes") is not None:
            ex["target_codes"] = torch.as_tensor(it["target_codes"], dtype=torch.long)
        if it.get("system_prompt"):
            ex["prompt_tokens"] = torch.tensor(list(self.tok.text_to_ids(it["system_prompt"])), dtype=torch.long)
        return ex

    def collate_fn(self, batch: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        pad = torch.nn.utils.rnn.pad_sequence
        out: Dict[str, torch.Tensor] = {"source_audio": pad([b["source_audio"] for b in batch], batch_first=True),
                                        "source_audio_lens": torch.tensor([b["source_audio"].numel() for b in batch])}
        out["target_tokens"], out["token_lens"] = collate_token_channel([b["target_tokens"] for b in batch], self.pad)
        out["source_tokens"], _ = collate_token_channel([b["source_tokens"] for b in batch], self.pad)
        if all("target_audio" in b for b in batch):
            out["target_audio"] = pad([b["target_audio"] for b in batch], batch_first=True)
            out["target_audio_lens"] = torch.tensor([b["target_audio"].numel() for b in batch])
        if all("target_codes" in b for b in batch):
            T = out["target_tokens"].shape[1]
            codes = [b["target_codes"][:T] for b in batch]
            out["target_codes"] = pad(codes, batch_first=True)
            if out["target_codes"].shape[1] < T:
                out["target_codes"] = torch.nn.functional.pad(out["target_codes"], (0, 0, 0, T - out["target_codes"].shape[1]))
        if any("prompt_tokens" in b for b in batch):
            ps = [b.get("prompt_tokens", torch.zeros(0, dtype=torch.long)) for b in batch]
            out["prompt_tokens"], out["prompt_token_lens"] = collate_token_channel(ps, self.pad)
        return out


def synthetic_duplex_conversations(num_samples: int, seed: int = 0, duration: float = 2.0, sample_rate: int = 16000, num_codebooks: int = 0, codebook_size: int = 16,
                                   frame_sec: float = 0.08) -> List[Dict[str, Any]]:
    g = np.random.default_rng(seed)
    out = []
    for _ in range(num_samples):
        n = int(duration * sample_rate)
        mid = float(g.uniform(0.3, 0.5)) * duration
        it = {"source_audio": (0.1 * g.standard_normal(n)).astype(np.float32),
              "turns": [{"role": "user", "start": 0.0, "end": mid, "text": "a b"}, {"role": "agent", "start": mid + 0.1, "end": duration - 0.05, "text": "c d e"}]}
        if num_codebooks:
            it["target_audio"] = (0.1 * g.standard_normal(n)).astype(np.float32)
            it["target_codes"] = g.integers(0, codebook_size, (int(math.ceil(duration / frame_sec)), num_codebooks)).tolist()
        out.append(it)
    return out


def build_duplex_dataloader(config, tokenizer, frame_sec: float, bos_id: int, eos_id: int, pad_id: int, num_codebooks: int = 0, codebook_size: int = 16,
                            rank: int = 0, world_size: int = 1) -> Optional[DataLoader]:
    if config is None:
        return None
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn, path = get("synthetic", None), get("manifest_filepath", None)
    if syn is None and path is None:
        return None
    kw = dict(frame_sec=frame_sec, sample_rate=int(get("sample_rate", 16000)), bos_id=bos_id, eos_id=eos_id, pad_id=pad_id, eos_delay=int(get("eos_delay", 0)))
    aug = get("augmenter", None)
    if aug is not None:
        kw["augmenter"] = AudioAugmenter(**dict(aug))
    if syn is not None:
        ds = DuplexConversationDataset(synthetic_duplex_conversations(num_codebooks=num_codebooks, codebook_size=codebook_size, frame_sec=frame_sec, **dict(syn)), tokenizer, **kw)
    else:
        ds = DuplexConversationDataset.from_manifest(path, tokenizer, **kw)
    sampler = torch.utils.data.distributed.DistributedSampler(ds, world_size, rank, shuffle=bool(get("shuffle", True))) if world_size > 1 else None
    return DataLoader(ds, batch_size=int(get("batch_size", 4)), shuffle=bool(get("shuffle", False)) and sampler is None, sampler=sampler, collate_fn=ds.collate_fn,
                      num_workers=int(get("num_workers", 0)))


# ------------------------------------------------------------------------------------------------ augmentation
class AudioAugmenter:
    """Applied to the user's channel: each effect fires with its own probability.  ``noise_pool`` / ``rir_pool`` are lists of arrays
    (or paths); without a noise pool white noise is used."""

    def __init__(self, noise_prob: float = 0.0, snr_range=(5.0, 30.0), noise_pool: Optional[Sequence] = None, rir_prob: float = 0.0, rir_pool: Optional[Sequence] = None,
                 gain_prob: float = 0.0, gain_db_range=(-12.0, 6.0), lowpass_prob: float = 0.0, lowpass_hz_range=(3000.0, 7000.0), seed: int = 0):
        self.p_noise, self.snr, self.noise_pool = noise_prob, snr_range, list(noise_pool or [])
        self.p_rir, self.rir_pool = rir_prob, list(rir_pool or [])
        self.p_gain, self.gain, self.p_lp, self.lp = gain_prob, gain_db_range, lowpass_prob, lowpass_hz_range
        self.rng = np.random.default_rng(seed)

    def _load(self, a, sr):
        if isinstance(a, str):
            from ..data.audio_to_text import load_audio

            a = load_audio(a, target_sr=sr)
        return torch.as_tensor(np.asarray(a), dtype=torch.float32).reshape(-1)

    def __call__(self, x: torch.Tensor, sample_rate: int) -> torch.Tensor:
        n = x.numel()
        if self.rir_pool and self.rng.random() < self.p_rir:
            h = self._load(self.rir_pool[int(self.rng.integers(len(self.rir_pool)))], sample_rate)
            nf = 1 << (n + h.numel() - 2).bit_length()
            y = torch.fft.irfft(torch.fft.rfft(x, nf) * torch.fft.rfft(h, nf), nf)[:n]
            x = y * (x.norm() / y.norm().clamp(min=1e-9))
        if self.rng.random() < self.p_lp:
            cut = float(self.rng.uniform(*self.lp))
            X = torch.fft.rfft(x)
            f = torch.fft.rfftfreq(n, 1.0 / sample_rate)
            x = torch.fft.irfft(X * torch.sigmoid((cut - f) / (0.02 * cut)), n)
        if self.rng.random() < self.p_noise:
            if self.noise_pool:
                nz = self._load(self.noise_pool[int(self.rng.integers(len(self.noise_pool)))], sample_rate)
                nz = nz.repeat(int(math.ceil(n / max(1, nz.numel()))))[:n]
            else:
                nz = torch.from_numpy(self.rng.standard_normal(n).astype(np.float32))
            snr = float(self.rng.uniform(*self.snr))
            x = x + nz * (x.pow(2).mean().sqrt() / nz.pow(2).mean().sqrt().clamp(min=1e-9)) * 10 ** (-snr / 20)
        if self.rng.random() < self.p_gain:
            x = x * 10 ** (float(self.rng.uniform(*self.gain)) / 20)
        return x.clamp(-1.0, 1.0)


# ------------------------------------------------------------------------------------------------ long audio through the perception module
def encode_audio_with_optional_chunking(perception, audio: torch.Tensor, audio_lens: torch.Tensor, chunk_size_seconds: Optional[float] = None,
                                        sampling_rate: int = 16000, min_chunk_seconds: float = 0.5) -> Tuple[torch.Tensor, torch.Tensor]:
    """Without ``chunk_size_seconds``: one call.  With it: every recording is cut into chunks of that length (a short remainder is
    merged into the previous chunk), all chunks of the batch go through the perception module as one batch, and the embeddings
    are put back together per recording — memory then depends on the chunk length, not on the recording length."""
    if not chunk_size_seconds:
        return perception(input_signal=audio, input_signal_length=audio_lens)
    n = int(chunk_size_seconds * sampling_rate)
    min_n = int(min_chunk_seconds * sampling_rate)
    pieces, owner = [], []
    for b in range(audio.shape[0]):
        L = int(audio_lens[b])
        cuts = list(range(0, L, n))
        if len(cuts) > 1 and L - cuts[-1] < min_n:
            cuts.pop()
        for k, s in enumerate(cuts):
            e = L if k == len(cuts) - 1 else s + n
            pieces.append(audio[b, s:e])
            owner.append(b)
    lens = torch.tensor([p.numel() for p in pieces], device=audio.device)
    batch = torch.nn.utils.rnn.pad_sequence(pieces, batch_first=True)
    emb, emb_len = perception(input_signal=batch, input_signal_length=lens)
    outs = [[] for _ in range(audio.shape[0])]
    for i, b in enumerate(owner):
        outs[b].append(emb[i, : int(emb_len[i])])
    joined = [torch.cat(o, dim=0) for o in outs]
    return torch.nn.utils.rnn.pad_sequence(joined, batch_first=True), torch.tensor([j.shape[0] for j in joined], device=audio.device)


# ------------------------------------------------------------------------------------------------ small parts
def configure_optimizers_exclude_norm_from_wd(model: torch.nn.Module, lr: float = 1e-4, weight_decay: float = 0.01, betas=(0.9, 0.98), optimizer_cls=torch.optim.AdamW,
                                              **kw):
    """Two parameter groups: weights of linear / embedding / convolution layers with weight decay; biases, normalisation gains and
    other one-dimensional parameters without."""
    decay, no_decay = [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (no_decay if p.dim() <= 1 or n.endswith(".bias") or "norm" in n.lower() else decay).append(p)
    return optimizer_cls([{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}], lr=lr, betas=betas, **kw)


def tokens_to_str(tokens: torch.Tensor, lengths: torch.Tensor, tokenizer, pad_id: int, eval_text_turn_taking: bool = False, bos_id: Optional[int] = None,
                  eos_id: Optional[int] = None) -> List[str]:
    """Frame-aligned token channels -> text; with ``eval_text_turn_taking`` the turn marks are kept as ``<bos>`` / ``<eos>`` so that
    text metrics also see when the agent started and stopped."""
    out = []
    for b in range(tokens.shape[0]):
        row = tokens[b, : int(lengths[b])].tolist()
        if eval_text_turn_taking:
            parts, cur = [], []
            for t in row:
                if t == pad_id:
                    continue
                if t in (bos_id, eos_id):
                    if cur:
                        parts.append(tokenizer.ids_to_text(cur))
                        cur = []
                    parts.append("<bos>" if t == bos_id else "<eos>")
                else:
                    cur.append(t)
            if cur:
                parts.append(tokenizer.ids_to_text(cur))
            out.append(" ".join(parts))
        else:
            out.append(tokenizer.ids_to_text([t for t in row if t not in (pad_id, bos_id, eos_id)]))
    return out


def build_speaker_tokens(speaker_cfg, tokenizer) -> List[int]:
    """Ids of the speaker-change tokens ``<|spltoken0|> ...`` (``num_speakers`` of them, or the explicit ``tokens`` list) used by
    multi-speaker speech LMs; every token must already be in the tokenizer."""
    if not speaker_cfg:
        return []
    get = speaker_cfg.get if hasattr(speaker_cfg, "get") else (lambda k, d=None: getattr(speaker_cfg, k, d))
    names = list(get("tokens", None) or [get("template", "<|spltoken{}|>").format(i) for i in range(int(get("num_speakers", 0)))])
    ids = []
    for n in names:
        i = tokenizer.token_to_id(n) if hasattr(tokenizer, "token_to_id") else None
        if i is None or i < 0:
            raise ValueError(f"speaker token {n!r} is not in the tokenizer")
        ids.append(int(i))
    return ids


class ForceAligner:
    """Adds word timestamps to the turns of a conversation with a CTC model: the audio of every turn is aligned to its text and
    the text is rewritten as ``<|t|> word`` marks, which ``build_token_channel`` then places word by word."""

    def __init__(self, asr_model, sample_rate: int = 16000):
        self.model, self.sr = asr_model, sample_rate

    def align_turn(self, audio: np.ndarray, text: str) -> List[Tuple[str, float, float]]:
        from ..decoding.forced_aligner import align_utterance

        _, words, _ = align_utterance(self.model, audio, text, self.sr)
        return [(w.text, float(w.start), float(w.end)) for w in words]

    def add_timestamps(self, item: Dict[str, Any], channel_key: str = "source_audio", roles: Sequence[str] = ("user", "User")) -> Dict[str, Any]:
        audio = item[channel_key]
        if isinstance(audio, str):
            from ..data.audio_to_text import load_audio

            audio = load_audio(audio, target_sr=self.sr)
        audio = np.asarray(audio, dtype=np.float32)
        out = dict(item, turns=[dict(t) for t in item["turns"]])
        for t in out["turns"]:
            if t["role"] not in roles or _TS.search(t["text"]):
                continue
            seg = audio[int(t["start"] * self.sr): int(t["end"] * self.sr)]
            try:
                words = self.align_turn(seg, t["text"])
            except (ValueError, RuntimeError):
                continue                                             # too short for its text: leave the turn unmarked
            t["text"] = " ".join(f"<|{s:.2f}|> {w}" for w, s, _ in words)
        return out

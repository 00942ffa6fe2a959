"""Speech-LLM data: multimodal conversations → prompt-formatted token streams with audio placeholders.

Input manifests are JSON lines in the reference's multimodal-conversation schema
(``common/data/lhotse/text_adapters.py`` ``NeMoMultimodalConversation``):
``{"id": ..., "conversations": [{"from": "User", "type": "audio", "value": "<path>", "duration": 3.2},
{"from": "User", "type": "text", "value": "Transcribe."}, {"from": "Assistant", "type": "text", "value": "..."}]}``.
Consecutive turns of one speaker are merged; audio turns become the ``audio_locator_tag`` inside the user message.  Batches
are formed by token budget (text tokens + audio seconds / ``token_equivalent_duration``) like the reference's multimodal
sampler (``sampling.py:30-200``).  ``SALMDataset`` semantics: ``speechlm2/data/salm_dataset.py``.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

from ..data.audio_to_text import load_audio


def read_conversations(path: str) -> List[Dict[str, Any]]:
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                out.append(json.loads(line))
    return out


def conversations_from_input_cfg(input_cfg, seed: int = 0, rank: int = 0, world: int = 1, max_examples: Optional[int] = None):
    """Any mixture of the cut pipeline's sources (``multimodal_conversation``, ``share_gpt``, ``lhotse_as_conversation``,
    ``nemo_sft_jsonl``, ``txt_pair``, plain audio manifests ...) as conversation records.  Audio cuts become
    (audio, transcript) turns, text pairs (question + source, target) turns.  ``max_examples`` bounds sources that repeat."""
    from ..core.config import DictConfig, to_container
    from ..data.cuts import parse_input_cfg

    if isinstance(input_cfg, DictConfig) or not isinstance(input_cfg, (list, str)):
        input_cfg = to_container(input_cfg, resolve=True)
    out = []
    for k, c in enumerate(parse_input_cfg(input_cfg, seed, rank, world)):
        if max_examples is not None and k >= max_examples:
            break
        kind = c.custom.get("kind")
        if kind == "conversation":
            out.append(c.custom["conversation"])
        elif kind == "sft":
            pre = [{"from": "System", "type": "text", "value": c.custom["system"]}] if c.custom.get("system") else []
            out.append({"id": c.id, "conversations": pre + [{"from": t["role"].title(), "type": "text", "value": t["value"]} for t in c.custom["turns"]]})
        elif kind == "text_pair":
            q = c.custom.get("question")
            out.append({"id": c.id, "conversations": [{"from": "User", "type": "text", "value": (q + " " if q else "") + c.custom["source"]},
                                                      {"from": "Assistant", "type": "text", "value": c.custom["target"]}]})
        elif kind == "text":
            out.append({"id": c.id, "conversations": [{"from": "Assistant", "type": "text", "value": c.text}]})
        else:
            a = {"from": "User", "type": "audio", "value": c.audio if isinstance(c.audio, str) else c.id, "duration": c.duration, "offset": c.offset}
            if not isinstance(c.audio, str):
                a["audio"] = c.load_audio()
            out.append({"id": c.id, "conversations": [a, {"from": "Assistant", "type": "text", "value": c.text}]})
    return out


class SALMDataset(Dataset):
    def __init__(self, conversations: Sequence[Dict[str, Any]], tokenizer, prompt_formatter, audio_locator_tag: str,
                 pad_id: int, sample_rate: int = 16000, token_equivalent_duration: float = 0.08):
        self.items = list(conversations)
        self.tokenizer, self.fm, self.tag, self.pad_id, self.sr = tokenizer, prompt_formatter, audio_locator_tag, pad_id, sample_rate
        self.ted = token_equivalent_duration

    def __len__(self):
        return len(self.items)

    def cost(self, idx: int) -> float:
        it = self.items[idx]
        c = 0.0
        for t in it["conversations"]:
            if t.get("type", "text") == "audio":
                c += float(t.get("duration", 1.0)) / self.ted
            else:
                c += len(t["value"]) / 3.0
        return c

    def __getitem__(self, idx):
        it = self.items[idx]
        turns: List[Dict[str, Any]] = []
        audios = []
        for t in it["conversations"]:
            role = "assistant" if t["from"].lower() in ("assistant", "agent", "gpt") else \
                ("system" if t["from"].lower() == "system" else "user")
            if t.get("type", "text") == "audio":
                v = t["audio"] if t.get("audio") is not None else t["value"]
                x = load_audio(v, target_sr=self.sr, offset=float(t.get("offset", 0.0) or 0.0), duration=t.get("duration")) \
                    if isinstance(v, str) else np.asarray(v, dtype=np.float32)
                audios.append(torch.as_tensor(x, dtype=torch.float32))
                text = self.tag
            else:
                text = t["value"]
            if turns and turns[-1]["role"] == role:
                turns[-1]["slots"]["message"] += " " + text
            else:
                turns.append({"role": role, "slots": {"message": text}})
        enc = self.fm.encode_dialog(turns)
        return {"input_ids": enc["input_ids"], "loss_mask": enc["mask"], "audios": audios}

    def collate(self, batch: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        L = max(b["input_ids"].numel() for b in batch)
        ids = torch.full((len(batch), L), self.pad_id, dtype=torch.long)
        mask = torch.zeros((len(batch), L), dtype=torch.bool)
        for i, b in enumerate(batch):
            n = b["input_ids"].numel()
            ids[i, :n] = b["input_ids"]
            mask[i, :n] = b["loss_mask"]
        auds = [a for b in batch for a in b["audios"]]
        alen = torch.tensor([a.numel() for a in auds], dtype=torch.long)
        audio = torch.zeros((len(auds), int(alen.max()) if len(auds) else 1))
        for i, a in enumerate(auds):
            audio[i, : a.numel()] = a
        # the number of positions with a target, counted here on the host: models use it to size per-target work without a device read
        return {"audios": audio, "audio_lens": alen, "input_ids": ids, "loss_mask": mask, "num_loss_tokens": int(mask.sum())}


def synthetic_conversations(num_samples: int, seed: int = 0, min_duration: float = 0.5, max_duration: float = 1.5,
                            sample_rate: int = 16000) -> List[Dict[str, Any]]:
    g = np.random.default_rng(seed)
    words = ["alpha", "bravo", "charlie", "delta", "echo", "foxtrot"]
    out = []
    for i in range(num_samples):
        d = float(g.uniform(min_duration, max_duration))
        k = int(g.integers(0, len(words)))
        t = np.arange(int(d * sample_rate)) / sample_rate
        x = (0.3 * np.sin(2 * np.pi * (250 + 150 * k) * t) + 0.01 * g.standard_normal(t.shape[0])).astype(np.float32)
        out.append({"id": f"syn{i}", "conversations": [
            {"from": "User", "type": "text", "value": "Transcribe:"},
            {"from": "User", "type": "audio", "value": x, "duration": d},
            {"from": "Assistant", "type": "text", "value": words[k]}]})
    return out


class TokenBudgetLoader:
    """Batches by ``batch_tokens`` (or fixed ``batch_size``), sharded over data-parallel ranks."""

    def __init__(self, ds: SALMDataset, batch_size: Optional[int] = None, batch_tokens: Optional[float] = None,
                 shuffle: bool = False, seed: int = 0, rank: int = 0, world_size: int = 1, drop_last: bool = False):
        self.ds, self.bs, self.bt, self.shuffle, self.seed = ds, batch_size, batch_tokens, shuffle, seed
        self.rank, self.world, self.drop_last = rank, world_size, drop_last
        self.epoch = 0

    def set_epoch(self, e: int):
        self.epoch = e

    def _batches(self) -> List[List[int]]:
        idx = list(range(len(self.ds)))
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(idx)
        out, cur, cost = [], [], 0.0
        for i in idx:
            c = self.ds.cost(i) if self.bt else 1.0
            limit = self.bt if self.bt else self.bs
            if cur and cost + c > limit:
                out.append(cur)
                cur, cost = [], 0.0
            cur.append(i)
            cost += c
        if cur and not self.drop_last:
            out.append(cur)
        n = len(out) // self.world * self.world if self.world > 1 else len(out)
        return out[:n][self.rank::self.world] if self.world > 1 else out

    def __len__(self):
        return len(self._batches())

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        for b in self._batches():
            yield self.ds.collate([self.ds[i] for i in b])


def build_salm_dataloader(config, tokenizer, prompt_formatter, audio_locator_tag: str, pad_id: int, rank: int = 0, world_size: int = 1):
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    syn = get("synthetic", None)
    if syn is not None:
        convs = synthetic_conversations(**dict(syn))
    elif get("input_cfg", None) is not None:
        convs = conversations_from_input_cfg(get("input_cfg"), seed=get("seed", 0), rank=rank, world=world_size,
                                             max_examples=get("max_examples", None))
    else:
        convs = read_conversations(get("manifest_filepath"))
    ds = SALMDataset(convs, tokenizer, prompt_formatter, audio_locator_tag, pad_id, sample_rate=get("sample_rate", 16000),
                     token_equivalent_duration=get("token_equivalent_duration", 0.08))
    return TokenBudgetLoader(ds, batch_size=get("batch_size", None) or (None if get("batch_tokens", None) else 4),
                             batch_tokens=get("batch_tokens", None), shuffle=get("shuffle", False), seed=get("seed", 0),
                             rank=rank, world_size=world_size, drop_last=get("drop_last", False))

"""Datasets of pre-extracted codec tokens for the token-level speech generators (EasyMagpieTTS, EAR-TTS).

A manifest line holds ``text`` (or ``text_tokens``), ``codes_path`` (``.npy``, int array ``[C, T]``) and optionally ``duration``.
``synthetic: {num_samples, ...}`` in the dataset config produces random tokens of the right shapes instead, which is what the
example configs and the tests run on.  ``frame_aligned=True`` yields the duplex layout (one text token per audio frame, PAD
outside the spoken span) used by the EAR-TTS models; otherwise text and codes keep their own lengths.
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

from ..core.config import cfg_get


class CodeDataset(Dataset):
    def __init__(self, cfg: Any, num_codebooks: int, codebook_size: int, text_vocab: int, tokenizer=None, frame_aligned: bool = False,
                 text_pad_id: int = 0):
        self.C, self.N, self.V, self.tok = num_codebooks, codebook_size, text_vocab, tokenizer
        self.frame_aligned, self.pad = frame_aligned, text_pad_id
        syn = cfg_get(cfg, "synthetic", None)
        self.items: List[Dict[str, Any]] = []
        if syn is not None:
            g = np.random.default_rng(int(cfg_get(syn, "seed", 0)))
            lo, hi = int(cfg_get(syn, "min_frames", 8)), int(cfg_get(syn, "max_frames", 24))
            for _ in range(int(cfg_get(syn, "num_samples", 16))):
                T = int(g.integers(lo, hi + 1))
                L = int(g.integers(3, max(4, T // 2)))
                self.items.append({"text_tokens": g.integers(3, self.V, L).tolist(), "codes": g.integers(0, self.N, (self.C, T))})
        else:
            with open(cfg_get(cfg, "manifest_filepath"), encoding="utf-8") as f:
                self.items = [json.loads(l) for l in f if l.strip()]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        it = self.items[i]
        codes = it["codes"] if "codes" in it else np.load(it["codes_path"])
        toks = it.get("text_tokens")
        if toks is None:
            toks = self.tok.text_to_ids(it["text"])
        return torch.as_tensor(np.asarray(codes), dtype=torch.long), torch.as_tensor(toks, dtype=torch.long)

    def collate(self, batch):
        B = len(batch)
        T = max(c.shape[1] for c, _ in batch)
        codes = torch.zeros(B, self.C, T, dtype=torch.long)
        clen = torch.tensor([c.shape[1] for c, _ in batch])
        for b, (c, _) in enumerate(batch):
            codes[b, :, : c.shape[1]] = c
        if self.frame_aligned:
            text = torch.full((B, T), self.pad, dtype=torch.long)
            for b, (c, t) in enumerate(batch):
                n = min(len(t), c.shape[1])
                text[b, :n] = t[:n]                                   # the words lead the speech that realises them
            return {"target_tokens": text, "target_codes": codes.transpose(1, 2).contiguous(), "target_lens": clen}
        L = max(len(t) for _, t in batch)
        text = torch.zeros(B, L, dtype=torch.long)
        for b, (_, t) in enumerate(batch):
            text[b, : len(t)] = t
        return {"text": text, "text_len": torch.tensor([len(t) for _, t in batch]), "codes": codes, "codes_len": clen}


def build_code_dataloader(cfg: Optional[Any], **kw) -> Optional[DataLoader]:
    if cfg is None:
        return None
    ds = CodeDataset(cfg, **kw)
    return DataLoader(ds, batch_size=int(cfg_get(cfg, "batch_size", 4)), shuffle=bool(cfg_get(cfg, "shuffle", False)), collate_fn=ds.collate,
                      num_workers=int(cfg_get(cfg, "num_workers", 0)))

"""Small parts around the MagpieTTS model: the special audio tokens that follow the codec's codes in every codebook, code-frame
utilities (BOS / EOS insertion and removal, padding to the frame-stacking factor, forbidding special tokens in sampling), the
MaskGit cosine schedule, and the character-aware sub-word encoder.

Reference: ``tts/modules/magpietts_modules.py``.
"""
from __future__ import annotations

import math
from enum import Enum
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

__all__ = ["CharAwareSubwordEncoder", "EOSDetectionMethod", "LocalTransformerType", "SpecialAudioToken", "add_eos_token", "add_special_tokens", "build_vocabs",
           "clear_forbidden_logits", "cosine_schedule", "pad_audio_codes", "remove_bos_token", "remove_eos_token", "remove_special_tokens"]


class LocalTransformerType(str, Enum):
    NO_LT = "none"
    AR = "autoregressive"
    MASKGIT = "maskgit"


class EOSDetectionMethod(str, Enum):
    """Which codebooks, and argmax or sampled tokens, decide that the utterance has ended."""
    ARGMAX_ANY = "argmax_any"
    ARGMAX_OR_MULTINOMIAL_ANY = "argmax_or_multinomial_any"
    ARGMAX_ALL = "argmax_all"
    ARGMAX_OR_MULTINOMIAL_ALL = "argmax_or_multinomial_all"
    ARGMAX_ZERO_CB = "argmax_zero_cb"
    ARGMAX_OR_MULTINOMIAL_ZERO_CB = "argmax_or_multinomial_zero_cb"

    def detect(self, argmax_tokens: torch.Tensor, sampled_tokens: torch.Tensor, eos_id: int) -> torch.Tensor:
        """``[B, C]`` tokens of one frame -> ``[B]`` whether the frame ends the utterance."""
        a, s = argmax_tokens == eos_id, sampled_tokens == eos_id
        hit = (a | s) if "multinomial" in self.value else a
        if self.value.endswith("any"):
            return hit.any(dim=1)
        if self.value.endswith("all"):
            return hit.all(dim=1)
        return hit[:, 0]


class SpecialAudioToken(Enum):
    """Offsets above the codec's codebook size; eight slots are reserved so that adding a token later does not change table sizes."""
    AUDIO_BOS = 0
    AUDIO_EOS = 1
    AUDIO_CONTEXT_BOS = 2
    AUDIO_CONTEXT_EOS = 3
    MASK_TOKEN = 4
    RESERVED_1 = 5
    RESERVED_2 = 6
    RESERVED_3 = 7

    @staticmethod
    def get_index(token: "SpecialAudioToken", base_codebook_size: int) -> int:
        return base_codebook_size + token.value

    @staticmethod
    def get_forbidden_tokens(base_codebook_size: int, forbid_audio_eos: bool = False) -> List[int]:
        return [base_codebook_size + t.value for t in SpecialAudioToken if forbid_audio_eos or t is not SpecialAudioToken.AUDIO_EOS]


def cosine_schedule(x: torch.Tensor) -> torch.Tensor:
    """Share of tokens still masked at progress ``x`` in [0, 1] of MaskGit decoding: 1 at the start, 0 at the end."""
    return torch.cos(x * (math.pi / 2))


def clear_forbidden_logits(logits: torch.Tensor, codebook_size: int, forbid_audio_eos: bool = False) -> torch.Tensor:
    logits[..., SpecialAudioToken.get_forbidden_tokens(codebook_size, forbid_audio_eos)] = float("-inf")
    return logits


def pad_audio_codes(audio_codes: torch.Tensor, frame_stacking_factor: int, value: int = 0) -> torch.Tensor:
    """[B, C, T] -> T padded up to a multiple of the stacking factor."""
    pad = (-audio_codes.shape[2]) % frame_stacking_factor
    return F.pad(audio_codes, (0, pad), value=value) if pad else audio_codes


def add_eos_token(codes: torch.Tensor, codes_len: torch.Tensor, eos_id: int, num_eos_tokens: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    out = F.pad(codes, (0, num_eos_tokens), value=0)
    pos = codes_len.view(-1, 1, 1) + torch.arange(num_eos_tokens, device=codes.device).view(1, 1, -1)
    out.scatter_(2, pos.expand(-1, codes.shape[1], -1), eos_id)
    return out, codes_len + num_eos_tokens


def add_special_tokens(codes, codes_len, bos_id: int, eos_id: int, num_bos_tokens: int = 1, num_eos_tokens: int = 1):
    codes = F.pad(codes, (num_bos_tokens, 0), value=bos_id)
    return add_eos_token(codes, codes_len + num_bos_tokens, eos_id, num_eos_tokens)


def remove_bos_token(codes, codes_len, num_tokens: int = 1):
    return codes[:, :, num_tokens:], codes_len - num_tokens


def remove_eos_token(codes, codes_len):
    """Drops the last valid position of every row (and one column of padding)."""
    out_len = codes_len - 1
    out = codes[:, :, :-1].clone()
    mask = torch.arange(out.shape[2], device=codes.device)[None, None, :] < out_len[:, None, None]
    return out * mask, out_len


def remove_special_tokens(codes, codes_len, num_bos_tokens: int = 1):
    codes, codes_len = remove_bos_token(codes, codes_len, num_bos_tokens)
    return remove_eos_token(codes, codes_len)


# ------------------------------------------------------------------------------------------------ character-aware sub-word encoder
def build_vocabs(subword_vocab: Dict[str, int], subword_padding_idx: int, special_vocab: Optional[Dict[str, int]] = None) -> Tuple[Dict[int, List[int]], Dict[str, int]]:
    """``{sub-word id: [character ids]}`` and the character vocabulary.  Word-boundary marks of the tokenizer (``▁``, ``Ġ``, ``##``)
    are spelled as a space; special tokens become single pseudo-characters."""
    chars: Dict[str, int] = {"<pad>": 0}
    table: Dict[int, List[int]] = {}
    special = special_vocab or {}
    for tok, i in subword_vocab.items():
        if i == subword_padding_idx:
            continue
        if tok in special or (tok.startswith("<") and tok.endswith(">") and len(tok) > 2):
            chars.setdefault(tok, len(chars))
            table[i] = [chars[tok]]
            continue
        spelled = tok.replace("▁", " ").replace("Ġ", " ")
        spelled = spelled[2:] if spelled.startswith("##") else spelled
        ids = []
        for ch in spelled:
            chars.setdefault(ch, len(chars))
            ids.append(chars[ch])
        table[i] = ids or [0]
    return table, chars


class CharAwareSubwordEncoder(nn.Module):
    """Embeds a sub-word as a function of its spelling: characters -> embedding -> a small Transformer over the characters of each
    sub-word -> mean over characters.  Sub-words that look alike get nearby embeddings, and rare sub-words borrow from frequent
    ones; the table-free design also lets the text vocabulary change without retraining an embedding matrix."""

    def __init__(self, d_embed: int, subword_vocab: Dict[str, int], subword_padding_idx: int, special_vocab: Optional[Dict[str, int]] = None, n_layers: int = 1,
                 n_heads: int = 4, max_chars: int = 32):
        super().__init__()
        self.pad_idx = subword_padding_idx
        table, self.char_vocab = build_vocabs(subword_vocab, subword_padding_idx, special_vocab)
        n = max(subword_vocab.values()) + 1
        L = min(max_chars, max(len(v) for v in table.values()))
        spell = torch.zeros(n, L, dtype=torch.long)
        for i, ids in table.items():
            spell[i, : min(L, len(ids))] = torch.tensor(ids[:L])
        self.register_buffer("spelling", spell, persistent=False)
        self.char_emb = nn.Embedding(len(self.char_vocab), d_embed, padding_idx=0)
        self.pos_emb = nn.Embedding(L, d_embed)
        self.layers = nn.ModuleList([nn.TransformerEncoderLayer(d_embed, n_heads, 2 * d_embed, 0.0, batch_first=True, norm_first=True) for _ in range(n_layers)])
        self.norm = nn.LayerNorm(d_embed)

    def forward(self, subword_ids: torch.Tensor, subword_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[B, T] -> [B, T, d_embed]; only the distinct sub-words of the batch are encoded."""
        uniq, inv = torch.unique(subword_ids, return_inverse=True)
        sp = self.spelling[uniq]                                          # [U, L]
        cm = sp != 0
        cm[:, 0] = True                                                   # never an empty row
        h = self.char_emb(sp) + self.pos_emb(torch.arange(sp.shape[1], device=sp.device))[None]
        for l in self.layers:
            h = l(h, src_key_padding_mask=~cm)
        h = self.norm(h)
        e = (h * cm.unsqueeze(-1)).sum(1) / cm.sum(1, keepdim=True)
        e = torch.where((uniq == self.pad_idx).unsqueeze(-1), torch.zeros_like(e), e)
        out = e[inv]
        return out * subword_mask.unsqueeze(-1).to(out.dtype) if subword_mask is not None else out

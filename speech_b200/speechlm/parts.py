"""Speech-LLM helpers: packed (THD) sequences, context-parallel batch helpers, encoder chunking for long audio, metrics.

Reference: ``speechlm2/parts/packed_sequences.py`` (per-utterance splice + next-token shift, lengths rounded to ``2·cp_size``,
total bumped to a multiple of ``tp_size``, ``cu_seqlens`` / ``position_ids``), ``parts/cp_helpers.py`` (split audio over CP
ranks with dummy padding, MAX all-reduce of lengths, differentiable all-gather), ``parts/encoder_chunking.py`` (split audio
into ≤ N-second chunks for the encoder, recombine embeddings), ``parts/metrics/*``.
"""
from __future__ import annotations

import math
from collections import Counter
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

IGNORE_INDEX = -100


# ---------------------------------------------------------------------------------------------- packed sequences
@dataclass
class PackedBatch:
    input_embeds: torch.Tensor        # [1, T_total, H]
    target_ids: torch.Tensor          # [1, T_total]
    position_ids: torch.Tensor        # [1, T_total]
    seq_ids: torch.Tensor             # [1, T_total]  (-1 on padding)
    cu_seqlens: torch.Tensor          # [n_seq + 1] int32
    max_seqlen: int


def pack_sequences(embeds: Sequence[torch.Tensor], targets: Sequence[torch.Tensor], cp_size: int = 1, tp_size: int = 1) -> PackedBatch:
    """Concatenate variable-length sequences (each already spliced with audio) into one row.  Inputs / targets are shifted
    per sequence for next-token prediction, every sequence is right-padded to a multiple of ``2 * cp_size`` and the total to
    a multiple of ``tp_size`` (sequence parallelism needs even shards)."""
    H = embeds[0].shape[-1]
    dev, dt = embeds[0].device, embeds[0].dtype
    es, ts, ps, ss, lens = [], [], [], [], []
    mult = max(1, 2 * cp_size) if cp_size > 1 else 1
    for i, (e, t) in enumerate(zip(embeds, targets)):
        e, t = e[:-1], t[1:]
        n = e.shape[0]
        pad = (-n) % mult
        es.append(torch.cat([e, e.new_zeros((pad, H))]) if pad else e)
        ts.append(torch.cat([t, t.new_full((pad,), IGNORE_INDEX)]) if pad else t)
        ps.append(torch.arange(n + pad, device=dev))
        ss.append(torch.full((n + pad,), i, device=dev, dtype=torch.long))
        lens.append(n + pad)
    total = sum(lens)
    extra = (-total) % max(1, tp_size)
    if extra:
        es.append(torch.zeros((extra, H), device=dev, dtype=dt))
        ts.append(torch.full((extra,), IGNORE_INDEX, device=dev, dtype=torch.long))
        ps.append(torch.arange(extra, device=dev))
        ss.append(torch.full((extra,), -1, device=dev, dtype=torch.long))
        lens.append(extra)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=dev)
    return PackedBatch(torch.cat(es).unsqueeze(0), torch.cat(ts).unsqueeze(0), torch.cat(ps).unsqueeze(0), torch.cat(ss).unsqueeze(0),
                       cu, max(lens))


def thd_partition_indices(cu_seqlens: torch.Tensor, cp_size: int, cp_rank: int) -> torch.Tensor:
    """Token indices of one context-parallel rank: every sequence is cut into ``2 * cp_size`` equal chunks and rank ``r``
    takes chunks ``r`` and ``2 * cp_size - 1 - r`` (load-balanced causal attention)."""
    out = []
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        n = b - a
        c = n // (2 * cp_size)
        if c == 0:
            if cp_rank == 0:
                out.append(torch.arange(a, b))
            continue
        for k in (cp_rank, 2 * cp_size - 1 - cp_rank):
            out.append(torch.arange(a + k * c, a + (k + 1) * c))
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


# ---------------------------------------------------------------------------------------------- context-parallel helpers
def split_audio_for_cp(audios: torch.Tensor, audio_lens: torch.Tensor, cp_size: int, cp_rank: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Give every CP rank ``ceil(N / cp)`` recordings (dummy one-sample recordings pad the tail); returns the local slice and
    the number of real recordings in it."""
    N = audios.shape[0]
    per = -(-N // cp_size)
    lo, hi = cp_rank * per, min(N, (cp_rank + 1) * per)
    real = max(0, hi - lo)
    a = audios[lo:hi] if real else audios[:0]
    l = audio_lens[lo:hi] if real else audio_lens[:0]
    if real < per:
        a = torch.cat([a, audios.new_zeros((per - real, audios.shape[1]))])
        l = torch.cat([l, audio_lens.new_ones(per - real)])
    return a, l, real


class _AllGatherCat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        ws = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        ws, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g.chunk(ws, dim=0)[r], None


def gather_embeddings_across_cp(emb: torch.Tensor, emb_len: torch.Tensor, group) -> Tuple[torch.Tensor, torch.Tensor]:
    """Differentiable all-gather of per-rank audio embeddings [n, T, H] (time padded to the global maximum first)."""
    if group is None or dist.get_world_size(group) == 1:
        return emb, emb_len
    T = torch.tensor([emb.shape[1]], device=emb.device)
    dist.all_reduce(T, op=dist.ReduceOp.MAX, group=group)
    emb = torch.nn.functional.pad(emb, (0, 0, 0, int(T) - emb.shape[1]))
    lens = [torch.empty_like(emb_len) for _ in range(dist.get_world_size(group))]
    dist.all_gather(lens, emb_len, group=group)
    return _AllGatherCat.apply(emb, group), torch.cat(lens)


# ---------------------------------------------------------------------------------------------- encoder chunking
def chunk_audio(audios: torch.Tensor, audio_lens: torch.Tensor, chunk_samples: int):
    """Split every recording into chunks of at most ``chunk_samples``.  Returns (chunks [M, chunk_samples], chunk_lens [M],
    owner [M])."""
    chunks, lens, owner = [], [], []
    for i in range(audios.shape[0]):
        n = int(audio_lens[i])
        for s in range(0, max(n, 1), chunk_samples):
            e = min(n, s + chunk_samples)
            c = audios[i, s:e]
            chunks.append(torch.nn.functional.pad(c, (0, chunk_samples - c.shape[0])))
            lens.append(max(e - s, 1))
            owner.append(i)
    return torch.stack(chunks), torch.tensor(lens, device=audios.device), torch.tensor(owner, device=audios.device)


def recombine_chunk_embeddings(emb: torch.Tensor, emb_lens: torch.Tensor, owner: torch.Tensor, n_audio: int):
    """Concatenate the valid frames of the chunks of each recording; returns padded [N, T, H] and lengths."""
    rows = [[] for _ in range(n_audio)]
    for k in range(emb.shape[0]):
        rows[int(owner[k])].append(emb[k, : int(emb_lens[k])])
    rows = [torch.cat(r) if r else emb.new_zeros((0, emb.shape[-1])) for r in rows]
    lens = torch.tensor([r.shape[0] for r in rows], device=emb.device)
    out = emb.new_zeros((n_audio, int(lens.max()) if n_audio else 0, emb.shape[-1]))
    for i, r in enumerate(rows):
        out[i, : r.shape[0]] = r
    return out, lens


def encode_in_chunks(perception, audios: torch.Tensor, audio_lens: torch.Tensor, chunk_seconds: float, sample_rate: int = 16000):
    ch, cl, owner = chunk_audio(audios, audio_lens, int(chunk_seconds * sample_rate))
    emb, el = perception(input_signal=ch, input_signal_length=cl)
    return recombine_chunk_embeddings(emb, el, owner, audios.shape[0])


# ---------------------------------------------------------------------------------------------- metrics
def token_accuracy(logits: torch.Tensor, targets: torch.Tensor) -> float:
    m = targets != IGNORE_INDEX
    return float(((logits.argmax(-1) == targets) & m).sum()) / max(1, int(m.sum()))


def perplexity(loss_sum: float, n_tokens: int) -> float:
    return math.exp(loss_sum / max(1, n_tokens))


def global_token_normalised_loss(loss_sum: torch.Tensor, n_tokens: torch.Tensor, group=None) -> torch.Tensor:
    """Cross entropy normalised by the number of labelled tokens over ALL data-parallel ranks (``salm_automodel.py:373-390``):
    the gradient then equals the gradient of the global mean instead of a mean of per-rank means."""
    n = n_tokens.detach().clone().float()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(n, group=group)
        return loss_sum * dist.get_world_size(group) / n.clamp(min=1)
    return loss_sum / n.clamp(min=1)


def bleu(hyps: Sequence[str], refs: Sequence[str], max_n: int = 4) -> float:
    """Corpus BLEU with brevity penalty (single reference, whitespace tokens)."""
    match, total = [0] * max_n, [0] * max_n
    hl = rl = 0
    for h, r in zip(hyps, refs):
        ht, rt = h.split(), r.split()
        hl, rl = hl + len(ht), rl + len(rt)
        for n in range(1, max_n + 1):
            hc = Counter(tuple(ht[i:i + n]) for i in range(len(ht) - n + 1))
            rc = Counter(tuple(rt[i:i + n]) for i in range(len(rt) - n + 1))
            match[n - 1] += sum(min(c, rc[g]) for g, c in hc.items())
            total[n - 1] += max(0, len(ht) - n + 1)
    if min(total) == 0 or min(match) == 0:
        return 0.0
    logp = sum(math.log(m / t) for m, t in zip(match, total)) / max_n
    bp = 1.0 if hl > rl else math.exp(1 - rl / max(hl, 1))
    return 100.0 * bp * math.exp(logp)

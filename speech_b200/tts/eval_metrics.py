"""Objective evaluation of synthesised speech: real-time factor, intelligibility, speaker similarity, Fréchet codec distance.

* ``frechet_distance(mu1, cov1, mu2, cov2)`` — ``|mu1 - mu2|^2 + tr(C1 + C2 - 2 (C1 C2)^{1/2})``; the matrix square root is
  taken through the symmetric form ``C1^{1/2} C2 C1^{1/2}`` (eigendecompositions only, no complex arithmetic).
* ``FrechetCodecDistance`` — accumulates codec-latent frames (the dequantised codes of an ``AudioCodecModel``) of real and
  generated audio and reports the distance between the two Gaussians.
* ``speaker_similarity`` — cosine similarity of speaker embeddings from any ``embed(audio, lengths)`` callable (a speaker
  verification model of this framework, or an injected one).
* ``intelligibility`` — transcribes generated audio with an ASR callable and scores WER / CER against the input text.
* ``RTFMetrics`` — wall-clock synthesis time against generated audio duration.
* ``MosPredictorWrapper`` — batches audio through an injected MOS predictor (e.g. a UTMOS checkpoint loaded by the caller;
  no predictor weights ship with this package).
* ``evaluate_tts`` — the harness: runs a model's ``do_tts`` over a manifest and fills all metrics that have their callable.

Reference: ``tts/modules/magpietts_inference/*`` (batch inference + RTF), ``tts/metrics/*`` (Fréchet codec distance),
``scripts/magpietts/evaluate_generated_audio.py`` (ASR-WER / speaker similarity / UTMOS).
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..utils.metrics import word_error_rate


def _sqrtm_psd(m: torch.Tensor) -> torch.Tensor:
    w, v = torch.linalg.eigh((m + m.T) / 2)
    return (v * w.clamp(min=0).sqrt()) @ v.T


def frechet_distance(mu1: torch.Tensor, cov1: torch.Tensor, mu2: torch.Tensor, cov2: torch.Tensor) -> float:
    mu1, mu2, cov1, cov2 = mu1.double(), mu2.double(), cov1.double(), cov2.double()
    r1 = _sqrtm_psd(cov1)
    cross = _sqrtm_psd(r1 @ cov2 @ r1)
    d = (mu1 - mu2).pow(2).sum() + torch.trace(cov1) + torch.trace(cov2) - 2 * torch.trace(cross)
    return float(d.clamp(min=0))


class _Gaussian:
    def __init__(self):
        self.n, self.s, self.ss = 0, None, None

    def update(self, x: torch.Tensor) -> None:
        x = x.detach().double().reshape(-1, x.shape[-1]).cpu()
        if self.s is None:
            self.s, self.ss = torch.zeros(x.shape[1], dtype=torch.double), torch.zeros(x.shape[1], x.shape[1], dtype=torch.double)
        self.n += x.shape[0]
        self.s += x.sum(0)
        self.ss += x.T @ x

    def stats(self):
        if self.n < 2:
            raise ValueError("at least two frames are needed")
        mu = self.s / self.n
        return mu, (self.ss - self.n * torch.outer(mu, mu)) / (self.n - 1)


class FrechetCodecDistance:
    """``update(real_latents=..., fake_latents=...)`` with tensors [..., D] (or audio, when a ``codec`` with
    ``encode`` + ``dequantize`` is given); ``compute()`` -> float."""

    def __init__(self, codec=None):
        self.codec, self.real, self.fake = codec, _Gaussian(), _Gaussian()

    @torch.no_grad()
    def _latents(self, audio: torch.Tensor, audio_len: torch.Tensor) -> torch.Tensor:
        tokens, tokens_len = self.codec.encode(audio=audio, audio_len=audio_len)
        z = self.codec.dequantize(tokens=tokens, tokens_len=tokens_len)                     # [B, D, T]
        keep = torch.arange(z.shape[-1], device=z.device)[None] < tokens_len[:, None]
        return z.transpose(1, 2)[keep]

    def update(self, real_latents=None, fake_latents=None, real_audio=None, fake_audio=None) -> None:
        if real_audio is not None:
            real_latents = self._latents(*real_audio)
        if fake_audio is not None:
            fake_latents = self._latents(*fake_audio)
        if real_latents is not None:
            self.real.update(real_latents)
        if fake_latents is not None:
            self.fake.update(fake_latents)

    def compute(self) -> float:
        return frechet_distance(*self.real.stats(), *self.fake.stats())


@torch.no_grad()
def speaker_similarity(embed: Callable, audio_a, len_a, audio_b, len_b) -> torch.Tensor:
    ea, eb = embed(audio_a, len_a), embed(audio_b, len_b)
    return torch.nn.functional.cosine_similarity(ea.float(), eb.float(), dim=-1)


def intelligibility(transcribe: Callable[[List[Any]], List[str]], audios: List[Any], texts: Sequence[str]) -> Dict[str, float]:
    hyp = [h.text if hasattr(h, "text") else str(h) for h in transcribe(audios)]
    norm = lambda s: " ".join("".join(ch for ch in s.lower() if ch.isalnum() or ch.isspace()).split())  # noqa: E731
    hyp, ref = [norm(h) for h in hyp], [norm(t) for t in texts]
    return {"wer": word_error_rate(hyp, ref), "cer": word_error_rate(hyp, ref, use_cer=True)}


class RTFMetrics:
    def __init__(self, sample_rate: int):
        self.sample_rate, self.wall, self.samples, self.n = sample_rate, 0.0, 0, 0

    def timed(self, fn: Callable, *a, **kw):
        sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)
        sync()
        t0 = time.perf_counter()
        out = fn(*a, **kw)
        sync()
        self.wall += time.perf_counter() - t0
        return out

    def add_audio(self, num_samples: int) -> None:
        self.samples += int(num_samples)
        self.n += 1

    def compute(self) -> Dict[str, float]:
        dur = self.samples / self.sample_rate
        return {"rtf": self.wall / dur if dur else float("inf"), "rtfx": dur / self.wall if self.wall else float("inf"),
                "audio_seconds": dur, "wall_seconds": self.wall, "utterances": self.n}


class MosPredictorWrapper:
    def __init__(self, predictor: Callable[[torch.Tensor, int], torch.Tensor], sample_rate: int, batch_size: int = 8):
        self.predictor, self.sample_rate, self.batch_size = predictor, sample_rate, batch_size

    @torch.no_grad()
    def __call__(self, audios: List[torch.Tensor]) -> List[float]:
        out: List[float] = []
        for i in range(0, len(audios), self.batch_size):
            chunk = audios[i:i + self.batch_size]
            n = max(a.shape[-1] for a in chunk)
            x = torch.stack([torch.nn.functional.pad(a.reshape(-1), (0, n - a.shape[-1])) for a in chunk])
            out.extend(float(v) for v in self.predictor(x, self.sample_rate).reshape(-1))
        return out


def evaluate_tts(model, items: Iterable[Dict[str, Any]], sample_rate: int, transcribe: Optional[Callable] = None,
                 speaker_embed: Optional[Callable] = None, mos: Optional[MosPredictorWrapper] = None, fcd: Optional[FrechetCodecDistance] = None,
                 **tts_kwargs) -> Dict[str, float]:
    """``items``: dicts with ``text`` and optionally ``audio`` (reference waveform, 1-D tensor) for similarity / FCD."""
    rtf = RTFMetrics(sample_rate)
    gen, texts, sims = [], [], []
    for it in items:
        audio, alen = rtf.timed(model.do_tts, it["text"], **tts_kwargs)
        wav = audio[0, : int(alen[0])].detach().float().cpu()
        rtf.add_audio(wav.numel())
        gen.append(wav)
        texts.append(it["text"])
        ref = it.get("audio")
        if ref is not None and speaker_embed is not None:
            sims.append(float(speaker_similarity(speaker_embed, wav[None], torch.tensor([wav.numel()]), ref[None], torch.tensor([ref.numel()]))[0]))
        if ref is not None and fcd is not None and fcd.codec is not None:
            fcd.update(real_audio=(ref[None], torch.tensor([ref.numel()])), fake_audio=(wav[None], torch.tensor([wav.numel()])))
    res: Dict[str, float] = dict(rtf.compute())
    if transcribe is not None:
        res.update(intelligibility(transcribe, gen, texts))
    if sims:
        res["speaker_similarity"] = sum(sims) / len(sims)
    if mos is not None:
        scores = mos(gen)
        res["mos"] = sum(scores) / max(1, len(scores))
    if fcd is not None and fcd.real.n >= 2 and fcd.fake.n >= 2:
        res["frechet_codec_distance"] = fcd.compute()
    return res

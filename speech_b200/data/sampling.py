"""Sampling constraints and example filters of the cut pipeline.

Constraints decide when a mini-batch is full; filters decide which examples are kept.  Both see audio cuts and text /
conversation examples alike: audio length is converted to tokens with ``token_equivalent_duration`` (seconds of audio
that one token is worth, normally frame shift x subsampling factor of the audio encoder).  Names and semantics follow
``common/data/lhotse/sampling.py`` (``MultimodalSamplingConstraint`` :30, ``FixedBucketBatchSizeConstraint2D`` :109,
``find_smallest_bucket`` :152, ``MultimodalFixedBucketBatchSizeConstraint2D`` :208, the filters :249-433).
"""
from __future__ import annotations

import math
from bisect import bisect_left
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence, Tuple, Union

import numpy as np

from .sources import measure_tokens


def _is_audio(ex) -> bool:
    return ex.custom.get("kind") is None


@dataclass
class TokenConstraint:
    """A batch is full when it holds ``max_examples`` examples or when ``longest length x count`` (the padded size) would
    exceed ``max_tokens``.  ``quadratic_length`` adds ``len**2 / quadratic_length`` to each example's length, which
    penalises long examples the way attention memory grows."""

    max_tokens: Optional[float] = None
    max_examples: Optional[int] = None
    quadratic_length: Optional[float] = None
    _longest: float = 0.0
    _count: int = 0

    def _effective(self, n: float) -> float:
        return n + n * n / self.quadratic_length if self.quadratic_length else n

    def add_length(self, n: float) -> None:
        self._longest = max(self._longest, self._effective(n))
        self._count += 1

    def exceeded(self) -> bool:
        if self.max_examples is not None and self._count > self.max_examples:
            return True
        return self.max_tokens is not None and self._longest * self._count > self.max_tokens

    def close_to_exceeding(self) -> bool:
        if self.max_examples is not None and self._count >= self.max_examples:
            return True
        return self.max_tokens is not None and self._longest * (self._count + 1) > self.max_tokens

    def reset(self) -> None:
        self._longest, self._count = 0.0, 0


@dataclass
class MultimodalSamplingConstraint:
    """Measures every example in tokens.  ``measure_total_length`` counts input + output (decoder-only models); otherwise
    only the input side (audio frames of a cut, context tokens of a text example)."""

    token_equivalent_duration: Optional[float] = None
    batch_size: Optional[int] = None
    batch_tokens: Optional[int] = None
    quadratic_factor: Optional[float] = None
    measure_total_length: bool = False
    tokenizer: Any = None
    _internal: TokenConstraint = field(default=None, repr=False)

    def __post_init__(self):
        self._internal = TokenConstraint(self.batch_tokens, self.batch_size, self.quadratic_factor)

    def measure_length(self, ex) -> float:
        i, o = measure_tokens(ex, self.tokenizer, self.token_equivalent_duration)
        return float(i + o) if self.measure_total_length else float(i)

    def add(self, ex) -> None:
        n = self.measure_length(ex)
        ex.custom["num_tokens"] = n
        self._internal.add_length(n)

    def exceeded(self) -> bool:
        return self._internal.exceeded()

    def close_to_exceeding(self) -> bool:
        return self._internal.close_to_exceeding()

    def reset(self) -> None:
        self._internal.reset()


def find_smallest_bucket(buckets, example_lens, strict: bool = True, max_ratio: Optional[Sequence[float]] = None) -> Optional[int]:
    """Index of the smallest bucket that holds the example, or ``None``.  1-D: ``buckets`` are ascending upper bounds.  2-D:
    ``buckets`` are ``(dim0, dim1)`` rows sorted ascending; *strict* looks only at the rows that share the first ``dim0``
    bound that fits (so an example with an unusually long second dimension is rejected rather than sent to a much larger
    bucket); lenient takes the first row that fits both.  ``max_ratio[i]`` bounds ``len1 / len0`` inside bucket ``i``."""
    if isinstance(example_lens, (int, float)):
        idx = bisect_left(list(buckets), example_lens)
        return None if idx == len(buckets) else idx
    b = np.asarray(buckets, dtype=np.float64)
    l0, l1 = float(example_lens[0]), float(example_lens[1])
    if strict:
        lo = bisect_left(b[:, 0].tolist(), l0)
        if lo == len(b):
            return None
        hi = lo
        while hi < len(b) and b[hi, 0] == b[lo, 0]:
            hi += 1
        j = bisect_left(b[lo:hi, 1].tolist(), l1)
        if j == hi - lo:
            return None
        fit = lo + j
        if max_ratio is not None and l0 > 0 and l1 / l0 > max_ratio[fit]:
            return None
        return fit
    ok = np.nonzero((l0 <= b[:, 0]) & (l1 <= b[:, 1]))[0]
    return int(ok[0]) if len(ok) else None


@dataclass
class FixedBucketBatchSizeConstraint2D:
    """Every bucket has its own fixed batch size.  Buckets are upper bounds on duration (1-D) or on (duration, number of
    output tokens) (2-D).  ``max_ratio`` optionally bounds tokens-per-second per bucket."""

    max_seq_len_buckets: Sequence[Union[float, Sequence[float]]]
    batch_sizes: Sequence[int]
    strict_2d: bool = True
    max_ratio: Optional[Sequence[float]] = None
    tokenizer: Any = None
    current_bucket: Optional[int] = None
    num_cuts: int = 0

    def __post_init__(self):
        if len(self.max_seq_len_buckets) != len(self.batch_sizes):
            raise ValueError("one batch size per bucket is required")
        if list(self.max_seq_len_buckets) != sorted(self.max_seq_len_buckets):
            raise ValueError("buckets must be sorted ascending")
        if self.max_ratio is not None and len(self.max_ratio) != len(self.max_seq_len_buckets):
            raise ValueError("one max_ratio per bucket is required")

    @property
    def bucketing_2d_enabled(self) -> bool:
        return isinstance(self.max_seq_len_buckets[0], Sequence) and len(self.max_seq_len_buckets[0]) == 2

    def measure_length(self, ex) -> Union[float, Tuple[float, float]]:
        if self.bucketing_2d_enabled:
            return ex.duration, float(measure_tokens(ex, self.tokenizer)[1])
        return ex.duration

    def select_bucket(self, ex=None, example_len=None) -> Optional[int]:
        if example_len is None:
            example_len = self.measure_length(ex)
        return find_smallest_bucket(self.max_seq_len_buckets, example_len, self.strict_2d, self.max_ratio)

    def add(self, ex) -> None:
        if self.current_bucket is None:
            self.current_bucket = self.select_bucket(ex)
        self.num_cuts += 1

    def exceeded(self) -> bool:
        return self.current_bucket is not None and self.num_cuts > self.batch_sizes[self.current_bucket]

    def close_to_exceeding(self) -> bool:
        return self.current_bucket is not None and self.num_cuts >= self.batch_sizes[self.current_bucket]

    def reset(self) -> None:
        self.current_bucket, self.num_cuts = None, 0


@dataclass
class MultimodalFixedBucketBatchSizeConstraint2D(FixedBucketBatchSizeConstraint2D):
    """Fixed batch size per bucket with lengths in tokens: 2-D buckets bound (input tokens, output tokens); 1-D buckets bound
    the input (or total, with ``measure_total_length``) token count."""

    token_equivalent_duration: Optional[float] = None
    measure_total_length: bool = False

    def measure_length(self, ex):
        i, o = measure_tokens(ex, self.tokenizer, self.token_equivalent_duration)
        if self.bucketing_2d_enabled:
            return float(i), float(o)
        return float(i + o) if self.measure_total_length else float(i)


# ------------------------------------------------------------------------------------------ filters
class DurationFilter:
    """Keeps audio examples with ``d_min <= duration <= d_max``; examples without audio pass."""

    def __init__(self, d_min: Optional[float], d_max: Optional[float]):
        self.d_min = -math.inf if d_min is None else d_min
        self.d_max = math.inf if d_max is None else d_max

    def __call__(self, ex) -> bool:
        return self.d_min <= ex.duration <= self.d_max if _is_audio(ex) else True


class ValidationStatusFilter:
    """Keeps cuts whose ``validation_status`` custom field equals ``keep`` (cuts without the field pass)."""

    def __init__(self, keep: str = "pass"):
        self.keep = keep

    def __call__(self, ex) -> bool:
        v = ex.custom.get("validation_status")
        return v is None or v == self.keep


class CERFilter:
    """Drops cuts whose recorded character error rate (``cer`` custom field, e.g. of pseudo-labels) exceeds ``max_cer``."""

    def __init__(self, max_cer: Optional[float]):
        self.max_cer = math.inf if max_cer is None else max_cer

    def __call__(self, ex) -> bool:
        v = ex.custom.get("cer")
        return v is None or float(v) <= self.max_cer


class ContextSpeakerSimilarityFilter:
    """TTS: keeps cuts whose context audio is close enough to the target speaker (``context_speaker_similarity`` field)."""

    def __init__(self, min_context_speaker_similarity: Optional[float]):
        self.min_sim = -math.inf if min_context_speaker_similarity is None else min_context_speaker_similarity

    def __call__(self, ex) -> bool:
        v = ex.custom.get("context_speaker_similarity")
        return v is None or float(v) >= self.min_sim


class TokenCountFilter:
    """Keeps examples whose token count (input, or input + output with ``measure_total_length``) lies in ``[t_min, t_max]``."""

    def __init__(self, t_min: Optional[float], t_max: Optional[float], measure_total_length: bool = False, tokenizer=None,
                 token_equivalent_duration: Optional[float] = None):
        self.t_min = -math.inf if t_min is None else t_min
        self.t_max = math.inf if t_max is None else t_max
        self.total, self.tokenizer, self.ted = measure_total_length, tokenizer, token_equivalent_duration
        self.enabled = t_min is not None or t_max is not None

    def __call__(self, ex) -> bool:
        if not self.enabled:
            return True
        i, o = measure_tokens(ex, self.tokenizer, self.ted)
        return self.t_min <= (i + o if self.total else i) <= self.t_max


class TokenPerSecondFilter:
    """Audio cuts only: output tokens per second of audio within ``[tps_min, tps_max]`` (catches bad transcripts)."""

    def __init__(self, tps_min: Optional[float], tps_max: Optional[float], tokenizer=None):
        self.lo = -math.inf if tps_min is None else tps_min
        self.hi = math.inf if tps_max is None else tps_max
        if self.lo > self.hi:
            raise ValueError("tps_min must not exceed tps_max")
        self.tokenizer = tokenizer
        self.enabled = tps_min is not None or tps_max is not None

    def __call__(self, ex) -> bool:
        if not self.enabled or not _is_audio(ex) or ex.duration <= 0:
            return True
        return self.lo <= measure_tokens(ex, self.tokenizer)[1] / ex.duration <= self.hi


class TokenPerTokenFilter:
    """Text examples only: output tokens per input token within ``[tpt_min, tpt_max]``."""

    def __init__(self, tpt_min: Optional[float], tpt_max: Optional[float], tokenizer=None):
        self.lo = -math.inf if tpt_min is None else tpt_min
        self.hi = math.inf if tpt_max is None else tpt_max
        if self.lo > self.hi:
            raise ValueError("tpt_min must not exceed tpt_max")
        self.tokenizer = tokenizer
        self.enabled = tpt_min is not None or tpt_max is not None

    def __call__(self, ex) -> bool:
        if not self.enabled or _is_audio(ex):
            return True
        i, o = measure_tokens(ex, self.tokenizer)
        return i > 0 and self.lo <= o / i <= self.hi


class BucketingFilter:
    """Drops examples that fit no bucket of a fixed-bucket constraint (they could never be batched)."""

    def __init__(self, constraint):
        self.constraint = constraint

    def __call__(self, ex) -> bool:
        if not isinstance(self.constraint, FixedBucketBatchSizeConstraint2D):
            return True
        return self.constraint.select_bucket(ex) is not None


def batches_from_constraint(examples: Sequence[Any], constraint, drop_last: bool = False) -> List[List[int]]:
    """Greedy batching of ``examples`` in the given order under any constraint above: a batch closes as soon as adding the
    next example would exceed it."""
    out: List[List[int]] = []
    cur: List[int] = []
    constraint.reset()
    for i, ex in enumerate(examples):
        constraint.add(ex)
        if constraint.exceeded() and cur:
            out.append(cur)
            cur = []
            constraint.reset()
            constraint.add(ex)
        cur.append(i)
        if constraint.close_to_exceeding():
            out.append(cur)
            cur = []
            constraint.reset()
    if cur and not drop_last:
        out.append(cur)
    return out

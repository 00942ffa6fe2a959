"""Option names of the streaming inference pipelines as enumerations that parse from config strings (case-insensitive, by member name or value).
Reference: ``asr/inference/utils/enums.py``.
"""
from __future__ import annotations

from enum import Enum, auto

from .framing import RequestType  # noqa: F401  (re-exported: frames of audio vs buffers of features)


class StrEnumMixin:
    @classmethod
    def from_str(cls, name: str):
        key = str(name).lower()
        for m in cls:
            if m.name.lower() == key or str(m.value).lower() == key:
                return m
        raise ValueError(f"Invalid {cls.__name__} `{name}`: must be one of {[m.name.lower() for m in cls]}")


class ASRDecodingType(StrEnumMixin, Enum):
    CTC = auto()
    RNNT = auto()
    SALM = auto()


class ASROutputGranularity(StrEnumMixin, Enum):
    WORD = auto()
    SEGMENT = auto()


class PipelineType(StrEnumMixin, Enum):
    BUFFERED = auto()
    CACHE_AWARE = auto()


class FeatureBufferPaddingMode(StrEnumMixin, Enum):
    LEFT = auto()
    RIGHT = auto()


class MergingStrategy(StrEnumMixin, Enum):
    LCS = auto()            # longest common subsequence between the tails of consecutive windows
    LCSUBSTR = auto()       # longest common substring

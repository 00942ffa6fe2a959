"""Neural types: semantic tags on module inputs and outputs, with a comparison lattice.

Covers the reference's ``NeuralType(axes, elements_type, optional)`` model
(``nemo/core/neural_types/neural_type.py:31``), its axis kinds (``axes.py:30-47``), the element
type hierarchy (``elements.py``) and the ``@typecheck`` decorator with global enable /
disable contexts (``nemo/core/classes/common.py:1234,1374-1420``).
"""
from __future__ import annotations

import contextlib
import enum
import functools
import threading
from typing import Any, Dict, Optional, Tuple


class NeuralTypeComparisonResult(enum.Enum):
    SAME = 0
    LESS = 1
    GREATER = 2
    DIM_INCOMPATIBLE = 3
    TRANSPOSE_SAME = 4
    CONTAINER_SIZE_MISMATCH = 5
    INCOMPATIBLE = 6
    SAME_TYPE_INCOMPATIBLE_PARAMS = 7
    UNCHECKED = 8


class AxisKind(enum.Enum):
    Batch = 0
    Time = 1
    Dimension = 2
    Channel = 3
    Width = 4
    Height = 5
    Any = 6
    Sequence = 7
    FlowGroup = 8
    Singleton = 9

    @staticmethod
    def from_str(label: str) -> "AxisKind":
        m = {"b": AxisKind.Batch, "t": AxisKind.Time, "time": AxisKind.Time, "d": AxisKind.Dimension,
             "c": AxisKind.Channel, "w": AxisKind.Width, "h": AxisKind.Height, "s": AxisKind.Sequence,
             "flowgroup": AxisKind.FlowGroup, "singleton": AxisKind.Singleton, "any": AxisKind.Any}
        key = label.lower().strip()
        if key not in m:
            raise ValueError(f"Cannot parse axis kind '{label}'")
        return m[key]


class AxisType:
    def __init__(self, kind: AxisKind, size: Optional[int] = None, is_list: bool = False):
        self.kind, self.size, self.is_list = kind, size, is_list

    def __repr__(self):
        return f"AxisType({self.kind.name}, size={self.size}, is_list={self.is_list})"


class ElementType:
    """Base of the element-type hierarchy; subclass relation defines LESS/GREATER."""

    type_parameters: Dict[str, Any] = {}
    fields: Optional[Tuple[str, ...]] = None

    def __str__(self):
        return self.__class__.__name__

    __repr__ = __str__

    def compare(self, second: "ElementType") -> NeuralTypeComparisonResult:
        a, b = type(self), type(second)
        if a is b:
            if self.type_parameters == second.type_parameters:
                return NeuralTypeComparisonResult.SAME
            return NeuralTypeComparisonResult.SAME_TYPE_INCOMPATIBLE_PARAMS
        if issubclass(a, b):
            return NeuralTypeComparisonResult.LESS
        if issubclass(b, a):
            return NeuralTypeComparisonResult.GREATER
        return NeuralTypeComparisonResult.INCOMPATIBLE


def _mk(name: str, base: type = ElementType, doc: str = "") -> type:
    return type(name, (base,), {"__doc__": doc or name})


VoidType = _mk("VoidType", doc="Matches anything; compare() always returns SAME.")
VoidType.compare = lambda self, second: NeuralTypeComparisonResult.SAME  # type: ignore
ChannelType = _mk("ChannelType")
EmbeddedTextType = _mk("EmbeddedTextType", ChannelType)
LogitsType = _mk("LogitsType")
ProbsType = _mk("ProbsType")
LogprobsType = _mk("LogprobsType")
LossType = _mk("LossType")
RegressionValuesType = _mk("RegressionValuesType")
CategoricalValuesType = _mk("CategoricalValuesType")
PredictionsType = _mk("PredictionsType")
LabelsType = _mk("LabelsType")
HypothesisType = _mk("HypothesisType", LabelsType)
LengthsType = _mk("LengthsType")
MaskType = _mk("MaskType", PredictionsType)
Target = _mk("Target")
ClassificationTarget = _mk("ClassificationTarget", Target)
ImageValue = _mk("ImageValue")
NormalizedImageValue = _mk("NormalizedImageValue", ImageValue)
ImageFeatureValue = _mk("ImageFeatureValue", ImageValue)
StringLabel = _mk("StringLabel", LabelsType)
StringType = _mk("StringType")
TokenIndex = _mk("TokenIndex")
Length = _mk("Length")
IntType = _mk("IntType")
FloatType = _mk("FloatType")
BoolType = _mk("BoolType")
NormalDistributionSamplesType = _mk("NormalDistributionSamplesType")
NormalDistributionMeanType = _mk("NormalDistributionMeanType")
NormalDistributionLogVarianceType = _mk("NormalDistributionLogVarianceType")
SequenceToSequenceAlignmentType = _mk("SequenceToSequenceAlignmentType")
TokenDurationType = _mk("TokenDurationType")
TokenLogDurationType = _mk("TokenLogDurationType")
LogDeterminantType = _mk("LogDeterminantType")
ProbabilityDistributionSamplesType = _mk("ProbabilityDistributionSamplesType")


class AudioSignal(ElementType):
    """Waveform; two signals are only the same type if their sample rates agree."""

    def __init__(self, freq: Optional[int] = None):
        self._params = {"freq": freq}

    @property
    def type_parameters(self):  # type: ignore[override]
        return self._params


SpectrogramType = _mk("SpectrogramType", ChannelType)
MelSpectrogramType = _mk("MelSpectrogramType", SpectrogramType)
MFCCSpectrogramType = _mk("MFCCSpectrogramType", SpectrogramType)
EncodedRepresentation = _mk("EncodedRepresentation", ChannelType)
AcousticEncodedRepresentation = _mk("AcousticEncodedRepresentation", EncodedRepresentation)
AudioEncodedRepresentation = _mk("AudioEncodedRepresentation", EncodedRepresentation)
TextEncodedRepresentation = _mk("TextEncodedRepresentation", EncodedRepresentation)
ImageEncodedRepresentation = _mk("ImageEncodedRepresentation", EncodedRepresentation)
SpeakerEmbeddingType = _mk("SpeakerEmbeddingType", EncodedRepresentation)


class NeuralType:
    def __init__(self, axes: Optional[Tuple] = None, elements_type: Optional[ElementType] = None, optional=False):
        if elements_type is None:
            elements_type = VoidType()
        if not isinstance(elements_type, ElementType):
            raise ValueError("elements_type must be an ElementType instance (did you forget the parentheses?)")
        self.elements_type = elements_type
        self.optional = optional
        if axes is not None:
            parsed = []
            for ax in axes:
                if isinstance(ax, str):
                    parsed.append(AxisType(AxisKind.from_str(ax)))
                elif isinstance(ax, AxisType):
                    parsed.append(ax)
                elif isinstance(ax, AxisKind):
                    parsed.append(AxisType(ax))
                else:
                    raise ValueError(f"Axis must be str, AxisKind or AxisType, got {type(ax)}")
            self.axes: Optional[Tuple[AxisType, ...]] = tuple(parsed)
        else:
            self.axes = None

    def compare(self, second: "NeuralType") -> NeuralTypeComparisonResult:
        if self.axes is None:
            if isinstance(self.elements_type, VoidType):
                return NeuralTypeComparisonResult.SAME
            return self.elements_type.compare(second.elements_type) if second.axes is None \
                else NeuralTypeComparisonResult.INCOMPATIBLE
        dim = self._compare_axes(second.axes)
        el = self.elements_type.compare(second.elements_type)
        if dim == 0:
            return el
        if dim == 1 and el == NeuralTypeComparisonResult.SAME:
            return NeuralTypeComparisonResult.TRANSPOSE_SAME
        if dim == 1:
            return NeuralTypeComparisonResult.INCOMPATIBLE
        if dim == 2:
            return NeuralTypeComparisonResult.DIM_INCOMPATIBLE
        return NeuralTypeComparisonResult.INCOMPATIBLE

    def _compare_axes(self, other) -> int:
        """0 same, 1 same up to a permutation, 2 size mismatch, 3 incompatible."""
        if self.axes is None and other is None:
            return 0
        if self.axes is None or other is None or len(self.axes) != len(other):
            return 3
        if len(self.axes) == 1 and self.axes[0].kind == AxisKind.Any:
            return 0
        same = True
        kinds_a: Dict[AxisKind, Optional[int]] = {}
        kinds_b: Dict[AxisKind, Optional[int]] = {}
        for a, b in zip(self.axes, other):
            kinds_a[a.kind] = a.size
            kinds_b[b.kind] = b.size
            if a.kind == AxisKind.Any or b.kind == AxisKind.Any:
                continue
            if a.kind != b.kind or a.is_list != b.is_list:
                same = False
            elif a.size != b.size and a.size is not None and b.size is not None:
                return 2
        if same:
            return 0
        if kinds_a.keys() == kinds_b.keys():
            for k in kinds_a:
                if kinds_a[k] != kinds_b[k] and kinds_a[k] is not None and kinds_b[k] is not None:
                    return 2
            return 1
        return 3

    def compare_and_raise_error(self, parent_type_name, port_name, second_object):
        res = self.compare(second_object)
        if res not in (NeuralTypeComparisonResult.SAME, NeuralTypeComparisonResult.GREATER):
            raise NeuralPortNmTensorMismatchError(parent_type_name, port_name, str(self), str(second_object), res)

    def __eq__(self, other):
        return isinstance(other, NeuralType) and self.compare(other) == NeuralTypeComparisonResult.SAME

    def __hash__(self):
        return hash(str(self))

    def __repr__(self):
        axes = None if self.axes is None else tuple(a.kind.name for a in self.axes)
        return f"NeuralType(axes={axes}, elements_type={self.elements_type}, optional={self.optional})"


class NeuralTypeError(Exception):
    pass


class NeuralPortNmTensorMismatchError(NeuralTypeError):
    def __init__(self, class_name, port_name, first_type, second_type, type_comatibility):
        super().__init__(
            f"\nIn {class_name}. \nPort: {port_name} and a tensor passed to it are of incompatible neural types:\n"
            f"\n{first_type} \n\n and \n\n{second_type}\n\nType comparison result: {type_comatibility}"
        )


_TYPECHECK_STATE = threading.local()


def is_typecheck_enabled() -> bool:
    return getattr(_TYPECHECK_STATE, "enabled", True)


class typecheck:
    """Decorator for ``forward``: keyword-only call convention plus input/output neural type checks.

    Tensor *rank* is checked against the declared axes, ``None`` is accepted for optional ports,
    and each returned tensor is tagged with ``.neural_type``.
    """

    def __init__(self, input_types=None, output_types=None, ignore_collections: bool = False):
        self.input_types, self.output_types = input_types, output_types

    def __call__(self, fn):
        @functools.wraps(fn)
        def wrapped(module, *args, **kwargs):
            if not is_typecheck_enabled():
                return fn(module, *args, **kwargs)
            in_types = self.input_types if self.input_types is not None else getattr(module, "input_types", None)
            out_types = self.output_types if self.output_types is not None else getattr(module, "output_types", None)
            if in_types is None and out_types is None:
                return fn(module, *args, **kwargs)
            if in_types is not None:
                if args:
                    raise TypeError("All arguments must be passed by kwargs only for typed methods")
                _validate_inputs(module, in_types, kwargs)
            out = fn(module, **kwargs) if in_types is not None else fn(module, *args, **kwargs)
            if out_types is not None:
                _attach_outputs(module, out_types, out)
            return out

        wrapped.__wrapped__ = fn
        return wrapped

    @staticmethod
    def set_typecheck_enabled(enabled: bool = True):
        _TYPECHECK_STATE.enabled = enabled

    @staticmethod
    @contextlib.contextmanager
    def disable_checks():
        prev = is_typecheck_enabled()
        _TYPECHECK_STATE.enabled = False
        try:
            yield
        finally:
            _TYPECHECK_STATE.enabled = prev

    @staticmethod
    @contextlib.contextmanager
    def disable_semantic_checks():
        prev = getattr(_TYPECHECK_STATE, "semantic", True)
        _TYPECHECK_STATE.semantic = False
        try:
            yield
        finally:
            _TYPECHECK_STATE.semantic = prev


def _validate_inputs(module, in_types, kwargs):
    name = type(module).__name__
    mandatory = [k for k, t in in_types.items() if not t.optional]
    for k in mandatory:
        if k not in kwargs:
            raise TypeError(f"{name}: missing mandatory typed input '{k}' (expected {list(in_types)})")
    for k, v in kwargs.items():
        if k not in in_types:
            raise TypeError(f"{name}: input argument '{k}' has no corresponding input_type; known: {list(in_types)}")
        t = in_types[k]
        if v is None:
            if not t.optional:
                raise TypeError(f"{name}: input '{k}' is not optional but None was passed")
            continue
        if getattr(_TYPECHECK_STATE, "semantic", True) and hasattr(v, "neural_type"):
            t.compare_and_raise_error(name, k, v.neural_type)
        if hasattr(v, "shape") and t.axes is not None:
            if not (len(t.axes) == 1 and t.axes[0].kind == AxisKind.Any) and len(v.shape) != len(t.axes):
                raise TypeError(
                    f"{name}: input '{k}' has shape {tuple(v.shape)} but its neural type declares "
                    f"{len(t.axes)} axes {tuple(a.kind.name for a in t.axes)}"
                )


def _attach_outputs(module, out_types, out):
    types = list(out_types.items())
    seq = out if isinstance(out, (tuple, list)) else (out,)
    if len(types) == 1 and isinstance(out, (tuple, list)) and not hasattr(out, "shape"):
        return
    for (pname, t), v in zip(types, seq):
        if hasattr(v, "shape"):
            try:
                v.neural_type = t
            except Exception:
                pass

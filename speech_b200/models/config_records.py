"""Typed config records of the ASR collection's models and pipelines: the offline diarizer (VAD, multi-scale speaker embeddings,
clustering, ASR options) with an inference preset, dataset / model records of the CTC and classification models, the MatchboxNet
presets, and a builder that keeps the interdependent fields of a classification model config consistent (labels ↔ decoder classes,
sample rate ↔ front end ↔ datasets, encoder width ↔ decoder input).
Reference: ``asr/models/configs/diarizer_config.py``, ``asr_models_config.py``, ``classification_models_config.py``, ``matchboxnet_config.py``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

from ..core import config_schemas as S
from ..modules import configs as M


# -------------------------------------------------------------------------------------------------------------- diarization
@dataclass
class DiarizerComponentConfig:
    def get(self, name: str, default: Any = None):
        return getattr(self, name, default)

    def __iter__(self):
        return iter(asdict(self))

    def dict(self) -> Dict[str, Any]:
        return asdict(self)


@dataclass
class ASRDiarizerParams(DiarizerComponentConfig):
    asr_based_vad: bool = False                          # speech / non-speech from the ASR word timestamps instead of a VAD model
    asr_based_vad_threshold: float = 1.0                  # silences up to this many seconds between words stay inside one speech segment
    asr_batch_size: Optional[int] = None
    decoder_delay_in_sec: Optional[float] = None          # constant latency of the decoder to subtract from word times
    word_ts_anchor_offset: Optional[float] = None
    word_ts_anchor_pos: str = "start"                     # start | end | mid: the point of a word that is matched against speaker segments
    fix_word_ts_with_VAD: bool = False
    colored_text: bool = False
    print_time: bool = True
    break_lines: bool = False


@dataclass
class ASRDiarizerConfig(DiarizerComponentConfig):
    model_path: Optional[str] = "stt_en_conformer_ctc_large"
    parameters: ASRDiarizerParams = field(default_factory=ASRDiarizerParams)


@dataclass
class VADParams(DiarizerComponentConfig):
    window_length_in_sec: float = 0.15
    shift_length_in_sec: float = 0.01
    smoothing: Union[str, bool] = "median"
    overlap: float = 0.5
    onset: float = 0.1
    offset: float = 0.1
    pad_onset: float = 0.1
    pad_offset: float = 0
    min_duration_on: float = 0
    min_duration_off: float = 0.2
    filter_speech_first: bool = True


@dataclass
class VADConfig(DiarizerComponentConfig):
    model_path: str = "vad_multilingual_marblenet"
    external_vad_manifest: Optional[str] = None
    parameters: VADParams = field(default_factory=VADParams)


@dataclass
class SpeakerEmbeddingsParams(DiarizerComponentConfig):
    window_length_in_sec: Tuple[float, ...] = (1.5, 1.25, 1.0, 0.75, 0.5)
    shift_length_in_sec: Tuple[float, ...] = (0.75, 0.625, 0.5, 0.375, 0.25)
    multiscale_weights: Tuple[float, ...] = (1, 1, 1, 1, 1)
    save_embeddings: bool = True


@dataclass
class SpeakerEmbeddingsConfig(DiarizerComponentConfig):
    model_path: Optional[str] = None
    parameters: SpeakerEmbeddingsParams = field(default_factory=SpeakerEmbeddingsParams)


@dataclass
class ClusteringParams(DiarizerComponentConfig):
    oracle_num_speakers: bool = False
    max_num_speakers: int = 8
    enhanced_count_thres: int = 80
    max_rp_threshold: float = 0.25
    sparse_search_volume: int = 30
    maj_vote_spk_count: bool = False
    chunk_cluster_count: int = 50                         # long-form clustering: clusters kept per chunk
    embeddings_per_chunk: int = 10000                      # long-form clustering: embeddings per chunk


@dataclass
class ClusteringConfig(DiarizerComponentConfig):
    parameters: ClusteringParams = field(default_factory=ClusteringParams)


@dataclass
class DiarizerConfig(DiarizerComponentConfig):
    manifest_filepath: Optional[str] = None
    out_dir: Optional[str] = None
    oracle_vad: bool = False
    collar: float = 0.25
    ignore_overlap: bool = True
    vad: VADConfig = field(default_factory=VADConfig)
    speaker_embeddings: SpeakerEmbeddingsConfig = field(default_factory=SpeakerEmbeddingsConfig)
    clustering: ClusteringConfig = field(default_factory=ClusteringConfig)
    asr: ASRDiarizerConfig = field(default_factory=ASRDiarizerConfig)


@dataclass
class NeuralDiarizerInferenceConfig(DiarizerComponentConfig):
    diarizer: DiarizerConfig = field(default_factory=DiarizerConfig)
    device: str = "cpu"
    verbose: bool = False
    batch_size: int = 64
    num_workers: int = 1
    sample_rate: int = 16000
    name: str = ""

    @classmethod
    def init_config(cls, diar_model_path: str, vad_model_path: str, map_location: str = "cpu", verbose: bool = False) -> "NeuralDiarizerInferenceConfig":
        """The preset an inference script starts from: speaker model and VAD model paths filled in, telephonic-style VAD thresholds."""
        return cls(DiarizerConfig(vad=VADConfig(model_path=vad_model_path), speaker_embeddings=SpeakerEmbeddingsConfig(model_path=diar_model_path)),
                   device=map_location, verbose=verbose)

    def to_dictconfig(self):
        return S.to_dictconfig(self)


# ------------------------------------------------------------------------------------------------------------------ ASR models
@dataclass
class ASRDatasetConfig(S.DatasetConfig):
    manifest_filepath: Optional[Any] = None
    sample_rate: int = S.MISSING
    labels: Any = S.MISSING
    trim_silence: bool = False
    is_tarred: bool = False
    tarred_audio_filepaths: Optional[Any] = None
    tarred_shard_strategy: str = "scatter"
    shard_manifests: bool = False
    shuffle_n: int = 0
    use_lhotse: bool = False
    use_start_end_token: bool = True
    return_sample_id: Optional[bool] = False
    int_values: bool = False
    augmentor: Optional[Dict[str, Any]] = None
    max_duration: Optional[float] = None
    min_duration: Optional[float] = None
    max_utts: int = 0
    blank_index: int = -1
    unk_index: int = -1
    normalize: bool = False
    trim: bool = True
    parser: Optional[str] = "en"
    eos_id: Optional[int] = None
    bos_id: Optional[int] = None
    pad_id: int = 0
    bucketing_strategy: str = "synced_randomized"
    bucketing_batch_size: Optional[Any] = None
    bucketing_weights: Optional[List[int]] = None
    channel_selector: Optional[Any] = None


@dataclass
class EncDecCTCConfig(S.ModelConfig):
    sample_rate: int = 16000
    repeat: int = 1
    dropout: float = 0.0
    separable: bool = False
    labels: Any = S.MISSING
    train_ds: ASRDatasetConfig = field(default_factory=lambda: ASRDatasetConfig(manifest_filepath=None, shuffle=True))
    validation_ds: ASRDatasetConfig = field(default_factory=lambda: ASRDatasetConfig(manifest_filepath=None, shuffle=False))
    test_ds: ASRDatasetConfig = field(default_factory=lambda: ASRDatasetConfig(manifest_filepath=None, shuffle=False))
    optim: Optional[S.OptimConfig] = field(default_factory=lambda: S.OptimConfig(name="novograd", sched=S.SchedConfig(name="CosineAnnealing")))
    preprocessor: M.AudioToMelSpectrogramPreprocessorConfig = field(default_factory=M.AudioToMelSpectrogramPreprocessorConfig)
    spec_augment: Optional[M.SpectrogramAugmentationConfig] = field(default_factory=M.SpectrogramAugmentationConfig)
    encoder: Dict[str, Any] = field(default_factory=dict)
    decoder: Dict[str, Any] = field(default_factory=dict)
    decoding: Dict[str, Any] = field(default_factory=lambda: {"strategy": "greedy_batch"})


@dataclass
class EncDecCTCModelConfig(S.NemoConfig):
    model: EncDecCTCConfig = field(default_factory=EncDecCTCConfig)


# ------------------------------------------------------------------------------------------------------- classification models
@dataclass
class EncDecClassificationDatasetConfig(S.DatasetConfig):
    manifest_filepath: Optional[str] = None
    sample_rate: int = S.MISSING
    labels: Any = S.MISSING
    trim_silence: bool = False
    is_tarred: bool = False
    tarred_audio_filepaths: Optional[str] = None
    tarred_shard_strategy: str = "scatter"
    shuffle_n: int = 0
    int_values: bool = False
    augmentor: Optional[Dict[str, Any]] = None
    max_duration: Optional[float] = None
    min_duration: Optional[float] = None
    cal_labels_occurrence: Optional[bool] = False
    channel_selector: Optional[Any] = None
    vad_stream: bool = False
    window_length_in_sec: float = 0.31
    shift_length_in_sec: float = 0.01
    normalize_audio: bool = False
    is_regression_task: bool = False
    bucketing_strategy: str = "synced_randomized"
    bucketing_batch_size: Optional[Any] = None
    bucketing_weights: Optional[List[int]] = None


@dataclass
class EncDecClassificationConfig(S.ModelConfig):
    sample_rate: int = 16000
    repeat: int = 1
    dropout: float = 0.0
    separable: bool = True
    kernel_size_factor: float = 1.0
    labels: Any = S.MISSING
    timesteps: int = S.MISSING
    train_ds: EncDecClassificationDatasetConfig = field(default_factory=lambda: EncDecClassificationDatasetConfig(shuffle=True, trim_silence=False))
    validation_ds: EncDecClassificationDatasetConfig = field(default_factory=lambda: EncDecClassificationDatasetConfig(shuffle=False))
    test_ds: EncDecClassificationDatasetConfig = field(default_factory=lambda: EncDecClassificationDatasetConfig(shuffle=False))
    optim: Optional[S.OptimConfig] = field(default_factory=lambda: S.OptimConfig(name="novograd", sched=S.SchedConfig(name="CosineAnnealing")))
    preprocessor: Any = field(default_factory=lambda: M.AudioToMFCCPreprocessorConfig())
    spec_augment: Optional[M.SpectrogramAugmentationConfig] = field(default_factory=M.SpectrogramAugmentationConfig)
    crop_or_pad_augment: Optional[M.CropOrPadSpectrogramAugmentationConfig] = field(default_factory=lambda: M.CropOrPadSpectrogramAugmentationConfig(audio_length=-1))
    encoder: Dict[str, Any] = field(default_factory=dict)
    decoder: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.crop_or_pad_augment is not None and self.crop_or_pad_augment.audio_length < 0 and self.timesteps != S.MISSING:
            self.crop_or_pad_augment.audio_length = self.timesteps


@dataclass
class EncDecClassificationModelConfig(S.NemoConfig):
    model: EncDecClassificationConfig = field(default_factory=EncDecClassificationConfig)


def _block(filters, repeat, kernel, stride=1, dilation=1, dropout=0.0, residual=False, separable=False) -> Dict[str, Any]:
    return dict(filters=filters, repeat=repeat, kernel=[kernel], stride=[stride], dilation=[dilation], dropout=dropout, residual=residual, separable=separable)


def matchboxnet_3x1x64() -> List[Dict[str, Any]]:
    """Prologue, three residual separable blocks (kernels 13 / 15 / 17, 64 channels), two epilogue blocks (dilated 29, then point-wise)."""
    return [_block(128, 1, 11), _block(64, 1, 13, residual=True, separable=True), _block(64, 1, 15, residual=True, separable=True),
            _block(64, 1, 17, residual=True, separable=True), _block(128, 1, 29, dilation=2, separable=True), _block(128, 1, 1)]


def matchboxnet_3x1x64_vad() -> List[Dict[str, Any]]:
    return matchboxnet_3x1x64()


@dataclass
class MatchboxNetModelConfig(EncDecClassificationConfig):
    sample_rate: int = 16000
    repeat: int = 1
    dropout: float = 0.0
    separable: bool = True
    kernel_size_factor: float = 1.0
    timesteps: int = 128
    labels: Any = S.MISSING
    preprocessor: Any = field(default_factory=lambda: M.AudioToMFCCPreprocessorConfig(window_size=0.025))
    spec_augment: Optional[M.SpectrogramAugmentationConfig] = field(
        default_factory=lambda: M.SpectrogramAugmentationConfig(freq_masks=2, time_masks=2, freq_width=15, time_width=25, rect_masks=5, rect_time=25, rect_freq=15))
    crop_or_pad_augment: Optional[M.CropOrPadSpectrogramAugmentationConfig] = field(default_factory=lambda: M.CropOrPadSpectrogramAugmentationConfig(audio_length=128))
    encoder: Dict[str, Any] = field(default_factory=lambda: {"_target_": "speech_b200.modules.conv_asr.ConvASREncoder", "activation": "relu", "feat_in": 64,
                                                            "jasper": matchboxnet_3x1x64()})
    decoder: Dict[str, Any] = field(default_factory=lambda: {"_target_": "speech_b200.modules.conv_asr.ConvASRDecoderClassification", "feat_in": 128, "num_classes": -1})


@dataclass
class MatchboxNetVADModelConfig(MatchboxNetModelConfig):
    timesteps: int = 64
    labels: Any = field(default_factory=lambda: ["background", "speech"])
    crop_or_pad_augment: Optional[M.CropOrPadSpectrogramAugmentationConfig] = None


class EncDecClassificationModelConfigBuilder(S.ModelConfigBuilder):
    """``name``: ``matchboxnet_3x1x64`` or ``matchboxnet_3x1x64_vad``.  Setters change one field each; ``build()`` propagates them: labels → dataset
    labels and decoder classes, sample rate → front end and datasets, repeat / dropout / separable / kernel scaling → every residual block of the
    encoder, last encoder width → decoder input, time steps → crop-or-pad length."""

    VALID_CONFIGS = ("matchboxnet_3x1x64", "matchboxnet_3x1x64_vad")

    def __init__(self, name: str = "matchboxnet_3x1x64", encoder_cfg_func=None):
        if name not in self.VALID_CONFIGS:
            raise ValueError(f"`name` must be one of {list(self.VALID_CONFIGS)}")
        self.name = name
        cfg = MatchboxNetVADModelConfig() if name.endswith("_vad") else MatchboxNetModelConfig()
        if encoder_cfg_func is not None:
            cfg.encoder["jasper"] = encoder_cfg_func()
        super().__init__(cfg)

    def set_labels(self, labels: List[str]):
        self.model_cfg.labels = list(labels)

    def set_separable(self, separable: bool):
        self.model_cfg.separable = separable

    def set_repeat(self, repeat: int):
        self.model_cfg.repeat = repeat

    def set_sample_rate(self, sample_rate: int):
        self.model_cfg.sample_rate = sample_rate

    def set_dropout(self, dropout: float = 0.0):
        self.model_cfg.dropout = dropout

    def set_timesteps(self, timesteps: int):
        self.model_cfg.timesteps = timesteps

    def set_is_regression_task(self, is_regression_task: bool):
        self.model_cfg.is_regression_task = is_regression_task

    def _finalize_cfg(self):
        c = self.model_cfg
        for ds in (c.train_ds, c.validation_ds, c.test_ds):
            if ds is not None:
                ds.labels, ds.sample_rate = c.labels, c.sample_rate
        c.preprocessor.sample_rate = c.sample_rate
        feat = getattr(c.preprocessor, "n_mfcc", None) or getattr(c.preprocessor, "features", 64)
        c.encoder["feat_in"] = feat
        blocks = c.encoder["jasper"]
        for b in blocks[:-1]:
            b["dropout"] = c.dropout
        for b in blocks[1:-2]:
            b["repeat"] = c.repeat
        for b in blocks[1:-1]:
            b["separable"] = c.separable
        for b in blocks:
            b["kernel_size_factor"] = c.kernel_size_factor
        c.decoder["feat_in"] = blocks[-1]["filters"]
        c.decoder["num_classes"] = len(c.labels) if c.labels != S.MISSING else -1
        if c.crop_or_pad_augment is not None:
            c.crop_or_pad_augment.audio_length = c.timesteps
